"""Each part alone against its plain formula, built through the part registry."""

import types

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
LIMIT = {torch.float32: 5e-6, torch.bfloat16: 2e-2}


def build(group, kind, dtype, prefix="", **params):
    from tinyvllm_b200.config.spec import PartSpec
    from tinyvllm_b200.parts import BuildContext, build_part
    return build_part(group, PartSpec(kind, params), BuildContext(DEV, dtype, prefix, build_part))


def bind_random(part, dtype, seed=0):
    """Random tensors for every declared parameter; returns them by checkpoint name (float32)."""
    from tinyvllm_b200.weights.loader import bind_tensors
    from tinyvllm_b200.weights.random_init import random_tensors
    targets = [(p, spec) for p in part.all_parts() for spec in p.param_specs()]
    tensors = {name: t.to(dtype).float() for name, t in random_tensors(targets, seed)}
    bind_tensors(targets, tensors, dtype=dtype, device=DEV)
    for p in part.all_parts():
        if hasattr(p, "finalize"):
            p.finalize()
    return tensors


def check(got, want, dtype):
    scale = want.abs().max().item() or 1.0
    err = (got.float().cpu() - want).abs().max().item() / scale
    assert err <= LIMIT[dtype], f"error {err:.3e} of scale"


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_norm_part(dtype):
    norm = build("norm", "rms_norm", dtype, prefix="x.norm", width=120, eps=2e-5)
    w = bind_random(norm, dtype)["x.norm.weight"]
    assert norm.weight.dtype == torch.float32            # drawn in 32-bit, a vector stays 32-bit
    torch.manual_seed(0)
    x, res = torch.randn(9, 120).to(dtype), torch.randn(9, 120).to(dtype)
    check(norm.forward(x.to(DEV)), plain.rms_norm(x.float(), w, 2e-5, dtype), dtype)
    y, m = norm.add(x.to(DEV), res.to(DEV))
    want_y, want_m = plain.add_rms_norm(x.float(), res.float(), w, 2e-5, dtype)
    check(y, want_y, dtype), check(m, want_m, dtype)
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    check(norm.add_rows(x.to(DEV), res.to(DEV), rows), want_y[[8, 2]], dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_feed_forward_part(dtype):
    ff = build("feed_forward", "swiglu", dtype, prefix="L.mlp", hidden_size=72, intermediate_size=200)
    w = bind_random(ff, dtype)
    torch.manual_seed(1)
    x = (torch.randn(33, 72) * 4).to(dtype)
    want = plain.mlp_block(w, "L", x.float(), dtype)
    check(ff.forward(x.to(DEV), None), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_embedding_and_head_parts(dtype):
    emb = build("embedding", "token_embedding", dtype, vocab_size=301, width=40, name="emb.weight")
    table = bind_random(emb, dtype)["emb.weight"]
    ids = torch.tensor([0, 300, 7], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).float().cpu(), table[[0, 300, 7]])
    head = build("head", "lm_head", dtype, vocab_size=301, width=40, name="head.weight", tied_to=None)
    w = bind_random(head, dtype, seed=3)["head.weight"]
    torch.manual_seed(2)
    x = torch.randn(5, 40).to(dtype)
    logits = head.forward(x.to(DEV))
    assert logits.dtype == torch.float32
    check(logits, x.float() @ w.T, dtype)
    tied = build("head", "lm_head", dtype, vocab_size=301, width=40, name="head.weight", tied_to="emb.weight")
    assert tied.param_specs() == []


def test_position_part_shares_tables():
    a = build("position", "rope_half_split", torch.float32, head_dim=48, theta=1e4, max_positions=777)
    b = build("position", "rope_half_split", torch.bfloat16, head_dim=48, theta=1e4, max_positions=777)
    a.finalize(), b.finalize()
    assert a.cos.data_ptr() == b.cos.data_ptr() and a.cos.shape == (777, 24)
    want_cos, want_sin = plain.rope_tables(48, 777, 1e4)
    assert (a.cos.cpu() - want_cos).abs().max() < 5e-7 and (a.sin.cpu() - want_sin).abs().max() < 5e-7


class OnePartModel:
    """The least a StepRunner needs to know of a model, around one mixer."""

    def __init__(self, mixer, dtype, max_positions=4096):
        self.mixer, self.device, self.dtype = mixer, DEV, dtype
        self.spec = types.SimpleNamespace(max_positions=max_positions, vocab_size=10)

    def cache_needs(self):
        return [self.mixer.cache_need()]

    def cache_sources(self):
        return [None]


def run_mixer_in_portions(runner, mixer, x, cuts, rid="r"):
    from tinyvllm_b200.engine.step import StepEntry
    runner.open(rid)
    outs, start = [], 0
    with torch.inference_mode():
        for count in cuts:
            entries = [StepEntry(rid, tuple([1] * count), ())]
            plan = runner.plan(entries)
            ctx = runner.build_context(entries, plan)
            outs.append(mixer.forward(x[start:start + count].to(DEV).contiguous(), ctx, 0))
            runner.manager.commit(plan)
            start += count
    runner.close(rid)
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_alone(dtype, window):
    from tinyvllm_b200.config.spec import PartSpec
    from tinyvllm_b200.engine.step import StepRunner
    hidden, nq, nkv, d = 56, 6, 3, 32
    mixer = build("mixer", "gqa_attention", dtype, prefix="L.self_attn", hidden_size=hidden,
                  num_heads=nq, num_kv_heads=nkv, head_dim=d, scale=0.21, qk_norm_eps=1e-5,
                  window=window,
                  position=PartSpec("rope_half_split", {"head_dim": d, "theta": 5e4, "max_positions": 4096}))
    w = bind_random(mixer, dtype)
    runner = StepRunner(OnePartModel(mixer, dtype), page_size=8, num_pages=64, max_requests=2)
    torch.manual_seed(3)
    x = torch.randn(300, hidden).to(dtype)
    got = run_mixer_in_portions(runner, mixer, x, [150, 2, 100, 1, 1, 46])
    cfg = {"nq": nq, "nkv": nkv, "d": d, "eps": 1e-5}
    cos, sin = plain.rope_tables(d, 300, 5e4)
    # the plain block fixes scale = d^-1/2; here the scale is a parameter, so restate with it
    t = x.shape[0]
    q = plain.linear(x.float(), w["L.self_attn.q_proj.weight"], dtype).view(t, nq, d)
    kk = plain.linear(x.float(), w["L.self_attn.k_proj.weight"], dtype).view(t, nkv, d)
    v = plain.linear(x.float(), w["L.self_attn.v_proj.weight"], dtype).view(t, nkv, d)
    q, kk = plain.qk_norm_rope(q, kk, w["L.self_attn.q_norm.weight"], w["L.self_attn.k_norm.weight"],
                               cos, sin, cfg["eps"], dtype)
    a = plain.causal_attention(q, kk, v, 0.21, window, dtype)
    want = plain.linear(a.reshape(t, nq * d), w["L.self_attn.o_proj.weight"], dtype)
    check(got, want, dtype)
    for pool in runner.manager.pools:
        assert pool.free_count == pool.num_pages


def test_attention_part_refuses_head_sizes_the_kernels_do_not_take():
    with pytest.raises(ValueError, match="steps of 16"):
        build("mixer", "gqa_attention", torch.float32, hidden_size=8, num_heads=2, num_kv_heads=1,
              head_dim=24, scale=1.0, qk_norm_eps=None, window=None)
    with pytest.raises(KeyError, match="no mixer part named 'nope'"):
        build("mixer", "nope", torch.float32)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_block_part_alone(dtype):
    """The arrangement of a layer (norm, mixer, norm, feed-forward, deferred residual sums) alone,
    as the first layer (no stream yet) and as a later one, in portions, against the plain parts."""
    from tinyvllm_b200.config.spec import PartSpec
    from tinyvllm_b200.engine.step import StepEntry, StepRunner
    from tinyvllm_b200.parts import BuildContext, build_part
    hidden, inter, nq, nkv, d, eps = 72, 104, 4, 2, 32, 3e-6
    spec = PartSpec("prenorm_residual", {
        "mixer_norm_name": "input_layernorm", "feed_forward_norm_name": "post_attention_layernorm",
        "mixer_name": "self_attn", "feed_forward_name": "mlp"})
    block = build_part(
        "block", spec, BuildContext(DEV, dtype, "L", build_part),
        mixer=PartSpec("gqa_attention", {
            "hidden_size": hidden, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "scale": d ** -0.5,
            "qk_norm_eps": eps, "window": None,
            "position": PartSpec("rope_half_split", {"head_dim": d, "theta": 1e4, "max_positions": 1024})}),
        feed_forward=PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}),
        norm=PartSpec("rms_norm", {"width": hidden, "eps": eps}))
    w = bind_random(block, dtype, seed=3)
    runner = StepRunner(OnePartModel(block.mixer, dtype, max_positions=1024), page_size=8, num_pages=64,
                        max_requests=2)
    torch.manual_seed(5)
    tokens = 140
    x = torch.randn(tokens, hidden).to(dtype)
    stream = torch.randn(tokens, hidden).to(dtype)
    cfg = {"nq": nq, "nkv": nkv, "d": d, "eps": eps}
    cos, sin = plain.rope_tables(d, tokens, 1e4)
    for first_layer in (True, False):
        if first_layer:
            want_stream = x.float()
            normed = plain.rms_norm(x.float(), w["L.input_layernorm.weight"], eps, dtype)
        else:
            normed, want_stream = plain.add_rms_norm(x.float(), stream.float(), w["L.input_layernorm.weight"],
                                                     eps, dtype)
        attended, _ = plain.attention_block(cfg, w, "L", normed, cos, sin, None, dtype)
        normed, want_stream = plain.add_rms_norm(attended, want_stream, w["L.post_attention_layernorm.weight"],
                                                 eps, dtype)
        want = plain.mlp_block(w, "L", normed, dtype)
        rid = f"r{first_layer}"
        runner.open(rid)
        outs, streams, sums, start = [], [], [], 0
        with torch.inference_mode():
            for count in (100, 2, 37, 1):
                entries = [StepEntry(rid, tuple([1] * count), ())]
                plan = runner.plan(entries)
                ctx = runner.build_context(entries, plan)
                part = slice(start, start + count)
                out, new_stream = block.forward(
                    x[part].to(DEV).contiguous(), None if first_layer else stream[part].to(DEV).contiguous(),
                    ctx, 0)
                if out is None:
                    # few bfloat16 rows: the down projection added its output to the stream itself
                    assert dtype == torch.bfloat16 and count <= 16
                    sums.append((part, new_stream))
                else:
                    outs.append((part, out)), streams.append((part, new_stream))
                runner.manager.commit(plan)
                start += count
        runner.close(rid)
        for part, out in outs:
            check(out, want[part], dtype)
        for part, new_stream in streams:
            check(new_stream, want_stream[part], dtype)
        for part, summed in sums:
            check(summed, (want.float() + want_stream.float()).to(dtype).float()[part], dtype)
        assert sums or dtype != torch.bfloat16
