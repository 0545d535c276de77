"""Each kernel alone against its plain reference, at sizes other than the engine's."""

import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def k():
    from tinyvllm_b200.ops import kernels
    return kernels


def close(got, want, dtype, *, f32=2e-6, bf16=1e-2):
    """|got - want| within a fraction of the largest |want| (float32: rounding of a few sums)."""
    scale = want.abs().max().item() or 1.0
    limit = f32 if dtype == torch.float32 else bf16
    err = (got.float().cpu() - want).abs().max().item() / scale
    assert err <= limit, f"error {err:.3e} of scale, allowed {limit:.1e}"


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_embed_rows(dtype):
    torch.manual_seed(0)
    table = torch.randn(1003, 200).to(dtype)
    ids = torch.tensor([0, 1002, 5, 5, 77], dtype=torch.int32)
    out = k().embed_rows(table.to(DEV), ids.to(DEV))
    assert torch.equal(out.cpu(), table[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("width", [48, 1000, 5120, 12000])
def test_rms_norm_and_residual(dtype, width):
    torch.manual_seed(width)
    x = (torch.randn(37, width) * 3).to(dtype)
    res = torch.randn(37, width).to(dtype)
    w = (1 + 0.1 * torch.randn(width)).to(dtype)
    got = k().rms_norm(x.to(DEV), w.to(DEV), 1e-5)
    close(got, plain.rms_norm(x.float(), w.float(), 1e-5, dtype), dtype, bf16=8e-3)
    got, new_res = k().rms_norm(x.to(DEV), w.to(DEV), 1e-5, residual=res.to(DEV))
    want, want_res = plain.add_rms_norm(x.float(), res.float(), w.float(), 1e-5, dtype)
    assert torch.equal(new_res.float().cpu(), want_res)            # the rounded sum is exact
    close(got, want, dtype, bf16=8e-3)
    rows = torch.tensor([36, 0, 5], dtype=torch.int32)
    picked = k().rms_norm(x.to(DEV), w.to(DEV), 1e-5, residual=res.to(DEV), rows=rows.to(DEV))
    assert torch.equal(picked.cpu(), got.cpu()[rows.long()])
    if dtype == torch.bfloat16:                                    # a 32-bit weight stays 32-bit
        got32 = k().rms_norm(x.to(DEV), w.float().to(DEV), 1e-5)
        close(got32, plain.rms_norm(x.float(), w.float(), 1e-5, dtype), dtype, bf16=8e-3)


def test_rms_norm_refuses_a_row_larger_than_shared_memory():
    from tinyvllm_b200.ops.kernels import KernelError
    x = torch.zeros(1, 60000, device=DEV)
    with pytest.raises(KernelError, match="larger"):
        k().rms_norm(x, torch.ones(60000, device=DEV), 1e-6)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_silu_mul(dtype):
    torch.manual_seed(1)
    gate_up = (torch.randn(19, 2 * 333) * 4).to(dtype)
    got = k().silu_mul(gate_up.to(DEV))
    close(got, plain.swiglu(gate_up.float(), dtype), dtype, f32=1e-6, bf16=8e-3)


def test_rope_tables_match_the_float32_formula():
    rope_d, theta = 64, 1_000_000.0
    inv_freq = 1.0 / (theta ** (torch.arange(0, rope_d, 2, dtype=torch.float32) / rope_d))
    cos, sin = k().rope_tables(inv_freq.to(DEV), 5000)
    want_cos, want_sin = plain.rope_tables(rope_d, 5000, theta)
    assert (cos.cpu() - want_cos).abs().max().item() < 5e-7
    assert (sin.cpu() - want_sin).abs().max().item() < 5e-7


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("heads", [(8, 2, 64), (3, 3, 80), (16, 8, 128), (2, 1, 256), (5, 5, 16), (40, 8, 32),
                                   (36, 4, 128), (36, 4, 128, 500), (36, 4, 128, 1300)])
def test_qk_norm_rope_store(dtype, heads):
    # 23 tokens: every batch of a token's heads has a CTA of its own; 500: two CTAs share three
    # batches; 1,300: one CTA goes round all of them
    nq, nkv, d = heads[:3]
    torch.manual_seed(d)
    tokens = heads[3] if len(heads) > 3 else 23
    page = 8
    pages = tokens // page + 7
    qkv = torch.randn(tokens, (nq + 2 * nkv) * d).to(dtype)
    qw, kw = (1 + 0.1 * torch.randn(d)).to(dtype), (1 + 0.1 * torch.randn(d)).to(dtype)
    positions = torch.randint(0, 3000, (tokens,), dtype=torch.int32)
    slots = torch.randperm(page * pages)[:tokens].to(torch.int32)
    cos, sin = plain.rope_tables(d, 3000, 10_000.0)
    kc = torch.zeros(pages, nkv, page, d, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    work = qkv.to(DEV).clone()
    k().qk_norm_rope_store(work, num_q=nq, num_kv=nkv, head_dim=d, positions=positions.to(DEV),
                           q_weight=qw.to(DEV), k_weight=kw.to(DEV), eps=1e-6, cos=cos.to(DEV),
                           sin=sin.to(DEV), slots=slots.to(DEV), key_cache=kc, value_cache=vc)
    q = qkv[:, :nq * d].float().view(tokens, nq, d)
    kk = qkv[:, nq * d:(nq + nkv) * d].float().view(tokens, nkv, d)
    vv = qkv[:, (nq + nkv) * d:].view(tokens, nkv, d)
    pos = positions.long()
    want_q, want_k = plain.qk_norm_rope(q, kk, qw.float(), kw.float(), cos[pos], sin[pos], 1e-6, dtype)
    close(work[:, :nq * d].view(tokens, nq, d), want_q, dtype, bf16=1.6e-2)
    flat_k = by_slot(kc)[slots.long().to(DEV)]
    close(flat_k, want_k, dtype, bf16=1.6e-2)
    assert torch.equal(by_slot(vc)[slots.long().to(DEV)].cpu(), vv)
    untouched = torch.ones(page * pages, dtype=torch.bool)
    untouched[slots.long()] = False
    assert by_slot(kc)[untouched.to(DEV)].abs().sum().item() == 0   # no stray writes
    # without slots nothing is written, q still is
    kc.zero_()
    k().qk_norm_rope_store(qkv.to(DEV).clone(), num_q=nq, num_kv=nkv, head_dim=d,
                           positions=positions.to(DEV), q_weight=qw.to(DEV), k_weight=kw.to(DEV),
                           eps=1e-6, cos=cos.to(DEV), sin=sin.to(DEV), slots=None, key_cache=kc,
                           value_cache=vc)
    assert kc.abs().sum().item() == 0


def by_slot(cache):
    """[pages, kv_heads, page, head_dim] seen as [pages * page, kv_heads, head_dim] (slot = page * size + offset)."""
    pages, nkv, page, d = cache.shape
    return cache.permute(0, 2, 1, 3).reshape(pages * page, nkv, d)


def paged_case(dtype, *, nq, nkv, d, page, lengths, queries, seed, boost=None, layout="shuffled"):
    """Requests with ``lengths`` keys each scattered over shuffled pages; the last ``queries[i]``
    positions of request i are query tokens.  ``boost`` = (request, key position, factor) scales one
    key so that its score stands out.  ``layout`` "rising": every request's pages are neighbours
    in rising order; "mixed": rising stretches of 1 to 9 pages in shuffled order, every third one
    falling."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-n // page) for n in lengths) + 3
    if layout == "shuffled":
        order = torch.randperm(total_pages, generator=g).tolist()
    elif layout == "rising":
        order = list(range(total_pages))[::-1]                     # pages are popped from the end
    else:
        stretches, at = [], 0
        while at < total_pages:
            n = int(torch.randint(1, 10, (1,), generator=g))
            stretch = list(range(at, min(total_pages, at + n)))
            stretches.append(stretch[::-1] if len(stretches) % 3 == 2 else stretch)
            at += n
        order = [page_id for i in torch.randperm(len(stretches), generator=g).tolist() for page_id in stretches[i]][::-1]
    kc = torch.zeros(total_pages, nkv, page, d)
    vc = torch.zeros_like(kc)
    kc.fill_(float("nan")), vc.fill_(float("nan"))              # reading a foreign slot shows
    blocks = max(-(-n // page) for n in lengths)
    tables = torch.full((len(lengths), blocks), -1, dtype=torch.int32)
    keys, values, q_rows, token_row, positions = [], [], [], [], []
    for r, n in enumerate(lengths):
        kr, vr = torch.randn(n, nkv, d, generator=g), torch.randn(n, nkv, d, generator=g)
        if boost and boost[0] == r:
            kr[boost[1]] *= boost[2]
        kr, vr = kr.to(dtype).float(), vr.to(dtype).float()
        keys.append(kr), values.append(vr)
        for b in range(-(-n // page)):
            tables[r, b] = order.pop()
            span = slice(b * page, min(n, (b + 1) * page))
            kc[tables[r, b], :, : span.stop - span.start] = kr[span].transpose(0, 1)
            vc[tables[r, b], :, : span.stop - span.start] = vr[span].transpose(0, 1)
        for p in range(n - queries[r], n):
            q_rows.append(torch.randn(nq, d, generator=g))
            token_row.append(r), positions.append(p)
    q = torch.stack(q_rows).to(dtype)
    return dict(q=q, kc=kc.to(dtype), vc=vc.to(dtype), tables=tables, keys=keys, values=values,
                token_row=torch.tensor(token_row, dtype=torch.int32),
                positions=torch.tensor(positions, dtype=torch.int32))


def plain_paged(case, scale, window, dtype):
    out = []
    for i in range(case["q"].shape[0]):
        r, p = int(case["token_row"][i]), int(case["positions"][i])
        out.append(plain.causal_attention(
            case["q"][i:i + 1].float(), case["keys"][r][:p + 1], case["values"][r][:p + 1], scale,
            window, dtype, q_positions=torch.tensor([p]))[0])
    return torch.stack(out)


def run_rows(case, *, nq, nkv, d, scale, window, max_chunks):
    kernels = k()
    q = case["q"].to(DEV).view(case["q"].shape[0], nq * d)
    scratch = None
    if max_chunks:
        scratch = torch.empty(kernels.attention_rows_scratch_floats(q.shape[0], nq, d, max_chunks),
                              dtype=torch.float32, device=DEV)
    return kernels.attention_rows(
        q, nq * d, case["kc"].to(DEV), case["vc"].to(DEV), case["tables"].to(DEV),
        case["token_row"].to(DEV), case["positions"].to(DEV), num_q=nq, num_kv=nkv, head_dim=d,
        window=window, scale=scale, scratch=scratch, max_chunks=max_chunks).view(-1, nq, d)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(8, 2, 64, 16), (6, 6, 48, 5), (16, 8, 128, 16), (4, 1, 256, 32)])
def test_attention_rows_prompt_portions_and_single_tokens(dtype, shape):
    nq, nkv, d, page = shape
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[300, 1, 70, 515],
                      queries=[40, 1, 1, 3], seed=d)
    scale = d ** -0.5
    want = plain_paged(case, scale, None, dtype)
    walked = run_rows(case, nq=nq, nkv=nkv, d=d, scale=scale, window=None, max_chunks=0)
    close(walked, want, dtype, f32=3e-6, bf16=8e-3)
    spread = run_rows(case, nq=nq, nkv=nkv, d=d, scale=scale, window=None, max_chunks=3)
    assert torch.equal(walked, spread)          # both modes do a row's arithmetic in the same order


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_attention_finds_a_far_key_among_hundreds(dtype):
    """One key, 700 positions back and across two chunk edges, is scaled to dominate."""
    nq, nkv, d, page = 4, 2, 64, 16
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[900], queries=[1], seed=3)
    far = 190
    case["q"][0] = (case["keys"][0][far].repeat_interleave(2, dim=0) * 4).to(dtype)   # q = 4 k_far per head
    want = plain_paged(case, 1.0, None, dtype)
    assert (want[0] - case["values"][0][far].repeat_interleave(2, dim=0)).abs().max() < 1e-2
    for chunks in (0, 4):
        got = run_rows(case, nq=nq, nkv=nkv, d=d, scale=1.0, window=None, max_chunks=chunks)
        close(got, want, dtype, f32=3e-6, bf16=8e-3)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("window", [1, 37, 256, 300])
def test_attention_window_edge(dtype, window):
    """The key just outside the window is made enormous: it must not be seen; the one just inside must."""
    nq, nkv, d, page = 2, 1, 32, 8
    length = 600
    outside = length - 1 - window
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[length], queries=[5], seed=window,
                      boost=(0, outside, 50.0) if outside >= 0 else None)
    want = plain_paged(case, 0.2, window, dtype)
    for chunks in (0, 3):
        got = run_rows(case, nq=nq, nkv=nkv, d=d, scale=0.2, window=window, max_chunks=chunks)
        close(got, want, dtype, f32=3e-6, bf16=8e-3)
    full = plain_paged(case, 0.2, None, dtype)
    assert (full[-1] - want[-1]).abs().max() > 1e-3       # the boosted key would have changed the result


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_attention_rows_with_too_few_chunks_stays_inside_its_scratch(dtype):
    """``max_chunks`` one too small for the longest context: the rows it cannot hold come out as
    NaN, the others are right, and nothing beyond tokens * heads * max_chunks * (head + 2) floats of
    the scratch is written.  The buffer handed over is several times larger than needed and filled
    with a sentinel, so every access of the kernels stays inside allocated memory either way."""
    kernels = k()
    nq, nkv, d, page = 4, 2, 32, 8
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[700, 100], queries=[2, 2], seed=9)
    scale = d ** -0.5
    want = plain_paged(case, scale, None, dtype)
    needed = 3                                        # positions up to 699: chunks 0, 1, 2
    q = case["q"].to(DEV).view(case["q"].shape[0], nq * d)
    for max_chunks in (needed, needed - 1):
        stated = kernels.attention_rows_scratch_floats(q.shape[0], nq, d, max_chunks)
        scratch = torch.full((8 * stated,), 12345.0, dtype=torch.float32, device=DEV)
        got = kernels.attention_rows(
            q, nq * d, case["kc"].to(DEV), case["vc"].to(DEV), case["tables"].to(DEV),
            case["token_row"].to(DEV), case["positions"].to(DEV), num_q=nq, num_kv=nkv, head_dim=d,
            window=None, scale=scale, scratch=scratch, max_chunks=max_chunks).view(-1, nq, d)
        torch.cuda.synchronize()
        assert (scratch[stated:] == 12345.0).all()                   # nothing written past the stated size
        if max_chunks == needed:
            close(got, want, dtype, f32=3e-6, bf16=8e-3)
        else:
            assert torch.isnan(got[:2].float()).all()                # the rows at positions 698, 699
            close(got[2:], want[2:], dtype, f32=3e-6, bf16=8e-3)     # the short request is untouched by it


def test_attention_padding_rows_give_zeros():
    case = paged_case(torch.float32, nq=2, nkv=1, d=16, page=4, lengths=[9], queries=[2], seed=0)
    case["token_row"][1] = -1
    case["positions"][1] = -1
    for chunks in (0, 2):
        got = run_rows(case, nq=2, nkv=1, d=16, scale=1.0, window=None, max_chunks=chunks)
        assert got[1].abs().sum().item() == 0 and torch.isfinite(got[0]).all()


def test_attention_refuses_sizes_it_does_not_take():
    from tinyvllm_b200.ops.kernels import KernelError
    def call(nq, nkv, d):
        ints = torch.zeros(1, dtype=torch.int32, device=DEV)
        cache = torch.zeros(1, nkv, 4, d, device=DEV)
        return k().attention_rows(torch.zeros(1, nq * d, device=DEV), nq * d, cache, cache,
                                  ints.view(1, 1), ints, ints, num_q=nq, num_kv=nkv, head_dim=d,
                                  window=None, scale=1.0)

    with pytest.raises(KernelError, match="head sizes"):
        call(2, 1, 272)
    with pytest.raises(KernelError, match="groups"):
        call(3, 2, 16)
    assert call(2, 1, 16).shape == (1, 32)


@pytest.mark.parametrize("shape", [(1, 7, 5), (70, 129, 33), (300, 200, 1000), (5, 1030, 64)])
def test_gemm_float32_any_size_and_row_independence(shape):
    m, n, kk = shape
    torch.manual_seed(m)
    a, w = torch.randn(m, kk), torch.randn(n, kk)
    got = k().gemm_nt_simt(a.to(DEV), w.to(DEV))
    want = (a.double() @ w.double().T).float()
    assert (got.cpu() - want).abs().max().item() <= 2e-6 * want.abs().max().item() * math.sqrt(kk)
    alone = k().gemm_nt_simt(a[:1].to(DEV), w.to(DEV))
    assert torch.equal(alone[0], got[0])                   # a row's sum does not depend on the batch
    strided = torch.randn(m, kk + 8)
    got2 = k().gemm_nt_simt(strided.to(DEV)[:, :kk], w.to(DEV))
    assert torch.allclose(got2.cpu(), strided[:, :kk] @ w.T, atol=1e-3, rtol=1e-4)


def test_gemm_bfloat16_inputs_float32_result():
    torch.manual_seed(0)
    a, w = torch.randn(9, 100).bfloat16(), torch.randn(333, 100).bfloat16()
    got = k().gemm_nt_simt(a.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert got.dtype == torch.float32
    assert torch.allclose(got.cpu(), a.float() @ w.float().T, atol=1e-4, rtol=1e-5)


def pack(rows):
    from tinyvllm_b200.sampling.params import SamplingParams
    from tinyvllm_b200.sampling.sampler import pack_rows
    params = [SamplingParams(temperature=t, top_k=tk, top_p=tp, seed=s) for t, tk, tp, s, _ in rows]
    return torch.from_numpy(pack_rows(params, [d for *_, d in rows])).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_sampling_matches_the_plain_rules(dtype):
    torch.manual_seed(5)
    # bfloat16 logits are made distinct (multiples of 1/32 below 8): with equal values at the
    # top-p boundary the kernel keeps all of them, the plain rule only the first ones
    vocab = 1531 if dtype == torch.float32 else 500
    rows = [(0.0, 0, 1.0, 0, 0), (1.0, 0, 1.0, 1, 0), (0.7, 40, 1.0, 2, 3), (1.3, 0, 0.8, 3, 9),
            (0.9, 25, 0.5, 2**40 + 7, 2**33 + 1), (1.0, 1, 1.0, 5, 5), (1.0, 0, 1e-4, 6, 1),
            (2.5, 5000, 0.95, 7, 2)]
    if dtype == torch.float32:
        logits = torch.randn(len(rows), vocab) * 2.5
    else:
        logits = torch.stack([(torch.randperm(vocab) - 250) / 32.0 for _ in rows]).to(dtype)
        assert all(len(set(row.tolist())) == vocab for row in logits)
    got = k().sample_rows(logits.to(DEV), pack(rows)).cpu().tolist()
    want = [plain.sample(logits[i].float(), *rows[i]) for i in range(len(rows))]
    assert got == want
    # a request's token does not depend on its row or its neighbours
    again = k().sample_rows(logits.flip(0).contiguous().to(DEV), pack(rows[::-1])).cpu().tolist()
    assert again == want[::-1]


def test_sampling_distribution_and_ties():
    logits = torch.tensor([[0.1, 3.0, 2.9, -1.0, 2.95, 0.0, 3.0]]).repeat(4000, 1)
    rows = [(0.7, 0, 1.0, seed, 1) for seed in range(4000)]
    got = k().sample_rows(logits.to(DEV), pack(rows)).cpu()
    freq = torch.bincount(got.long(), minlength=7).float() / 4000
    assert (freq - torch.softmax(logits[0] / 0.7, 0)).abs().max().item() < 0.03
    greedy = k().sample_rows(logits[:1].to(DEV), pack([(0.0, 0, 1.0, 0, 0)])).item()
    assert greedy == 1                                         # of equal logits the smaller id wins
    tied = torch.zeros(1, 50)
    top2 = {k().sample_rows(tied.to(DEV), pack([(1.0, 2, 1.0, seed, 0)])).item() for seed in range(40)}
    assert top2 == {0, 1}                                      # top-k among ties keeps the smaller ids


# ------------------------------------------------------------ tiled bfloat16 kernels
def prefill_tile_lists(case):
    """Tiles of up to 64 consecutive query tokens per request, from the flat case."""
    rows, firsts, counts = [], [], []
    token_row = case["token_row"].tolist()
    start = 0
    while start < len(token_row):
        end = start
        while end < len(token_row) and token_row[end] == token_row[start]:
            end += 1
        for first in range(start, end, 64):
            rows.append(token_row[start]), firsts.append(first), counts.append(min(64, end - first))
        start = end
    as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return as_int(rows), as_int(firsts), as_int(counts)


@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("shape", [(8, 2, 64, 16), (4, 4, 128, 16), (16, 8, 128, 5), (2, 1, 64, 64)])
def test_attention_prefill_tiles(shape, window):
    nq, nkv, d, page = shape
    dtype = torch.bfloat16
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[300, 1, 70, 515, 64],
                      queries=[130, 1, 70, 3, 64], seed=d + nq)
    scale = d ** -0.5
    want = plain_paged(case, scale, window, dtype)
    tile_row, tile_first, tile_count = prefill_tile_lists(case)
    q = case["q"].to(DEV).view(-1, nq * d)
    got = k().attention_prefill(q, nq * d, case["kc"].to(DEV), case["vc"].to(DEV), case["tables"].to(DEV),
                                case["positions"].to(DEV), tile_row, tile_first, tile_count, num_q=nq,
                                num_kv=nkv, head_dim=d, window=window, scale=scale).view(-1, nq, d)
    close(got, want, dtype, bf16=1.2e-2)


def test_attention_prefill_window_edge_and_far_key():
    nq, nkv, d, page, dtype = 2, 1, 64, 16, torch.bfloat16
    for window in (64, 65, 200):
        length = 700
        outside = length - 1 - window
        case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[length], queries=[90],
                          seed=window, boost=(0, outside, 30.0))
        want = plain_paged(case, 0.2, window, dtype)
        tiles = prefill_tile_lists(case)
        got = k().attention_prefill(case["q"].to(DEV).view(-1, nq * d), nq * d, case["kc"].to(DEV),
                                    case["vc"].to(DEV), case["tables"].to(DEV), case["positions"].to(DEV),
                                    *tiles, num_q=nq, num_kv=nkv, head_dim=d, window=window,
                                    scale=0.2).view(-1, nq, d)
        close(got, want, dtype, bf16=1.2e-2)


def finite_cache(case, dtype):
    """The case's caches with the unused slots at a large finite value instead of NaN: the tcgen05
    kernel copies whole pages and multiplies what lies past a request's end by zero."""
    fill = lambda c: torch.nan_to_num(c.float(), nan=3.0e4).to(dtype).to(DEV)
    return fill(case["kc"]), fill(case["vc"])


def run_prefill_tc(case, *, nq, nkv, d, window, scale):
    from tinyvllm_b200.ops.attention import prefill_tiles
    counts, starts, previous = [], [], None
    for row, position in zip(case["token_row"].tolist(), case["positions"].tolist()):
        if row != previous:
            counts.append(0), starts.append(position)
            previous = row
        counts[-1] += 1
    big, rest, _ = prefill_tiles(counts, starts, tensor_memory=True)
    as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    kc, vc = finite_cache(case, torch.bfloat16)
    q = case["q"].to(DEV).view(-1, nq * d)
    args = (q, nq * d, kc, vc, case["tables"].to(DEV), case["positions"].to(DEV))
    heads = dict(num_q=nq, num_kv=nkv, head_dim=d, window=window, scale=scale)
    out = torch.full((q.shape[0], nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    if big[0]:
        k().attention_prefill_tc(*args, *map(as_int, big), **heads, out=out)
    if rest[0]:
        k().attention_prefill(*args, *map(as_int, rest), **heads, out=out)
    assert k().attention_prefill_tc_status() == 0
    return out.view(-1, nq, d), big, rest


@pytest.mark.parametrize("window", [None, 70, 129])
@pytest.mark.parametrize("shape", [(1, 1, 16), (4, 2, 16), (16, 8, 8), (6, 2, 32), (2, 1, 128)])
def test_attention_prefill_tc(shape, window):
    """The tcgen05 tile kernel alone (with the 64-row kernel for the short rests of entries):
    portions that start anywhere, tiles cut by the end of an entry, shuffled pages."""
    nq, nkv, page = shape
    d, dtype = 128, torch.bfloat16
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[300, 1, 70, 515, 64, 1000],
                      queries=[130, 1, 70, 3, 64, 777], seed=nq + page)
    want = plain_paged(case, d ** -0.5, window, dtype)
    got, big, rest = run_prefill_tc(case, nq=nq, nkv=nkv, d=d, window=window, scale=d ** -0.5)
    assert big[0] and rest[0]                      # both kernels had tiles
    assert sum(big[2]) + sum(rest[2]) == case["q"].shape[0]
    close(got, want, dtype, bf16=1.2e-2)


@pytest.mark.parametrize("layout", ["rising", "mixed"])
@pytest.mark.parametrize("shape", [(4, 2, 8), (4, 2, 16), (16, 8, 16), (2, 1, 32)])
def test_attention_prefill_tc_pages_that_lie_together(shape, layout):
    """Pages of fewer than 32 tokens are copied two or four at a time where the block table names
    neighbours in rising order: whole requests of such pages, and stretches of 1 to 9 pages, rising
    and falling, that start anywhere in a block of keys (a foreign page read shows as NaN)."""
    nq, nkv, page = shape
    d, dtype = 128, torch.bfloat16
    for window in (None, 200):
        case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[300, 1, 70, 515, 64, 1000],
                          queries=[130, 1, 70, 3, 64, 777], seed=nq + page, layout=layout)
        if layout == "rising":
            first = case["tables"][5, :1000 // page]
            assert torch.equal(first, first[0] + torch.arange(first.numel(), dtype=torch.int32))
        want = plain_paged(case, d ** -0.5, window, dtype)
        got, big, rest = run_prefill_tc(case, nq=nq, nkv=nkv, d=d, window=window, scale=d ** -0.5)
        assert big[0]
        close(got, want, dtype, bf16=1.2e-2)
    # two q heads an item
    case = paged_case(dtype, nq=16, nkv=8, d=d, page=16, lengths=[3700, 130, 600], queries=[3700, 130, 300],
                      seed=5, layout=layout)
    want = plain_paged(case, d ** -0.5, None, dtype)
    got, big, rest = run_prefill_tc(case, nq=16, nkv=8, d=d, window=None, scale=d ** -0.5)
    close(got, want, dtype, bf16=1.2e-2)


@pytest.mark.parametrize("window", [None, 1000])
def test_attention_prefill_tc_two_heads_an_item(window):
    """Enough tiles that the launcher gives every item two q heads of a kv head (a softmax group
    each, every K and V tile used by both): a long prompt beside shorter ones, groups of 2 and 4."""
    for nq, nkv, lengths, queries in ((16, 8, [3700, 130, 600], [3700, 130, 300]), (16, 4, [3900], [3900])):
        d, dtype = 128, torch.bfloat16
        case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=16, lengths=lengths, queries=queries, seed=nq + nkv)
        want = plain_paged(case, d ** -0.5, window, dtype)
        got, big, rest = run_prefill_tc(case, nq=nq, nkv=nkv, d=d, window=window, scale=d ** -0.5)
        assert len(big[0]) * nq >= 3 * torch.cuda.get_device_properties(0).multi_processor_count    # pairs are used
        close(got, want, dtype, bf16=1.2e-2)


def test_attention_prefill_tc_window_edge_far_key_and_growing_maximum():
    """One key far back scaled up so that its score stands out (it must be found, or be cut off
    exactly at the window's edge), and keys that grow towards the end so that every row's
    reference has to move several times."""
    nq, nkv, d, page, dtype = 2, 1, 128, 16, torch.bfloat16
    for window in (None, 128, 129, 400):
        length = 900
        outside = length - 1 - (window or 500)
        case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[length], queries=[300],
                          seed=window or 1, boost=(0, outside, 12.0))
        want = plain_paged(case, 0.2, window, dtype)
        got, _, _ = run_prefill_tc(case, nq=nq, nkv=nkv, d=d, window=window, scale=0.2)
        close(got, want, dtype, bf16=1.2e-2)
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=[1024], queries=[1024], seed=3)
    ramp = torch.linspace(0.2, 3.0, 1024)
    case["keys"][0] = (case["keys"][0] * ramp[:, None, None]).to(dtype).float()
    for block in range(1024 // page):
        span = slice(block * page, (block + 1) * page)
        case["kc"][case["tables"][0, block]] = case["keys"][0][span].transpose(0, 1).to(dtype)
    want = plain_paged(case, 0.5, None, dtype)
    got, _, _ = run_prefill_tc(case, nq=nq, nkv=nkv, d=d, window=None, scale=0.5)
    close(got, want, dtype, bf16=1.2e-2)


def test_attention_prefill_tc_refuses():
    from tinyvllm_b200.ops.kernels import KernelError
    assert not k().attention_prefill_tc_supports(64, 4, 2, 16)
    assert not k().attention_prefill_tc_supports(128, 4, 2, 5)
    z = lambda *shape: torch.zeros(*shape, dtype=torch.bfloat16, device=DEV)
    i = lambda *v: torch.tensor(v, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="does not take"):
        k().attention_prefill_tc(z(4, 128), 128, z(3, 2, 16, 64), z(3, 2, 16, 64), i(0).view(1, 1), i(0, 1, 2, 3),
                                 i(0), i(0), i(4), num_q=2, num_kv=2, head_dim=64, window=None, scale=1.0)


@pytest.mark.parametrize("window", [None, 150])
@pytest.mark.parametrize("shape", [(4, 2, 64, 16, 8), (8, 2, 128, 16, 4), (2, 2, 128, 7, 1),
                                   (8, 1, 256, 32, 5), (16, 8, 128, 16, 8), (16, 2, 128, 16, 8), (8, 1, 64, 8, 3),
                                   # groups of 5 (40 q heads on 8 kv heads), 3, 6 and 7: fewer heads than the tile
                                   # holds; 12 = two CTAs of 6; 10 at head size 256 = two of 5 would not fit: five of 2
                                   (10, 2, 128, 16, 4), (3, 1, 64, 16, 2), (12, 2, 128, 16, 8), (7, 1, 128, 32, 3),
                                   (24, 2, 64, 16, 2), (10, 1, 256, 16, 2),
                                   # head size 128 walks tiles of 16 keys: pages that hold half a tile, three tiles
                                   (16, 8, 128, 8, 8), (4, 2, 128, 48, 6), (64, 8, 128, 16, 1)])
def test_attention_decode_fused(shape, window):
    """Raw projection in, attention out: against q/k norm + rotation + attention of the plain
    functions, with the new key and value checked in the cache."""
    nq, nkv, d, page, splits = shape
    dtype = torch.bfloat16
    lengths = [1, 2, 63, 64, 65, 300, 511, 1000]
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=lengths, queries=[1] * len(lengths),
                      seed=d + nq)
    requests = len(lengths)
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(requests, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qw, kw = (1 + 0.1 * torch.randn(d, generator=g)), (1 + 0.1 * torch.randn(d, generator=g))
    cos, sin = plain.rope_tables(d, 1200, 10_000.0)
    positions = case["positions"]
    # the slot of the new token is the one the block table gives for its position
    slots = torch.tensor([int(case["tables"][r, int(p) // page]) * page + int(p) % page
                          for r, p in enumerate(positions)], dtype=torch.int32)
    kc, vc = case["kc"].to(DEV).clone(), case["vc"].to(DEV).clone()
    got = k().attention_decode(
        qkv.to(DEV), num_q=nq, num_kv=nkv, head_dim=d, positions=positions.to(DEV),
        token_row=case["token_row"].to(DEV), slots=slots.to(DEV), q_weight=qw.to(DEV), k_weight=kw.to(DEV),
        eps=1e-6, cos=cos.to(DEV), sin=sin.to(DEV), key_cache=kc, value_cache=vc,
        block_tables=case["tables"].to(DEV), window=window, scale=d ** -0.5, splits=splits,
        max_context=1024).view(requests, nq, d)
    q = qkv[:, :nq * d].float().view(requests, nq, d)
    kn = qkv[:, nq * d:(nq + nkv) * d].float().view(requests, nkv, d)
    vn = qkv[:, (nq + nkv) * d:].float().view(requests, nkv, d)
    pos = positions.long()
    want_q, want_k = plain.qk_norm_rope(q, kn, qw, kw, cos[pos], sin[pos], 1e-6, dtype)
    rows = []
    for r, p in enumerate(pos.tolist()):
        keys = torch.cat([case["keys"][r][:p], want_k[r:r + 1]])
        values = torch.cat([case["values"][r][:p], vn[r:r + 1]])
        rows.append(plain.causal_attention(want_q[r:r + 1], keys, values, d ** -0.5, window, dtype,
                                           q_positions=torch.tensor([p]))[0])
    close(got, torch.stack(rows), dtype, bf16=1.2e-2)
    stored_k = by_slot(kc)[slots.long().to(DEV)]
    close(stored_k, want_k, dtype, bf16=1.6e-2)
    assert torch.equal(by_slot(vc)[slots.long().to(DEV)].float().cpu(), vn)
    # the same tokens once more, now that their keys and values are in the cache and with q
    # prepared (the decoded tokens of a step that also holds prompt portions): the same result
    prepared = qkv.clone()
    prepared[:, :nq * d] = want_q.reshape(requests, nq * d).to(dtype)
    prepared[:, nq * d:] = 0                                   # k and v of the projection are not read
    again = k().attention_decode(
        prepared.to(DEV), num_q=nq, num_kv=nkv, head_dim=d, positions=positions.to(DEV),
        token_row=case["token_row"].to(DEV), slots=None, q_weight=None, k_weight=None, eps=0.0, cos=None,
        sin=None, key_cache=kc, value_cache=vc, block_tables=case["tables"].to(DEV), window=window,
        scale=d ** -0.5, splits=splits, max_context=1024, new_in_cache=True).view(requests, nq, d)
    close(again, torch.stack(rows), dtype, bf16=1.2e-2)


@pytest.mark.parametrize("window", [None, 2000])
@pytest.mark.parametrize("plan", [(4, 4), (6, 2), (2, 3)])
def test_attention_decode_request_cut_over_several_clusters(plan, window):
    """A request's keys cut over several clusters per kv head, whose first CTAs leave their pieces
    in global memory for the cluster that arrives last: requests long and short (pieces that hold
    no key), from a length on only, and twice in a row (the counters are left at zero)."""
    pieces, groups = plan
    nq, nkv, d, page, dtype = 4, 2, 128, 16, torch.bfloat16
    lengths = [3000, 37, 700]
    case = paged_case(dtype, nq=nq, nkv=nkv, d=d, page=page, lengths=lengths, queries=[1] * len(lengths), seed=pieces)
    requests = len(lengths)
    assert k().attention_decode_fits_wide(requests * groups, num_q=nq, num_kv=nkv, head_dim=d, page_size=page,
                                          splits=pieces, max_context=3100, weight_dtype=torch.float32)
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(requests, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qw, kw = (1 + 0.1 * torch.randn(d, generator=g)), (1 + 0.1 * torch.randn(d, generator=g))
    cos, sin = plain.rope_tables(d, 3100, 10_000.0)
    positions = case["positions"]
    slots = torch.tensor([int(case["tables"][r, int(p) // page]) * page + int(p) % page
                          for r, p in enumerate(positions)], dtype=torch.int32)
    q = qkv[:, :nq * d].float().view(requests, nq, d)
    kn = qkv[:, nq * d:(nq + nkv) * d].float().view(requests, nkv, d)
    vn = qkv[:, (nq + nkv) * d:].float().view(requests, nkv, d)
    pos = positions.long()
    want_q, want_k = plain.qk_norm_rope(q, kn, qw, kw, cos[pos], sin[pos], 1e-6, dtype)
    rows = []
    for r, p in enumerate(pos.tolist()):
        keys = torch.cat([case["keys"][r][:p], want_k[r:r + 1]])
        values = torch.cat([case["values"][r][:p], vn[r:r + 1]])
        rows.append(plain.causal_attention(want_q[r:r + 1], keys, values, d ** -0.5, window, dtype,
                                           q_positions=torch.tensor([p]))[0])
    want = torch.stack(rows)
    for far_from in (1, 600, 5000):                 # all requests; the two longer ones; none
        for _ in range(2):
            kc, vc = case["kc"].to(DEV).clone(), case["vc"].to(DEV).clone()
            got = k().attention_decode(
                qkv.to(DEV), num_q=nq, num_kv=nkv, head_dim=d, positions=positions.to(DEV),
                token_row=case["token_row"].to(DEV), slots=slots.to(DEV), q_weight=qw.to(DEV), k_weight=kw.to(DEV),
                eps=1e-6, cos=cos.to(DEV), sin=sin.to(DEV), key_cache=kc, value_cache=vc,
                block_tables=case["tables"].to(DEV), window=window, scale=d ** -0.5, splits=pieces,
                max_context=3100, far_groups=groups, far_from=far_from).view(requests, nq, d)
            close(got, want, dtype, bf16=1.2e-2)
            flat_k = by_slot(kc)[slots.long().to(DEV)]
            close(flat_k, want_k, dtype, bf16=1.6e-2)                  # the new key is stored once, by its piece
            assert torch.equal(by_slot(vc)[slots.long().to(DEV)].cpu(), vn.to(dtype))
    from tinyvllm_b200.ops.kernels import KernelError
    with pytest.raises(KernelError):               # more clusters than the GPU holds at once
        k().attention_decode(
            qkv.to(DEV), num_q=nq, num_kv=nkv, head_dim=d, positions=positions.to(DEV),
            token_row=case["token_row"].to(DEV), slots=slots.to(DEV), q_weight=qw.to(DEV), k_weight=kw.to(DEV),
            eps=1e-6, cos=cos.to(DEV), sin=sin.to(DEV), key_cache=case["kc"].to(DEV), value_cache=case["vc"].to(DEV),
            block_tables=case["tables"].to(DEV), window=window, scale=d ** -0.5, splits=8, max_context=3100,
            far_groups=8, far_from=1)


def test_attention_decode_pieces_fitted_to_few_rows():
    """With two or three rows the number of pieces is the largest with which the kernel's form for
    small grids has all its clusters on the GPU at once; one row and four or more keep theirs."""
    import types

    from tinyvllm_b200.ops.attention import decode_splits, fitted_splits
    mixer = types.SimpleNamespace(num_heads=16, num_kv_heads=8, head_dim=128, q_norm_weight=torch.ones(128))
    asked = decode_splits(4096, 2)
    assert asked == 8
    for rows in (1, 2, 3, 4, 8):
        pieces = fitted_splits(decode_splits(4096, rows), rows, mixer, 16, 4096)
        fits = k().attention_decode_fits_wide(rows, num_q=16, num_kv=8, head_dim=128, page_size=16, splits=pieces,
                                              max_context=4096, weight_dtype=torch.float32)
        if rows == 1:
            assert pieces == 8 and fits
        elif rows <= 3:
            assert 4 <= pieces <= 8
            assert fits or pieces == 8                # nothing fitted: the asked number stays
            if pieces < 8:                            # and one piece more would not have fitted
                assert not k().attention_decode_fits_wide(rows, num_q=16, num_kv=8, head_dim=128, page_size=16,
                                                          splits=pieces + 1, max_context=4096,
                                                          weight_dtype=torch.float32)
        else:
            assert pieces == decode_splits(4096, rows)
    # a grid larger than the GPU never fits; a shape the kernel does not take neither
    assert not k().attention_decode_fits_wide(64, num_q=16, num_kv=8, head_dim=128, page_size=16, splits=8,
                                              max_context=4096)
    assert not k().attention_decode_fits_wide(1, num_q=16, num_kv=8, head_dim=80, page_size=16, splits=8,
                                              max_context=4096)


def test_attention_decode_padding_and_unsupported():
    from tinyvllm_b200.ops.kernels import KernelError
    assert k().attention_decode_supports(128, 16, 8, 8)
    assert not k().attention_decode_supports(48, 4, 2, 8)
    assert k().attention_decode_supports(128, 6, 2, 8)           # groups of 3 run on the tile for 4
    assert not k().attention_decode_supports(128, 7, 2, 8)       # no whole number of q heads per kv head
    assert not k().attention_decode_supports(128, 16, 8, 9)
    with pytest.raises(KernelError, match="does not take"):
        k().attention_decode(torch.zeros(1, 4 * 48, dtype=torch.bfloat16, device=DEV), num_q=2, num_kv=1,
                             head_dim=48, positions=None, token_row=None, slots=None, q_weight=None,
                             k_weight=None, eps=0.0, cos=None, sin=None, key_cache=None, value_cache=None,
                             block_tables=None, window=None, scale=1.0, splits=1, max_context=64)


@pytest.mark.parametrize("shape", [(1, 64, 128), (8, 1024, 4096), (8, 3072, 1024), (5, 1000, 136),
                                   (17, 2048, 1024), (32, 520, 72), (3, 8, 16)])
def test_gemm_small_m(shape):
    m, kk, n = shape
    torch.manual_seed(n)
    x, w = torch.randn(m, kk).bfloat16(), (torch.randn(n, kk) * 0.05).bfloat16()
    want = x.float() @ w.float().T
    got = k().gemm_small_m(x.to(DEV), w.to(DEV), 1)
    assert got.dtype == torch.float32
    close(got, want, torch.float32, f32=2e-5)
    got16 = k().gemm_small_m(x.to(DEV), w.to(DEV), 0)
    assert got16.dtype == torch.bfloat16
    close(got16, want, torch.bfloat16, bf16=5e-3)
    alone = k().gemm_small_m(x[:1].to(DEV), w.to(DEV), 1)
    assert torch.equal(alone[0], got[0])                    # a row's sum does not depend on the batch
    if n % 2 == 0:
        gate_up = k().gemm_small_m(x.to(DEV), w.to(DEV), 2)
        assert gate_up.shape == (m, n // 2)
        close(gate_up, plain.swiglu(want, torch.bfloat16), torch.bfloat16, bf16=1e-2)


@pytest.mark.parametrize("tile", [0, 128, 256])
@pytest.mark.parametrize("shape", [(128, 64, 128), (200, 72, 272), (333, 136, 400), (1000, 1032, 784),
                                   (4099, 512, 1024)])
def test_gemm_tc(shape, tile):
    """The tcgen05 product alone: tiles cut by m, n and k edges, both tile widths, several tiles
    per CTA (the last shape has more tiles than SMs), plain and with the activation."""
    m, kk, n = shape
    torch.manual_seed(m + n)
    x, w = (torch.randn(m, kk) * 0.5).bfloat16(), (torch.randn(n, kk) * 0.05).bfloat16()
    # make one row and one column stand out, so that a tile written to the wrong place shows
    x[m // 2] *= 4
    w[n // 3] *= 4
    want = x.float() @ w.float().T
    got = k().gemm_tc(x.to(DEV), w.to(DEV), 0, tile_n=tile)
    assert got.dtype == torch.bfloat16 and got.shape == (m, n)
    assert k().gemm_tc_status() == 0
    close(got, want, torch.bfloat16, bf16=5e-3)
    gate_up = k().gemm_tc(x.to(DEV), w.to(DEV), 2, tile_n=tile)
    assert gate_up.shape == (m, n // 2)
    assert k().gemm_tc_status() == 0
    close(gate_up, plain.swiglu(want, torch.bfloat16), torch.bfloat16, bf16=1e-2)
    # into a view with a row stride of its own, beside columns that must stay as they are
    wide = torch.full((m, n + 16), 7.0, dtype=torch.bfloat16, device=DEV)
    k().gemm_tc(x.to(DEV), w.to(DEV), 0, out=wide[:, 8:n + 8], tile_n=tile)
    assert torch.equal(wide[:, 8:n + 8], got)
    assert bool((wide[:, :8] == 7).all()) and bool((wide[:, n + 8:] == 7).all())


@pytest.mark.parametrize("shape", [(1, 64, 384), (8, 520, 1000), (16, 4096, 4104), (17, 1024, 6144),
                                   (40, 3072, 2048), (64, 8, 256), (100, 776, 3000), (128, 2048, 1280)])
def test_gemm_stream(shape):
    """The weight-streaming tcgen05 product alone: every padded batch size (16, 32, 64, 128), tiles
    cut by n and k edges, tiles shared by several CTAs (their partial sums are added by whoever
    arrives last) and tiles one CTA has to itself; bfloat16 and float32 results, the activation,
    the addition to the residual stream."""
    m, kk, n = shape
    torch.manual_seed(m + n)
    x, w = (torch.randn(m, kk) * 0.5).bfloat16(), (torch.randn(n, kk) * 0.05).bfloat16()
    # make one row and one column stand out, so that a tile written to the wrong place shows
    x[m // 2] *= 4
    w[n // 3] *= 4
    want = x.float() @ w.float().T
    got = k().gemm_stream(x.to(DEV), w.to(DEV), 0)
    assert got.dtype == torch.bfloat16 and got.shape == (m, n)
    assert k().gemm_stream_status() == 0
    close(got, want, torch.bfloat16, bf16=5e-3)
    # the sum does not depend on which CTA came last
    for _ in range(3):
        assert torch.equal(k().gemm_stream(x.to(DEV), w.to(DEV), 0), got)
    logits = k().gemm_stream(x.to(DEV), w.to(DEV), 1)
    assert logits.dtype == torch.float32
    close(logits, want, torch.float32, f32=2e-5)
    assert torch.equal(logits.bfloat16(), got)
    if n % 2 == 0:
        gate_up = k().gemm_stream(x.to(DEV), w.to(DEV), 2)
        assert gate_up.shape == (m, n // 2)
        close(gate_up, plain.swiglu(want, torch.bfloat16), torch.bfloat16, bf16=1e-2)
    stream = torch.randn(m, n).bfloat16()
    summed = k().gemm_stream(x.to(DEV), w.to(DEV), 0, add_stream=stream.to(DEV))
    assert torch.equal(summed.cpu(), (got.cpu().float() + stream.float()).bfloat16())
    # into a view with a row stride of its own, beside columns that must stay as they are
    wide = torch.full((m, n + 16), 7.0, dtype=torch.bfloat16, device=DEV)
    k().gemm_stream(x.to(DEV), w.to(DEV), 0, out=wide[:, 8:n + 8])
    assert torch.equal(wide[:, 8:n + 8], got)
    assert bool((wide[:, :8] == 7).all()) and bool((wide[:, n + 8:] == 7).all())
    assert k().gemm_stream_status() == 0
    # every launch leaves the counters as it found them
    from tinyvllm_b200.ops import kernels
    assert int(kernels._stream_scratch_of(torch.device(DEV))[1].abs().sum()) == 0


def test_gemm_stream_rows_do_not_depend_on_the_batch():
    torch.manual_seed(6)
    x, w = torch.randn(100, 512).bfloat16().to(DEV), (torch.randn(3000, 512) * 0.05).bfloat16().to(DEV)
    whole = k().gemm_stream(x, w, 0)
    for first, count in ((0, 1), (3, 8), (40, 33), (30, 70)):
        assert torch.equal(whole[first:first + count], k().gemm_stream(x[first:first + count], w, 0))
    assert k().gemm_stream_status() == 0


def test_gemm_stream_refuses():
    from tinyvllm_b200.ops.kernels import KernelError
    with pytest.raises(KernelError, match="m <= 128"):
        k().gemm_stream(torch.zeros(129, 64, dtype=torch.bfloat16, device=DEV),
                        torch.zeros(16, 64, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(KernelError, match="multiple of 8"):
        k().gemm_stream(torch.zeros(8, 60, dtype=torch.bfloat16, device=DEV),
                        torch.zeros(16, 60, dtype=torch.bfloat16, device=DEV))


def test_gemm_tc_rows_do_not_depend_on_the_batch():
    torch.manual_seed(5)
    x, w = torch.randn(700, 256).bfloat16().to(DEV), (torch.randn(384, 256) * 0.05).bfloat16().to(DEV)
    whole = k().gemm_tc(x, w, 0)
    part = k().gemm_tc(x[300:500], w, 0)
    assert torch.equal(whole[300:500], part)
    assert k().gemm_tc_status() == 0


def test_gemm_tc_refuses():
    from tinyvllm_b200.ops.kernels import KernelError
    with pytest.raises(KernelError, match="multiples of 8"):
        k().gemm_tc(torch.zeros(128, 60, dtype=torch.bfloat16, device=DEV),
                    torch.zeros(16, 60, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(KernelError, match="multiples of 8"):
        k().gemm_tc(torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV),
                    torch.zeros(12, 64, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(KernelError, match="bfloat16"):
        k().gemm_tc(torch.zeros(128, 64, device=DEV), torch.zeros(16, 64, device=DEV))


def test_gemm_small_m_refuses():
    from tinyvllm_b200.ops.kernels import KernelError
    with pytest.raises(KernelError, match="up to 32 rows"):
        k().gemm_small_m(torch.zeros(33, 64, dtype=torch.bfloat16, device=DEV),
                         torch.zeros(16, 64, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(KernelError, match="multiples of 8"):
        k().gemm_small_m(torch.zeros(2, 60, dtype=torch.bfloat16, device=DEV),
                         torch.zeros(16, 60, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("weight_dtype", [torch.float32, torch.bfloat16], ids=["w32", "w16"])
@pytest.mark.parametrize("shape", [(8, 1024, 512), (1, 256, 48), (19, 1000, 272), (32, 2048, 64)])
def test_gemm_small_m_with_norm_prologue(shape, weight_dtype):
    m, kk, n = shape
    torch.manual_seed(m + n)
    h, res = (torch.randn(m, kk) * 2).bfloat16(), torch.randn(m, kk).bfloat16()
    w = (torch.randn(n, kk) * 0.05).bfloat16()
    nw = (1 + 0.1 * torch.randn(kk)).to(weight_dtype)
    x, stream = plain.add_rms_norm(h.float(), res.float(), nw.float(), 1e-5, torch.bfloat16)
    got, new_stream = k().gemm_small_m(h.to(DEV), w.to(DEV), 1, norm_weight=nw.to(DEV),
                                       residual=res.to(DEV), eps=1e-5)
    assert torch.equal(new_stream.float().cpu(), stream)
    close(got, x @ w.float().T, torch.bfloat16, bf16=6e-3)
    # without a residual: plain norm, no new stream
    got, none = k().gemm_small_m(h.to(DEV), w.to(DEV), 0, norm_weight=nw.to(DEV), eps=1e-5)
    assert none is None
    close(got, plain.rms_norm(h.float(), nw.float(), 1e-5, torch.bfloat16) @ w.float().T,
          torch.bfloat16, bf16=8e-3)
    if n % 2 == 0:
        act, _ = k().gemm_small_m(h.to(DEV), w.to(DEV), 2, norm_weight=nw.to(DEV),
                                  residual=res.to(DEV), eps=1e-5)
        close(act, plain.swiglu(x @ w.float().T, torch.bfloat16), torch.bfloat16, bf16=1.2e-2)


@pytest.mark.parametrize("weight_dtype", [torch.float32, torch.bfloat16], ids=["w32", "w16"])
@pytest.mark.parametrize("shape", [(8, 1024, 512, 3072), (1, 256, 48, 96), (13, 1000, 264, 40), (16, 2048, 1000, 64),
                                   (27, 320, 72, 130), (5, 512, 2048, 96), (9, 128, 5120, 48)])
def test_gemm_small_m_adds_to_the_stream_and_the_next_product_norms_it(shape, weight_dtype):
    """Two products with a pre-norm between them and no norm kernel: the first adds its result to
    the residual stream and stores the rows' sums of squares tile by tile, the second normalises
    the stream with them while loading it."""
    m, k_first, width, n_second = shape
    torch.manual_seed(m + width)
    x = torch.randn(m, k_first).bfloat16()
    w_first = (torch.randn(width, k_first) * 0.05).bfloat16()
    stream = (torch.randn(m, width) * 3).bfloat16()
    if m > 2:
        stream[2] *= 40                        # rows of very different size: a row's own sum must be used
    nw = (1 + 0.1 * torch.randn(width)).to(weight_dtype)
    w_second = (torch.randn(n_second, width) * 0.05).bfloat16()
    product = (x.float() @ w_first.float().T).bfloat16().float()
    want_stream = (product + stream.float()).bfloat16().float()
    summed, squares = k().gemm_small_m(x.to(DEV), w_first.to(DEV), 0, add_stream=stream.to(DEV))
    # the accumulation order of the product differs from torch's: a result may round to the neighbour
    for row in range(m):                       # row by row: the large row must not hide the others
        close(summed[row], want_stream[row], torch.bfloat16, bf16=8e-3)
    tiles, padded = -(-width // 16), -(-m // 8) * 8
    assert squares.shape == (tiles, padded)
    got_squares = squares.sum(0).cpu()
    assert torch.allclose(got_squares[:m], (summed.float().cpu() ** 2).sum(1), rtol=1e-5)
    assert torch.all(got_squares[m:] == 0)
    # the second product takes the stream the first one made, so that the comparison is of the norm alone
    normed = plain.rms_norm(summed.float().cpu(), nw.float(), 1e-5, torch.bfloat16)
    got = k().gemm_small_m(summed, w_second.to(DEV), 0, norm_weight=nw.to(DEV), eps=1e-5, row_squares=squares)
    close(got, normed @ w_second.float().T, torch.bfloat16, bf16=8e-3)
    if n_second % 2 == 0:
        act = k().gemm_small_m(summed, w_second.to(DEV), 2, norm_weight=nw.to(DEV), eps=1e-5, row_squares=squares)
        close(act, plain.swiglu(normed @ w_second.float().T, torch.bfloat16), torch.bfloat16, bf16=1.2e-2)


def test_a_wait_that_is_never_satisfied_ends_by_itself_and_is_reported():
    """The bounded mbarrier wait of the tcgen05 kernels, on a barrier nothing arrives on: it gives
    up after about a second, records its code, raises the CTA's abort flag, the kernel returns and
    the context goes on working."""
    status, waited = k().wait_probe(77)
    assert status == 77
    assert 500 <= waited <= 20_000          # millions of SM cycles: the limit is 2e9
    x = torch.arange(8, device=DEV)
    assert int((x * 2).sum()) == 56          # the device still answers
    assert k().gemm_tc_status() == 0 and k().attention_prefill_tc_status() == 0
