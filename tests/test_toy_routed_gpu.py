"""More parts defined HERE and plugged in without touching the framework: a feed-forward with
routing (a router picks one of several small experts per token) and another position encoding
(rotation angles of interpolated positions), in an architecture whose layers choose between them."""

import pytest
import torch

import plain_qwen3 as plain
import replay_helpers as rh
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

STRETCH = 4.0          # positions are divided by this before the angles are taken


def register_routed_parts():
    from tinyvllm_b200 import register_architecture
    from tinyvllm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
    from tinyvllm_b200.parts import ParamSpec, Part, register_part

    class TopOneExperts(Part):
        """y = p * W2[e] relu(W1[e] x) with e = argmax of the router logits R x and p their softmax
        value at e; router logits and softmax in float32."""

        def __init__(self, ctx, *, width, inter, experts):
            self.width, self.inter, self.experts = width, inter, experts
            self.prefix = ctx.prefix
            self.router = self.up = self.down = None

        def param_specs(self):
            specs = [ParamSpec.single("router", f"{self.prefix}.router.weight", (self.experts, self.width))]
            specs.append(ParamSpec.packed(
                "up", [(f"{self.prefix}.experts.{e}.up.weight", self.inter) for e in range(self.experts)], self.width))
            specs.append(ParamSpec.packed(
                "down", [(f"{self.prefix}.experts.{e}.down.weight", self.width) for e in range(self.experts)],
                self.inter))
            return specs

        def forward(self, x, ctx):
            logits = x.float() @ self.router.float().T
            chosen = logits.argmax(dim=-1)
            weight = torch.softmax(logits, dim=-1).gather(1, chosen[:, None])
            up = self.up.float().view(self.experts, self.inter, self.width)[chosen]          # [t, inter, width]
            down = self.down.float().view(self.experts, self.width, self.inter)[chosen]      # [t, width, inter]
            hidden = torch.relu(torch.bmm(up, x.float()[:, :, None]))
            return (weight * torch.bmm(down, hidden)[:, :, 0]).to(x.dtype)

    class StretchedRope(Part):
        """Half-split rotation by the angles of position / STRETCH: the tables the attention kernels
        read are this part's own."""

        pairing = "half_split"          # the pairing the fused q/k kernels apply to the tables

        def __init__(self, ctx, *, head_dim, theta, max_positions):
            self.head_dim, self.theta, self.max_positions = head_dim, float(theta), max_positions
            self.device = ctx.device
            self.cos = self.sin = None

        def finalize(self):
            exponent = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim
            inv_freq = 1.0 / (self.theta ** exponent)
            angles = (torch.arange(self.max_positions, dtype=torch.float32) / STRETCH)[:, None] * inv_freq[None, :]
            self.cos, self.sin = angles.cos().to(self.device), angles.sin().to(self.device)

    class RoutedConfig:
        architecture = "ToyRoutedForCausalLM"

        def __init__(self, data):
            self.data = dict(data)

        @classmethod
        def from_json(cls, data):
            return cls(data)

        def to_json(self):
            return {"architectures": [self.architecture],
                    **{k: v for k, v in self.data.items() if k != "architectures"}}

        def to_spec(self):
            d = self.data
            width = d["width"]
            norm = PartSpec("rms_norm", {"width": width, "eps": d["eps"]})
            block = PartSpec("prenorm_residual", {
                "mixer_norm_name": "input_layernorm", "feed_forward_norm_name": "post_attention_layernorm",
                "mixer_name": "self_attn", "feed_forward_name": "mlp"})
            dense = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": d["inter"]})
            routed = PartSpec("toy_top_one_experts", {"width": width, "inter": d["expert_inter"],
                                                      "experts": d["experts"]})

            def attention(position_kind):
                return PartSpec("gqa_attention", {
                    "hidden_size": width, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                    "head_dim": d["head_dim"], "scale": d["head_dim"] ** -0.5, "qk_norm_eps": d["eps"],
                    "window": None,
                    "position": PartSpec(position_kind, {"head_dim": d["head_dim"], "theta": d["theta"],
                                                         "max_positions": d["max_positions"]})})

            layers = tuple(
                LayerSpec(f"model.layers.{i}", block,
                          attention("toy_stretched_rope" if stretched else "rope_half_split"),
                          routed if is_routed else dense, norm)
                for i, (stretched, is_routed) in enumerate(d["layers"]))
            return ModelSpec(
                architecture=self.architecture, vocab_size=d["vocab"], hidden_size=width,
                max_positions=d["max_positions"],
                embedding=PartSpec("token_embedding", {"vocab_size": d["vocab"], "width": width,
                                                       "name": "model.embed_tokens.weight"}),
                layers=layers, order=tuple(RunStep(i, None) for i in range(len(layers))),
                final_norm=norm.with_params(name="model.norm.weight"),
                head=PartSpec("lm_head", {"vocab_size": d["vocab"], "width": width,
                                          "name": "lm_head.weight", "tied_to": None}))

    register_part("feed_forward", "toy_top_one_experts", TopOneExperts)
    register_part("position", "toy_stretched_rope", StretchedRope)
    register_architecture(RoutedConfig.architecture, RoutedConfig)
    return RoutedConfig


ROUTED = {"vocab": 89, "width": 40, "inter": 72, "expert_inter": 24, "experts": 3, "heads": 2, "kv_heads": 2,
          "head_dim": 16, "eps": 2e-6, "theta": 5e3, "max_positions": 256,
          # (stretched positions?, routed feed-forward?) layer by layer
          "layers": [[True, False], [False, True], [True, True]]}


def routed_plain_forward(data, w, tokens):
    """Whole-sequence oracle from the plain functions (float32), routing restated here."""
    dt = torch.float32
    h = plain.embed(w["model.embed_tokens.weight"], torch.tensor(tokens), dt)
    cfg = {"nq": data["heads"], "nkv": data["kv_heads"], "d": data["head_dim"], "eps": data["eps"]}
    d, n = data["head_dim"], len(tokens)
    plain_cos, plain_sin = plain.rope_tables(d, n, data["theta"])
    inv_freq = 1.0 / (data["theta"] ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angles = (torch.arange(n, dtype=torch.float32) / STRETCH)[:, None] * inv_freq[None, :]
    res = None
    for layer, (stretched, is_routed) in enumerate(data["layers"]):
        p = f"model.layers.{layer}"
        if res is None:
            res, x = h, plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], data["eps"], dt)
        else:
            x, res = plain.add_rms_norm(h, res, w[f"{p}.input_layernorm.weight"], data["eps"], dt)
        cos, sin = (angles.cos(), angles.sin()) if stretched else (plain_cos, plain_sin)
        mixed, _ = plain.attention_block(cfg, w, p, x, cos, sin, None, dt)
        x, res = plain.add_rms_norm(mixed, res, w[f"{p}.post_attention_layernorm.weight"], data["eps"], dt)
        if is_routed:
            logits = x @ w[f"{p}.mlp.router.weight"].T
            chosen = logits.argmax(dim=-1)
            weight = torch.softmax(logits, dim=-1)
            rows = []
            for t in range(n):
                e = int(chosen[t])
                hidden = torch.relu(w[f"{p}.mlp.experts.{e}.up.weight"] @ x[t])
                rows.append(weight[t, e] * (w[f"{p}.mlp.experts.{e}.down.weight"] @ hidden))
            h = torch.stack(rows)
        else:
            h = plain.mlp_block(w, p, x, dt)
    x, _ = plain.add_rms_norm(h, res, w["model.norm.weight"], data["eps"], dt)
    return x @ w["lm_head.weight"].T


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner
    from tinyvllm_b200.weights.random_init import write_model_folder

    config_class = register_routed_parts()
    folder = write_model_folder(tmp_path / "routed", config_class(ROUTED), seed=11)
    assert type(read_model_config(folder)).__name__ == "RoutedConfig"
    model = Model(read_model_config(folder).to_spec(), device="cuda:0", dtype=torch.float32).load(folder)
    kinds = [(type(b.mixer.position).__name__, type(b.feed_forward).__name__) for b in model.blocks]
    assert kinds == [("StretchedRope", "SwiGLU"), ("RopeHalfSplit", "TopOneExperts"),
                     ("StretchedRope", "TopOneExperts")]
    # the two position encodings have tables of their own
    assert not torch.equal(model.blocks[0].mixer.position.cos, model.blocks[1].mixer.position.cos)
    runner = StepRunner(model, page_size=4, num_pages=40, max_requests=3)
    weights = plain.read_weights(folder)
    requests = {f"q{n}": random_tokens(ROUTED["vocab"], n, 70 + n) for n in (1, 12, 37, 64, 25)}
    expected = {rid: routed_plain_forward(ROUTED, weights, tokens) for rid, tokens in requests.items()}
    # the router's choices differ along a sequence, or the test would not see a wrong expert
    x = plain.embed(weights["model.embed_tokens.weight"], torch.tensor(requests["q64"]), torch.float32)
    assert len(set((x @ weights["model.layers.1.mlp.router.weight"].T).argmax(-1).tolist())) > 1
    for name, steps in (("whole", rh.whole(requests)), ("tail", rh.tail_by_one(requests, tail=6)),
                        ("portions", rh.portions(requests, seed=5, sizes=(2, 3, 7, 13))),
                        ("mixed", rh.mixed(requests, seed=6, live=3, decode_tail=4, sizes=(2, 5, 9)))):
        rh.compare(rh.run_steps(runner, steps), expected, torch.float32, what=f"routed {name}")


def test_a_position_encoding_with_another_pairing_is_refused_by_the_fused_kernels(tmp_path):
    """The attention kernels rotate q and k themselves, with the half-split pairing: a position part
    that pairs elements otherwise must not reach them with its tables (wrong results would be silent)."""
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepEntry, StepRunner
    from tinyvllm_b200.ops.kernels import KernelError
    from tinyvllm_b200.weights.random_init import write_model_folder

    config_class = register_routed_parts()
    folder = write_model_folder(tmp_path / "routed", config_class(ROUTED), seed=11)
    model = Model(read_model_config(folder).to_spec(), device="cuda:0", dtype=torch.float32).load(folder)
    model.blocks[0].mixer.position.pairing = "interleaved"
    runner = StepRunner(model, page_size=4, num_pages=40, max_requests=2)
    runner.open("r")
    with pytest.raises(KernelError, match="half-split pairing.*'interleaved'"):
        runner.run([StepEntry("r", (1, 2, 3), (2,))])
    runner.manager.check()
    assert all(pool.free_count == pool.num_pages for pool in runner.manager.pools)        # the step's pages went back
