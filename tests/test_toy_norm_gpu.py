"""Another norm, defined HERE and plugged in without touching the framework: a centred norm
(y = (x - mean) * rsqrt(var + eps) * weight).  The framework's products may take an RMS norm into
their own kernel for small batches; they ask the norm part whether it is of that kind
(``folds_into_product``) and must leave this one alone.  Run in bfloat16 with one and two rows a
step, where the folding would happen, against the oracle with the norm restated."""

import pytest
import torch

import plain_qwen3 as plain
import replay_helpers as rh
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu


def register_centred_norm():
    from tinyvllm_b200 import register_architecture
    from tinyvllm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
    from tinyvllm_b200.parts import ParamSpec, Part, register_part

    class CentredNorm(Part):
        def __init__(self, ctx, *, width, eps, name=None):
            self.width, self.eps = width, float(eps)
            self.name = name if name is not None else f"{ctx.prefix}.weight"
            self.weight = None

        def param_specs(self):
            return [ParamSpec.single("weight", self.name, (self.width,), role="vector", init="around_one")]

        def forward(self, x):
            f = x.float()
            centred = f - f.mean(-1, keepdim=True)
            r = torch.rsqrt((centred * centred).mean(-1, keepdim=True) + self.eps)
            return (centred * r * self.weight.float()).to(x.dtype)

        def add(self, x, residual):
            stream = (x.float() + residual.float()).to(x.dtype)
            return self.forward(stream), stream

        def add_rows(self, x, residual, rows):
            index = rows.long()
            if residual is None:
                return self.forward(x[index])
            return self.add(x[index], residual[index])[0]

    class CentredConfig:
        architecture = "ToyCentredNormForCausalLM"

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
            norm = PartSpec("toy_centred_norm", {"width": width, "eps": d["eps"]})
            block = PartSpec("prenorm_residual", {
                "mixer_norm_name": "input_layernorm", "feed_forward_norm_name": "post_attention_layernorm",
                "mixer_name": "self_attn", "feed_forward_name": "mlp"})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": width, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                "head_dim": d["head_dim"], "scale": d["head_dim"] ** -0.5, "qk_norm_eps": d["eps"], "window": None,
                "position": PartSpec("rope_half_split", {"head_dim": d["head_dim"], "theta": d["theta"],
                                                         "max_positions": d["max_positions"]})})
            dense = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": d["inter"]})
            layers = tuple(LayerSpec(f"model.layers.{i}", block, mixer, dense, norm) for i in range(d["layers"]))
            return ModelSpec(
                architecture=self.architecture, vocab_size=d["vocab"], hidden_size=width,
                max_positions=d["max_positions"],
                embedding=PartSpec("token_embedding", {"vocab_size": d["vocab"], "width": width,
                                                       "name": "model.embed_tokens.weight"}),
                layers=layers, order=tuple(RunStep(i, None) for i in range(len(layers))),
                final_norm=norm.with_params(name="model.norm.weight"),
                head=PartSpec("lm_head", {"vocab_size": d["vocab"], "width": width,
                                          "name": "lm_head.weight", "tied_to": None}))

    register_part("norm", "toy_centred_norm", CentredNorm)
    register_architecture(CentredConfig.architecture, CentredConfig)
    return CentredConfig


CENTRED = {"vocab": 130, "width": 128, "inter": 192, "layers": 2, "heads": 4, "kv_heads": 2, "head_dim": 64,
           "eps": 1e-5, "theta": 1e4, "max_positions": 512}


def centred_norm(x, w, eps, dt):
    centred = x - x.mean(-1, keepdim=True)
    r = torch.rsqrt((centred * centred).mean(-1, keepdim=True) + eps)
    return plain.rnd(centred * r * w, dt)


def centred_plain_forward(data, w, tokens, dt):
    """Whole-sequence oracle: the plain functions with the centred norm in place of the RMS norm."""
    h = plain.embed(w["model.embed_tokens.weight"], torch.tensor(tokens), dt)
    cfg = {"nq": data["heads"], "nkv": data["kv_heads"], "d": data["head_dim"], "eps": data["eps"]}
    cos, sin = plain.rope_tables(data["head_dim"], len(tokens), data["theta"])
    res = None
    for layer in range(data["layers"]):
        p = f"model.layers.{layer}"
        win, wpost = plain.rnd(w[f"{p}.input_layernorm.weight"], dt), plain.rnd(w[f"{p}.post_attention_layernorm.weight"], dt)
        if res is None:
            res = h
        else:
            res = plain.rnd(h + res, dt)
        x = centred_norm(res, win, data["eps"], dt)
        mixed, _ = plain.attention_block(cfg, w, p, x, cos, sin, None, dt)
        res = plain.rnd(mixed + res, dt)
        h = plain.mlp_block(w, p, centred_norm(res, wpost, data["eps"], dt), dt)
    x = centred_norm(plain.rnd(h + res, dt), plain.rnd(w["model.norm.weight"], dt), data["eps"], dt)
    return x @ plain.rnd(w["lm_head.weight"], dt).T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_norm_of_another_kind_is_not_folded_into_the_products(dtype, tmp_path):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner
    from tinyvllm_b200.weights.random_init import write_model_folder

    config_class = register_centred_norm()
    folder = write_model_folder(tmp_path / "centred", config_class(CENTRED), seed=5)
    model = Model(read_model_config(folder).to_spec(), device="cuda:0", dtype=dtype).load(folder)
    assert type(model.blocks[0].mixer_norm).__name__ == "CentredNorm"
    assert not getattr(model.blocks[0].mixer_norm, "folds_into_product", False)
    runner = StepRunner(model, page_size=16, num_pages=40, max_requests=3)
    weights = plain.read_weights(folder)
    requests = {f"n{n}": random_tokens(CENTRED["vocab"], n, 30 + n) for n in (1, 20, 75, 140)}
    expected = {rid: centred_plain_forward(CENTRED, weights, tokens, dtype) for rid, tokens in requests.items()}
    # an RMS norm in its place gives other logits: the test would see a norm that was swapped
    as_rms = plain.forward({**{"V": CENTRED["vocab"], "H": CENTRED["width"], "I": CENTRED["inter"],
                               "L": CENTRED["layers"], "nq": CENTRED["heads"], "nkv": CENTRED["kv_heads"],
                               "d": CENTRED["head_dim"], "max_pos": CENTRED["max_positions"],
                               "theta": CENTRED["theta"], "eps": CENTRED["eps"], "tied": False,
                               "windows": [None] * CENTRED["layers"]}}, weights, requests["n75"], dtype)
    assert (as_rms - expected["n75"]).abs().max() > 0.05 * expected["n75"].abs().max()
    for name, steps in (("whole", rh.whole(requests)), ("tail", rh.tail_by_one(requests, tail=10)),
                        ("mixed", rh.mixed(requests, seed=2, live=2, decode_tail=6, sizes=(2, 5, 9)))):
        with torch.inference_mode():
            got = rh.run_steps(runner, steps)
        rh.compare(got, expected, dtype, what=f"centred norm {name}")
