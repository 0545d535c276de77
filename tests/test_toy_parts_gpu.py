"""Parts and an architecture defined HERE, registered, built and stepped without touching the
framework: a mixer with per-request state of its own, layers that choose their mixer one by one,
and a run list that names a layer twice and lets a run read another run's cache."""

import json

import pytest
import torch

import plain_qwen3 as plain
import replay_helpers as rh
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

DECAY = 0.5


def register_toy_parts():
    from tinyvllm_b200 import register_architecture
    from tinyvllm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
    from tinyvllm_b200.parts import ParamSpec, Part, StateNeed, register_part

    class DecayMixer(Part):
        """s_t = DECAY * s_{t-1} + x_t per request, y_t = s_t * w: a recurrence whose state lives
        in the request's state slot between steps."""

        def __init__(self, ctx, *, width):
            self.width = width
            self.name = f"{ctx.prefix}.w"
            self.dtype = ctx.dtype
            self.w = None

        def param_specs(self):
            return [ParamSpec.single("w", self.name, (self.width,), role="vector", init="around_one")]

        def cache_need(self):
            return StateNeed((self.width,), torch.float32)

        def forward(self, x, ctx, run):
            arena = ctx.storage.state_of(run)
            out = torch.empty_like(x)
            first = 0
            for _request, _start, count, slot, _fresh in ctx.host_rows:
                state = arena[slot].clone()
                for t in range(first, first + count):
                    state = DECAY * state + x[t].float()
                    out[t] = (state * self.w.float()).to(x.dtype)
                arena[slot] = state
                first += count
            return out

    class ToyConfig:
        architecture = "ToyMixedForCausalLM"

        def __init__(self, data):
            self.data = dict(data)

        @classmethod
        def from_json(cls, data):
            return cls(data)

        def to_json(self):
            return {"architectures": [self.architecture], **{k: v for k, v in self.data.items()
                                                            if k != "architectures"}}

        def to_spec(self):
            d = self.data
            width = d["width"]
            norm = PartSpec("rms_norm", {"width": width, "eps": d["eps"]})
            ff = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": d["inter"]})
            block = PartSpec("prenorm_residual", {
                "mixer_norm_name": "input_layernorm", "feed_forward_norm_name": "post_attention_layernorm",
                "mixer_name": "self_attn", "feed_forward_name": "mlp"})
            attention = PartSpec("gqa_attention", {
                "hidden_size": width, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                "head_dim": d["head_dim"], "scale": d["head_dim"] ** -0.5, "qk_norm_eps": d["eps"],
                "window": None,
                "position": PartSpec("rope_half_split", {"head_dim": d["head_dim"], "theta": d["theta"],
                                                         "max_positions": d["max_positions"]})})
            decay = PartSpec("toy_decay", {"width": width})
            layers = tuple(
                LayerSpec(f"model.layers.{i}", block, decay if kind == "decay" else attention, ff, norm)
                for i, kind in enumerate(d["mixers"]))
            return ModelSpec(
                architecture=self.architecture, vocab_size=d["vocab"], hidden_size=width,
                max_positions=d["max_positions"],
                embedding=PartSpec("token_embedding", {"vocab_size": d["vocab"], "width": width,
                                                       "name": "model.embed_tokens.weight"}),
                layers=layers,
                order=tuple(RunStep(layer, source) for layer, source in d["order"]),
                final_norm=norm.with_params(name="model.norm.weight"),
                head=PartSpec("lm_head", {"vocab_size": d["vocab"], "width": width,
                                          "name": "lm_head.weight", "tied_to": None}))

    register_part("mixer", "toy_decay", DecayMixer)
    register_architecture(ToyConfig.architecture, ToyConfig)
    return ToyConfig


def toy_plain_forward(data, w, tokens):
    """Whole-sequence oracle of the toy model from the plain functions (float32)."""
    dt = torch.float32
    ids = torch.tensor(tokens)
    h = plain.embed(w["model.embed_tokens.weight"], ids, dt)
    cfg = {"nq": data["heads"], "nkv": data["kv_heads"], "d": data["head_dim"], "eps": data["eps"]}
    cos, sin = plain.rope_tables(data["head_dim"], len(tokens), data["theta"])
    res, produced = None, []
    for layer, source in data["order"]:
        p = f"model.layers.{layer}"
        if res is None:
            res, x = h, plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], data["eps"], dt)
        else:
            x, res = plain.add_rms_norm(h, res, w[f"{p}.input_layernorm.weight"], data["eps"], dt)
        if data["mixers"][layer] == "decay":
            state, rows = torch.zeros(data["width"]), []
            for t in range(len(tokens)):
                state = DECAY * state + x[t]
                rows.append(state * w[f"{p}.self_attn.w"])
            mixed, kv = torch.stack(rows), None
        else:
            mixed, kv = plain.attention_block(cfg, w, p, x, cos, sin, None, dt,
                                              None if source is None else produced[source])
        produced.append(kv)
        x, res = plain.add_rms_norm(mixed, res, w[f"{p}.post_attention_layernorm.weight"], data["eps"], dt)
        h = plain.mlp_block(w, p, x, dt)
    x, _ = plain.add_rms_norm(h, res, w["model.norm.weight"], data["eps"], dt)
    return x @ w["lm_head.weight"].T


TOY = {"vocab": 97, "width": 48, "inter": 80, "heads": 3, "kv_heads": 1, "head_dim": 16, "eps": 1e-5,
       "theta": 1e4, "max_positions": 512,
       "mixers": ["attention", "decay", "attention"],
       # layer 1 (the recurrence) runs twice, each run with state of its own; the last run is
       # layer 0 again, attending over the keys and values that run 0 wrote
       "order": [[0, None], [1, None], [2, None], [1, None], [0, 0]]}


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.weights.random_init import write_model_folder
    config_class = register_toy_parts()
    folder = write_model_folder(tmp_path_factory.mktemp("toy"), config_class(TOY), seed=9)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyMixedForCausalLM"]
    assert type(read_model_config(folder)).__name__ == "ToyConfig"
    return folder


def test_toy_architecture_is_built_from_the_registry_and_steps(toy):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner
    from tinyvllm_b200.parts import KVNeed, StateNeed

    model = Model(read_model_config(toy).to_spec(), device="cuda:0", dtype=torch.float32).load(toy)
    needs = model.cache_needs()
    assert [type(n) for n in needs] == [KVNeed, StateNeed, KVNeed, StateNeed, KVNeed]
    runner = StepRunner(model, page_size=4, num_pages=40, max_requests=3)
    assert len(runner.manager.groups) == 1 and runner.manager.groups[0].runs == (0, 2)
    assert sorted(runner.storage.state) == [1, 3]             # the two runs of layer 1: own arenas
    assert runner.storage.where[4] == runner.storage.where[0]  # run 4 reads run 0's pages

    weights = plain.read_weights(toy)
    requests = {f"t{n}": random_tokens(TOY["vocab"], n, 40 + n) for n in (1, 9, 33, 70, 21, 50)}
    expected = {rid: toy_plain_forward(TOY, weights, tokens) for rid, tokens in requests.items()}
    for name, steps in (("whole", rh.whole(requests)), ("tail", rh.tail_by_one(requests, tail=8)),
                        ("portions", rh.portions(requests, seed=2, sizes=(2, 3, 5, 11))),
                        ("mixed", rh.mixed(requests, seed=4, live=3, decode_tail=5, sizes=(2, 3, 9)))):
        # three state slots for six requests: slots are taken again and must start at zero
        got = rh.run_steps(runner, steps)
        if name != "tail":
            assert len(got) == sum(len(t) for t in requests.values())
        rh.compare(got, expected, torch.float32, what=f"toy {name}")
    assert runner.manager.slots.free_count == 3


def test_unknown_part_kind_is_a_clear_error(toy):
    from tinyvllm_b200.config.spec import PartSpec
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    import dataclasses
    spec = read_model_config(toy).to_spec()
    layer = dataclasses.replace(spec.layers[0], feed_forward=PartSpec("no_such_ff", {}))
    bad = dataclasses.replace(spec, layers=(layer,) + spec.layers[1:])
    with pytest.raises(KeyError, match="no feed_forward part named 'no_such_ff'.*swiglu"):
        Model(bad, device="cuda:0", dtype=torch.float32)
