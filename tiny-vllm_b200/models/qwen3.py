"""Dense Qwen3: typed configuration and its description as parts.

Everything this file knows comes from config.json keys; the sizes reach the
parts as parameters of the spec.  Keys and checks follow
tinyvllm/models/qwen3.py:25-36 (required keys), :100-121 and :123-201
(validation).  Unlike the reference, which refuses ``use_sliding_window``
(:186-189), a window is accepted and turns the named layers into windowed
attention layers with a cache group of their own.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "num_key_value_heads",
    "head_dim",
    "max_position_embeddings",
)


def _positive_int(name: str, value: Any) -> int:
    if type(value) is not int or value <= 0:
        raise ConfigError(f"{name} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float = 1_000_000.0      # default of tinyvllm/layers.py:175
    rms_norm_eps: float = 1e-6           # default of tinyvllm/layers.py:136
    tie_word_embeddings: bool = False
    eos_token_ids: tuple[int, ...] = ()
    # window[i] is None for full attention, else the number of keys layer i sees
    layer_windows: tuple[int | None, ...] = ()

    architecture = "Qwen3ForCausalLM"

    def __post_init__(self) -> None:
        for name in _REQUIRED:
            _positive_int(name, getattr(self, name))
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2:
            raise ConfigError("head_dim must be even")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.layer_windows:
            object.__setattr__(self, "layer_windows", (None,) * self.num_hidden_layers)
        if len(self.layer_windows) != self.num_hidden_layers:
            raise ConfigError("layer_windows must have one entry per layer")
        for window in self.layer_windows:
            if window is not None:
                _positive_int("sliding_window", window)
        for token in self.eos_token_ids:
            if type(token) is not int or not 0 <= token < self.vocab_size:
                raise ConfigError(f"eos_token_id {token!r} is not a token of the vocabulary")

    # ------------------------------------------------------------------ json
    @classmethod
    def from_json(cls, data: Mapping[str, Any]) -> "Qwen3Config":
        if data.get("model_type") != "qwen3":
            raise ConfigError("only model_type='qwen3' is supported")
        missing = [name for name in _REQUIRED if name not in data]
        if missing:
            raise ConfigError("missing config.json keys: " + ", ".join(sorted(missing)))
        if data.get("hidden_act", "silu") != "silu":
            raise ConfigError("only hidden_act='silu' is supported")
        if data.get("attention_bias", False):
            raise ConfigError("attention_bias is not supported")
        scaling = data.get("rope_scaling")
        if scaling and not (isinstance(scaling, Mapping)
                            and scaling.get("rope_type", scaling.get("type")) == "default"):
            raise ConfigError("rope_scaling is not supported")

        layers = data["num_hidden_layers"]
        _positive_int("num_hidden_layers", layers)
        windows: list[int | None] = [None] * layers
        if data.get("use_sliding_window", False):
            size = data.get("sliding_window")
            _positive_int("sliding_window", size)
            kinds = data.get("layer_types")
            if kinds is None:
                first = data.get("max_window_layers", layers)
                if type(first) is not int or first < 0:
                    raise ConfigError("max_window_layers must be a non-negative integer")
                kinds = ["full_attention" if i < first else "sliding_attention"
                         for i in range(layers)]
            if not isinstance(kinds, list) or len(kinds) != layers:
                raise ConfigError("layer_types must have one entry per layer")
            for i, kind in enumerate(kinds):
                if kind == "sliding_attention":
                    windows[i] = size
                elif kind != "full_attention":
                    raise ConfigError(f"layer_types[{i}] = {kind!r} is not supported")

        eos = data.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif type(eos) is int:
            eos_ids = (eos,)
        elif isinstance(eos, list):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("eos_token_id must be an integer or a list of integers")

        theta = data.get("rope_theta", 1_000_000.0)
        eps = data.get("rms_norm_eps", 1e-6)
        if type(theta) not in (int, float) or type(eps) not in (int, float):
            raise ConfigError("rope_theta and rms_norm_eps must be numbers")
        tied = data.get("tie_word_embeddings", False)
        if type(tied) is not bool:
            raise ConfigError("tie_word_embeddings must be true or false")
        return cls(
            **{name: data[name] for name in _REQUIRED},
            rope_theta=float(theta),
            rms_norm_eps=float(eps),
            tie_word_embeddings=tied,
            eos_token_ids=eos_ids,
            layer_windows=tuple(windows),
        )

    def to_json(self) -> dict[str, Any]:
        data: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            **{name: getattr(self, name) for name in _REQUIRED},
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
        }
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        sizes = {w for w in self.layer_windows if w is not None}
        if len(sizes) > 1:
            raise ConfigError("config.json can hold one sliding_window size only")
        if sizes:
            data["use_sliding_window"] = True
            data["sliding_window"] = sizes.pop()
            data["layer_types"] = [
                "full_attention" if w is None else "sliding_attention"
                for w in self.layer_windows
            ]
        else:
            data["use_sliding_window"] = False
        return data

    # ------------------------------------------------------------------ spec
    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"width": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec("rope_half_split", {
            "head_dim": self.head_dim,
            "theta": self.rope_theta,
            "max_positions": self.max_position_embeddings,
        })
        feed_forward = PartSpec("swiglu", {
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
        })
        block = PartSpec("prenorm_residual", {
            "mixer_norm_name": "input_layernorm",
            "feed_forward_norm_name": "post_attention_layernorm",
            "mixer_name": "self_attn",
            "feed_forward_name": "mlp",
        })
        layers = []
        for index, window in enumerate(self.layer_windows):
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "scale": self.head_dim ** -0.5,   # tinyvllm/models/qwen3.py:228
                "qk_norm_eps": self.rms_norm_eps,  # tinyvllm/models/qwen3.py:250-261
                "window": window,
                "position": position,
            })
            layers.append(LayerSpec(
                prefix=f"model.layers.{index}",
                block=block, mixer=mixer, feed_forward=feed_forward, norm=norm,
            ))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {
                "vocab_size": self.vocab_size,
                "width": self.hidden_size,
                "name": "model.embed_tokens.weight",
            }),
            layers=tuple(layers),
            order=tuple(RunStep(i) for i in range(self.num_hidden_layers)),
            final_norm=norm.with_params(name="model.norm.weight"),
            head=PartSpec("lm_head", {
                "vocab_size": self.vocab_size,
                "width": self.hidden_size,
                "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None,
                "name": "lm_head.weight",
            }),
            eos_token_ids=self.eos_token_ids,
        )


register_architecture(Qwen3Config.architecture, Qwen3Config)
