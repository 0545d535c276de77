"""Configuration: config.json keys, the registry, engine limits.  No GPU."""

import json

import pytest

from tiny_configs import TINY_CONFIGS
from tinyvllm_b200 import EngineConfig, architecture_names, read_model_config, register_architecture
from tinyvllm_b200.config.registry import ConfigError, parse_model_config
from tinyvllm_b200.models import Qwen3Config


def base_json():
    return TINY_CONFIGS["b"].to_json()


def test_round_trip_and_spec():
    for name, config in TINY_CONFIGS.items():
        data = json.loads(json.dumps(config.to_json()))
        again = parse_model_config(data)
        assert again == config, name
        spec = config.to_spec()
        assert len(spec.layers) == config.num_hidden_layers == len(spec.order)
        assert spec.vocab_size == config.vocab_size
        mixer = spec.layers[0].mixer.params
        assert mixer["num_heads"] == config.num_attention_heads
        assert mixer["head_dim"] == config.head_dim
        assert mixer["scale"] == config.head_dim ** -0.5
        assert [layer.mixer.params["window"] for layer in spec.layers] == list(config.layer_windows)
        assert spec.head.params["tied_to"] == ("model.embed_tokens.weight" if config.tie_word_embeddings else None)


def test_registry_names_and_unknown_architecture():
    assert "Qwen3ForCausalLM" in architecture_names()
    data = base_json()
    data["architectures"] = ["NoSuchModel"]
    with pytest.raises(ConfigError, match="unknown architecture 'NoSuchModel'.*Qwen3ForCausalLM"):
        parse_model_config(data)
    data["architectures"] = []
    with pytest.raises(ConfigError, match="exactly one"):
        parse_model_config(data)
    with pytest.raises(TypeError):
        register_architecture("Broken", object)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "head_dim",
                                 "max_position_embeddings"])
def test_required_keys(key):
    data = base_json()
    del data[key]
    with pytest.raises(ConfigError, match=key):
        parse_model_config(data)
    data = base_json()
    data[key] = 0
    with pytest.raises(ConfigError, match=key):
        parse_model_config(data)


@pytest.mark.parametrize("change, message", [
    ({"model_type": "llama"}, "model_type"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"num_key_value_heads": 4}, "multiple"),
    ({"head_dim": 31}, "even"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 8, "layer_types": ["full_attention"]}, "layer_types"),
    ({"use_sliding_window": True, "sliding_window": 8,
      "layer_types": ["full_attention", "chunked", "full_attention"]}, "chunked"),
    ({"eos_token_id": 99999}, "eos_token_id"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_refused_options(change, message):
    data = base_json()
    data.update(change)
    with pytest.raises(ConfigError, match=message):
        parse_model_config(data)


def test_defaults_and_windows():
    data = base_json()
    for key in ("rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        data.pop(key, None)
    config = parse_model_config(data)
    assert config.rope_theta == 1_000_000.0 and config.rms_norm_eps == 1e-6
    assert config.tie_word_embeddings is False and config.eos_token_ids == ()
    data.update({"use_sliding_window": True, "sliding_window": 16, "max_window_layers": 1,
                 "eos_token_id": [3, 7]})
    config = parse_model_config(data)
    assert config.layer_windows == (None, 16, 16) and config.eos_token_ids == (3, 7)


def test_read_model_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="cannot read"):
        read_model_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_model_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(base_json()))
    assert isinstance(read_model_config(tmp_path), Qwen3Config)


def test_engine_config_validation(tmp_path):
    ok = EngineConfig(model=tmp_path)
    assert ok.dtype == "bfloat16" and ok.kv_block_size == 16 and ok.max_model_len == 4096
    with pytest.raises(ValueError, match="does not exist"):
        EngineConfig(model=tmp_path / "absent")
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(model=tmp_path, dtype="float16")
    with pytest.raises(ValueError, match="max_num_seqs"):
        EngineConfig(model=tmp_path, max_num_seqs=0)
    with pytest.raises(ValueError, match="between 0 and 1"):
        EngineConfig(model=tmp_path, gpu_memory_utilization=1.5)
    with pytest.raises(ValueError, match="both"):
        EngineConfig(model=tmp_path, prefill_reserve_tokens=0)
    with pytest.raises(ValueError, match="chunk"):
        EngineConfig(model=tmp_path, prefill_chunk_size=8192)
    with pytest.raises(TypeError):
        EngineConfig(model=tmp_path, enforce_eager=1)
