"""Weights by name: dtype rules, packing, one error for everything wrong, random mode.  No GPU."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from tiny_configs import SEEDS, TINY_CONFIGS
from tinyvllm_b200.engine.model import Model
from tinyvllm_b200.weights.loader import WeightsError, load_checkpoint
from tinyvllm_b200.weights.random_init import random_tensors, write_model_folder


def cpu_model(name, dtype):
    return Model(TINY_CONFIGS[name].to_spec(), device="cpu", dtype=dtype)


def load(model, folder, dtype):
    load_checkpoint(model.param_targets(), folder, dtype=dtype, device="cpu",
                    aliases=model._name_aliases())


def test_folder_has_config_and_tensors(model_folders):
    for name, folder in model_folders.items():
        config = TINY_CONFIGS[name]
        assert json.loads((folder / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
        tensors = load_file(str(folder / "model.safetensors"))
        assert ("lm_head.weight" in tensors) == (not config.tie_word_embeddings)
        assert tensors["model.embed_tokens.weight"].shape == (config.vocab_size, config.hidden_size)
        q = tensors["model.layers.0.self_attn.q_proj.weight"]
        assert q.shape == (config.num_attention_heads * config.head_dim, config.hidden_size)
        assert abs(q.std().item() - 0.02) < 0.004
        norm = tensors["model.layers.0.input_layernorm.weight"]
        assert 0.9 <= norm.min().item() and norm.max().item() <= 1.1


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a = write_model_folder(tmp_path / "a", TINY_CONFIGS["a"], 5)
    b = write_model_folder(tmp_path / "b", TINY_CONFIGS["a"], 5)
    c = write_model_folder(tmp_path / "c", TINY_CONFIGS["a"], 6)
    ta, tb, tc = (load_file(str(f / "model.safetensors")) for f in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["model.norm.weight"], tc["model.norm.weight"])


def test_packing_and_dtype_rules(model_folders):
    name = "b"
    config = TINY_CONFIGS[name]
    stored = load_file(str(model_folders[name] / "model.safetensors"))
    model = cpu_model(name, torch.bfloat16)
    load(model, model_folders[name], torch.bfloat16)
    attention = model.blocks[1].mixer
    q_rows = config.num_attention_heads * config.head_dim
    kv_rows = config.num_key_value_heads * config.head_dim
    assert attention.qkv_weight.dtype == torch.bfloat16
    assert attention.qkv_weight.shape == (q_rows + 2 * kv_rows, config.hidden_size)
    assert torch.equal(attention.qkv_weight[q_rows:q_rows + kv_rows],
                       stored["model.layers.1.self_attn.k_proj.weight"].to(torch.bfloat16))
    mlp = model.blocks[2].feed_forward
    assert torch.equal(mlp.gate_up_weight[config.intermediate_size:],
                       stored["model.layers.2.mlp.up_proj.weight"].to(torch.bfloat16))
    # a vector the file stores in 32-bit stays 32-bit; matrices and tables take the storage dtype
    assert model.final_norm.weight.dtype == torch.float32
    assert attention.q_norm_weight.dtype == torch.float32
    assert model.embedding.weight.dtype == torch.bfloat16
    # in a float32 model everything is float32 and exact
    model32 = cpu_model(name, torch.float32)
    load(model32, model_folders[name], torch.float32)
    assert torch.equal(model32.head.weight, stored["lm_head.weight"])


def test_vectors_stored_in_bfloat16_stay_bfloat16(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_CONFIGS["a"], 0, dtype=torch.bfloat16)
    model = cpu_model("a", torch.bfloat16)
    load(model, folder, torch.bfloat16)
    assert model.final_norm.weight.dtype == torch.bfloat16
    model32 = cpu_model("a", torch.float32)
    load(model32, folder, torch.float32)
    assert model32.final_norm.weight.dtype == torch.float32


def test_one_error_lists_everything(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_CONFIGS["b"], SEEDS["b"])
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.0.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(3)
    tensors["model.layers.1.self_attn.o_proj.weight"] = torch.zeros(5, 7)
    tensors["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(8)
    save_file(tensors, str(folder / "model.safetensors"))
    model = cpu_model("b", torch.float32)
    with pytest.raises(WeightsError) as info:
        load(model, folder, torch.float32)
    error = info.value
    assert set(error.missing) == {"model.layers.0.mlp.down_proj.weight", "model.norm.weight"}
    assert error.unexpected == ("model.layers.9.extra.weight",)
    assert {name for name, _, _ in error.wrong_shape} == {
        "model.layers.1.self_attn.o_proj.weight", "model.layers.2.self_attn.q_norm.weight"}
    text = str(error)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape", "[5, 7]", "expected [96, 192]"):
        assert needle in text


def test_tied_head_may_be_stored_and_no_shards_is_an_error(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_CONFIGS["a"], 0)
    tensors = {name: tensor.clone() for name, tensor in load_file(str(folder / "model.safetensors")).items()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(folder / "model.safetensors"))
    load(cpu_model("a", torch.float32), folder, torch.float32)
    # stored under the head's name only: it is the embedding (tinyvllm/models/qwen3.py:637-641, :682-686)
    embedding = tensors.pop("model.embed_tokens.weight")
    tensors["lm_head.weight"] = embedding * 2
    save_file(tensors, str(folder / "model.safetensors"))
    model = cpu_model("a", torch.float32)
    load(model, folder, torch.float32)
    assert torch.equal(model.embedding.weight, embedding * 2)
    (folder / "model.safetensors").unlink()
    with pytest.raises(WeightsError, match="no .safetensors"):
        load(cpu_model("a", torch.float32), folder, torch.float32)


def test_index_file_names_shards(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_CONFIGS["a"], 0)
    tensors = load_file(str(folder / "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(folder / "part-1.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(folder / "part-2.safetensors"))
    (folder / "model.safetensors").unlink()
    index = {"weight_map": {k: ("part-1.safetensors" if i < half else "part-2.safetensors")
                            for i, k in enumerate(names)}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    load(cpu_model("a", torch.float32), folder, torch.float32)
    (folder / "part-2.safetensors").unlink()
    with pytest.raises(WeightsError, match="absent"):
        load(cpu_model("a", torch.float32), folder, torch.float32)


def test_random_stream_order_is_declaration_order():
    model = Model(TINY_CONFIGS["a"].to_spec(), device="meta", dtype=torch.float32)
    names = [name for name, _ in random_tensors(model.param_targets(), 0)]
    assert names[0] == "model.embed_tokens.weight"
    assert names[1] == "model.layers.0.input_layernorm.weight"
    assert names[-1] == "model.norm.weight"
    assert len(names) == len(set(names)) == 2 + 11 * 2
