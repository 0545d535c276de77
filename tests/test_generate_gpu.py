"""Generation through the Python entry point against the plain implementation."""

import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import PAGE_SIZES, TINY_CONFIGS, random_tokens

pytestmark = pytest.mark.gpu


def engine_config(folder, name, dtype="float32", **more):
    from tinyvllm_b200 import EngineConfig

    base = dict(model=folder, dtype=dtype, max_model_len=512, max_num_seqs=4,
                max_num_batched_tokens=64, prefill_chunk_size=24, kv_block_size=PAGE_SIZES[name],
                kv_cache_memory_bytes=16 * 1024 * 1024, prefill_reserve_tokens=0,
                prefill_reserve_requests=0)
    base.update(more)
    return EngineConfig(**base)


@pytest.mark.parametrize("eager", [True, False], ids=["eager", "graphs"])
@pytest.mark.parametrize("name", sorted(TINY_CONFIGS))
def test_greedy_generation_matches_plain(name, eager, model_folders):
    from tinyvllm_b200 import LLM, SamplingParams

    config = TINY_CONFIGS[name]
    folder = model_folders[name]
    prompts = [random_tokens(config.vocab_size, n, 300 + n) for n in (1, 9, 40, 77, 130)]
    with LLM(engine_config(folder, name, enforce_eager=eager)) as llm:
        outputs = llm.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
        if not eager:
            assert llm.engine.graph_steps > 0
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    for prompt, output in zip(prompts, outputs):
        assert output.prompt_token_count == len(prompt)
        assert output.finish_reason == "length"
        assert list(output.output_token_ids) == plain.greedy_generate(cfg, weights, prompt, 10)


def test_long_decoding(model_folders):
    """300 decoded tokens from a short prompt, graphs on, float32: every token equals the oracle's."""
    from tinyvllm_b200 import LLM, SamplingParams

    name = "a"
    folder = model_folders[name]
    prompt = random_tokens(TINY_CONFIGS[name].vocab_size, 5, 77)
    with LLM(engine_config(folder, name, max_model_len=400)) as llm:
        output = llm.generate([prompt], SamplingParams(max_new_tokens=300, ignore_eos=True))[0]
    assert len(output.output_token_ids) == 300
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    sequence = prompt + list(output.output_token_ids)
    logits = plain.forward(cfg, weights, sequence[:-1])
    assert logits[len(prompt) - 1:].argmax(-1).tolist() == list(output.output_token_ids)
