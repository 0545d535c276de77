"""Generation through the Python entry point against the plain implementation."""

import pytest

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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_runs_give_the_tokens_of_single_steps(dtype, model_folders):
    """Several decode steps back to back, fed on the device, against one step at a time: the same
    tokens for greedy and for seeded sampling, requests that stop on a token inside a run, requests
    that end by length at different times, and a newcomer while others decode."""
    from tinyvllm_b200 import GenerateRequest, SamplingParams
    from tinyvllm_b200.engine.engine import Engine

    name = "e" if dtype == "bfloat16" else "b"
    config = TINY_CONFIGS[name]
    folder = model_folders[name]
    prompts = [random_tokens(config.vocab_size, n, 500 + n) for n in (3, 17, 40, 9)]
    samplings = [SamplingParams(max_new_tokens=23, ignore_eos=True),
                 SamplingParams(max_new_tokens=9, temperature=0.8, top_k=20, seed=5, ignore_eos=True),
                 SamplingParams(max_new_tokens=30, temperature=1.1, top_p=0.9, seed=11, ignore_eos=True),
                 SamplingParams(max_new_tokens=14, ignore_eos=True)]
    results = {}
    for run_steps in (1, 4):
        engine = Engine.from_config(engine_config(folder, name, dtype=dtype, decode_run_steps=run_steps))
        try:
            # stop tokens: whatever the first request produces as its 6th token ends it there
            if run_steps == 1:
                probe = engine.generate([GenerateRequest(tuple(prompts[0]), samplings[0])])[0]
                stop = probe.output_token_ids[5]
            engine.scheduler.eos_token_ids = frozenset({stop})
            stopping = SamplingParams(max_new_tokens=23)
            ids = [engine.submit(p, s) for p, s in zip(prompts[:3], [stopping] + samplings[1:3])]
            outputs = {}
            steps = 0
            while engine.has_unfinished():
                if steps == 3:
                    ids.append(engine.submit(prompts[3], samplings[3]))       # arrives while others decode
                for done in engine.step().finished:
                    outputs[done.request_id] = (tuple(done.output_token_ids), done.finish_reason)
                steps += 1
            results[run_steps] = [outputs[i] for i in ids]
            if run_steps > 1:
                assert engine.steps_run > steps          # some calls ran several decode steps
        finally:
            engine.close()
    assert results[1] == results[4]
    assert results[1][0][1] == "stop" and len(results[1][0][0]) <= 6
