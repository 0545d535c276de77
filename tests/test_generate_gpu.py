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
    for run_steps in (1, 4, 32):
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
    assert results[1] == results[4] == results[32]
    assert results[1][0][1] == "stop" and len(results[1][0][0]) <= 6


def test_a_request_cancelled_while_a_run_is_in_flight_leaves_the_others_alone(model_folders):
    """Steps of a run are launched ahead of the ones read: a cancel between two calls ends the run
    after what was launched, the other requests get the tokens they get without it, and every page
    comes back."""
    from tinyvllm_b200 import GenerateRequest, SamplingParams
    from tinyvllm_b200.engine.engine import Engine

    name, dtype = "e", "bfloat16"
    config = TINY_CONFIGS[name]
    folder = model_folders[name]
    prompts = [random_tokens(config.vocab_size, n, 700 + n) for n in (11, 30, 5)]
    sampling = SamplingParams(max_new_tokens=40, ignore_eos=True)
    engine = Engine.from_config(engine_config(folder, name, dtype=dtype, decode_run_steps=1))
    try:
        alone = engine.generate([GenerateRequest(tuple(p), sampling) for p in prompts])
    finally:
        engine.close()
    engine = Engine.from_config(engine_config(folder, name, dtype=dtype, decode_run_steps=32))
    try:
        ids = [engine.submit(p, sampling) for p in prompts]
        outputs, calls, cancelled_at = {}, 0, None
        while engine.has_unfinished():
            if engine._run is not None and cancelled_at is None and calls >= 6:
                assert engine.cancel(ids[1])
                cancelled_at = calls
            for done in engine.step().finished:
                outputs[done.request_id] = done
            calls += 1
        assert cancelled_at is not None and engine._run is None
        assert outputs[ids[1]].finish_reason == "cancelled"
        cut = list(outputs[ids[1]].output_token_ids)
        assert 0 < len(cut) < 40 and cut == list(alone[1].output_token_ids)[:len(cut)]
        for i in (0, 2):
            assert list(outputs[ids[i]].output_token_ids) == list(alone[i].output_token_ids)
        engine.runner.manager.check()
        assert all(pool.free_count == pool.num_pages for pool in engine.runner.manager.pools)
    finally:
        engine.close()


def test_streamed_tokens_are_the_generated_ones(model_folders, capsys):
    """LLM.stream yields every token as it comes and the outputs of generate; the command line
    prints them with --stream."""
    import json

    from tinyvllm_b200 import LLM, SamplingParams
    from tinyvllm_b200.__main__ import main

    name = "b"
    folder = model_folders[name]
    prompts = [random_tokens(TINY_CONFIGS[name].vocab_size, n, 900 + n) for n in (4, 31)]
    sampling = SamplingParams(max_new_tokens=12, ignore_eos=True)
    with LLM(engine_config(folder, name)) as llm:
        want = [list(o.output_token_ids) for o in llm.generate(prompts, sampling)]
        tokens, outputs = {0: [], 1: []}, {}
        for index, item in llm.stream(prompts, sampling):
            if isinstance(item, int):
                assert index not in outputs                      # tokens come before the request's output
                tokens[index].append(item)
            else:
                outputs[index] = item
        assert [tokens[0], tokens[1]] == want
        assert [list(outputs[i].output_token_ids) for i in (0, 1)] == want
    main(["--model", str(folder), "--dtype", "float32", "--max-new-tokens", "12", "--ignore-eos", "--stream",
          "--kv-block-size", str(PAGE_SIZES[name]), "--kv-cache-mib", "16", "--max-model-len", "512",
          "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", ",".join(map(str, prompts[1]))])
    lines = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    streamed = {0: [], 1: []}
    for line in lines[:-1]:
        streamed[line["prompt"]].append(line["token_id"])
    assert [streamed[0], streamed[1]] == want
    assert [record["output_token_ids"] for record in lines[-1]["outputs"]] == want
