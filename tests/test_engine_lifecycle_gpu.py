"""The engine over several batches of requests, with steps captured as CUDA graphs while it serves.

What a measurement or a server does between batches: requests are cancelled while a run of decode
steps is in flight, taken as finished, and new ones are submitted, whose prompt steps have the
shapes of the batch before and are therefore captured and then replayed.  Every logit row must be
the one of an engine that never captures anything."""

import gc

import pytest
import torch

from tiny_configs import PAGE_SIZES, TINY_CONFIGS, random_tokens

pytestmark = pytest.mark.gpu


def engine_config(folder, name, **more):
    from tinyvllm_b200 import EngineConfig

    base = dict(model=folder, dtype="bfloat16", max_model_len=1024, max_num_seqs=4,
                max_num_batched_tokens=256, prefill_chunk_size=128, kv_block_size=PAGE_SIZES[name],
                kv_cache_memory_bytes=32 * 1024 * 1024, prefill_reserve_tokens=0,
                prefill_reserve_requests=0)
    base.update(more)
    return EngineConfig(**base)


def record_logits(engine, rows):
    """The logits of every step that goes through the step runner (prompt portions, alone or beside
    decoded tokens) are copied to ``rows``."""
    launch = engine.runner.launch

    def recording(prepared):
        logits = launch(prepared)
        if logits is not None:
            rows.append(logits.clone())
        return logits

    engine.runner.launch = recording


def batches_with_cancels(engine, prompts, rounds, decode_calls):
    """``rounds`` times: submit the prompts, prefill, decode for some calls, cancel everything while
    the run is in flight, take what finished.  Returns the tokens of every call."""
    from tinyvllm_b200 import SamplingParams

    sampling = SamplingParams(max_new_tokens=200, ignore_eos=True)
    seen = []
    for _ in range(rounds):
        for prompt in prompts:
            engine.submit(prompt, sampling)
        while engine.scheduler.prefilling or engine.scheduler.waiting:
            seen.append(engine.step().tokens)
        for _ in range(decode_calls):
            seen.append(engine.step().tokens)
        for request_id in list(engine.scheduler.decoding):
            assert engine.cancel(request_id)
        engine.scheduler.take_finished()              # while the run's last steps are still in flight
    while engine.in_run:
        engine.step()
    engine.scheduler.take_finished()
    return seen


def test_batches_after_cancelled_runs_capture_and_replay_multi_entry_steps(model_folders):
    from tinyvllm_b200.engine.engine import Engine

    name = "e"                                       # head size 128: the tcgen05 kernels are on the path
    vocab = TINY_CONFIGS[name].vocab_size
    prompts = [random_tokens(vocab, n, 40 + n) for n in (150, 90, 60, 200)]

    # an engine that was dropped without close(): what it held is garbage that only the cyclic
    # collector frees, at a time of its choosing
    dropped = Engine.from_config(engine_config(model_folders[name], name))
    batches_with_cancels(dropped, prompts, 2, 3)
    del dropped

    results = {}
    for eager in (True, False):
        # both engines decode through the same graphs; one of them never captures a step
        engine = Engine.from_config(engine_config(model_folders[name], name))
        if eager:
            engine.runner.enable_step_graphs(0)
        engine.runner.CAPTURE_EVERY_STEPS = 1         # every shape that has come three times is captured
        rows = []
        record_logits(engine, rows)
        threshold = gc.get_threshold()
        gc.set_threshold(50)                          # collections all the time, as a busy host has them
        try:
            tokens = batches_with_cancels(engine, prompts, 5, 5)
        finally:
            gc.set_threshold(*threshold)
        if not eager:
            assert engine.runner._step_graph_limit > 0, "a capture failed and the runner fell back to eager"
            captured = engine.runner._step_graphs
            assert any(signature[0][4] > 1 for signature in captured), "no step of several entries was captured"
        engine.runner.manager.check()
        assert all(pool.free_count == pool.num_pages for pool in engine.runner.manager.pools)
        results[eager] = (tokens, rows)
        engine.close()
    # prompt steps (eager, captured, replayed) give the eager engine's logits bit for bit
    eager_rows, graph_rows = results[True][1], results[False][1]
    assert len(eager_rows) == len(graph_rows) > 0
    for index, (a, b) in enumerate(zip(eager_rows, graph_rows)):
        assert a.shape == b.shape and torch.equal(a, b), f"sampled step {index}"
    assert results[True][0] == results[False][0]


def test_a_failed_capture_leaves_the_engine_eager_and_right(model_folders, monkeypatch):
    """Graphs are an optimisation: when a step cannot be captured the step's eager logits stand and
    the runner stays eager."""
    from tinyvllm_b200 import SamplingParams
    from tinyvllm_b200.engine import step as step_module
    from tinyvllm_b200.engine.engine import Engine

    name = "e"
    vocab = TINY_CONFIGS[name].vocab_size
    prompts = [random_tokens(vocab, n, 90 + n) for n in (70, 70)]
    sampling = SamplingParams(max_new_tokens=3, ignore_eos=True)

    class Refused(RuntimeError):
        pass

    def refuse(*arguments, **keywords):
        raise Refused("no capture today")

    outputs = {}
    for broken in (False, True):
        engine = Engine.from_config(engine_config(model_folders[name], name, decode_run_steps=1))
        if broken:
            monkeypatch.setattr(step_module, "capture", refuse)
        got = []
        for _ in range(5):                            # the same shapes again and again: eager, capture, replay
            from tinyvllm_b200 import GenerateRequest

            got.append([tuple(o.output_token_ids) for o in
                        engine.generate([GenerateRequest(tuple(p), sampling) for p in prompts])])
        if broken:
            assert engine.runner._step_graph_limit == 0 and not engine.runner._step_graphs
        else:
            assert engine.runner._step_graphs
        outputs[broken] = got
        engine.close()
    assert outputs[False] == outputs[True]
    assert all(again == outputs[True][0] for again in outputs[True])


def test_request_ids_that_come_again_get_their_own_block_tables(model_folders):
    """The decode graphs keep each row's block table on the device from step to step and upload only
    what was added.  Two requests end in swapped order and their ids are used again for longer
    prompts: the new requests must not read the pages of the old ones."""
    from tinyvllm_b200 import SamplingParams
    from tinyvllm_b200.engine.engine import Engine

    name = "e"
    vocab = TINY_CONFIGS[name].vocab_size
    page = PAGE_SIZES[name]
    first = {0: random_tokens(vocab, page + 3, 1), 1: random_tokens(vocab, 2 * page + 5, 2)}
    again = {1: random_tokens(vocab, 3 * page + 7, 3), 0: random_tokens(vocab, 4 * page + 1, 4)}

    def run(eager: bool):
        engine = Engine.from_config(engine_config(model_folders[name], name, enforce_eager=eager,
                                                  decode_run_steps=1))
        outputs = []
        try:
            # request 1 ends first (fewer new tokens), then request 0
            engine.submit(first[0], SamplingParams(max_new_tokens=9, ignore_eos=True), request_id=0)
            engine.submit(first[1], SamplingParams(max_new_tokens=5, ignore_eos=True), request_id=1)
            done = {}
            while engine.has_unfinished():
                for output in engine.step().finished:
                    done[output.request_id] = tuple(output.output_token_ids)
            outputs.append(done)
            # the ids come again, in the other order, with longer prompts
            engine.submit(again[1], SamplingParams(max_new_tokens=8, ignore_eos=True), request_id=1)
            engine.submit(again[0], SamplingParams(max_new_tokens=8, ignore_eos=True), request_id=0)
            done = {}
            while engine.has_unfinished():
                for output in engine.step().finished:
                    done[output.request_id] = tuple(output.output_token_ids)
            outputs.append(done)
            if not eager:
                assert engine.graph_steps > 0
        finally:
            engine.close()
        return outputs

    assert run(False) == run(True)
