"""The engine against the plain implementation, for every way of cutting the work.

Each test replays the same requests through the step function (the one that
generation uses) in float32 and in bfloat16 and compares every logit row with
the whole-sequence oracle of tests/plain_qwen3.py."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import replay_helpers as rh
from tiny_configs import PAGE_SIZES, TINY_CONFIGS, random_tokens

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]
LENGTHS = {
    "a": (1, 7, 19, 70, 300, 600),
    "b": (3, 16, 31, 50, 290, 700),
    "c": (5, 45, 130, 530),
    "d": (2, 64, 65, 200, 640),
    "e": (1, 33, 128, 300, 513),
}


def requests_of(name: str) -> dict:
    vocab = TINY_CONFIGS[name].vocab_size
    return {f"{name}{n}": random_tokens(vocab, n, 1000 + n) for n in LENGTHS[name]}


def make_runner(folder, dtype, page_size, pages, max_requests=8):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner

    model = Model(read_model_config(folder).to_spec(), device="cuda:0", dtype=dtype).load(folder)
    return StepRunner(model, page_size=page_size, num_pages=pages, max_requests=max_requests)


def peak_pages(steps, page_size):
    held, peak = {}, 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-n // page_size) for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


@pytest.fixture(scope="module")
def runners(model_folders):
    """One roomy runner per (configuration, dtype); every trace ends all its requests."""
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            pages = -(-3000 // PAGE_SIZES[name])
            cache[(name, dtype)] = make_runner(model_folders[name], dtype, PAGE_SIZES[name], pages)
        return cache[(name, dtype)]

    return get


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", sorted(TINY_CONFIGS))
def test_whole_requests(name, dtype, runners, model_folders):
    requests = requests_of(name)
    with torch.inference_mode():
        got = rh.run_steps(runners(name, dtype), rh.whole(requests))
    assert len(got) == sum(len(t) for t in requests.values())
    rh.compare(got, rh.oracle(model_folders[name], requests, dtype), dtype, what=f"whole {name}")


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", sorted(TINY_CONFIGS))
def test_last_32_tokens_one_by_one(name, dtype, runners, model_folders):
    requests = requests_of(name)
    with torch.inference_mode():
        got = rh.run_steps(runners(name, dtype), rh.tail_by_one(requests))
    rh.compare(got, rh.oracle(model_folders[name], requests, dtype), dtype, what=f"tail {name}")


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", sorted(TINY_CONFIGS))
def test_portions_of_changing_size(name, dtype, runners, model_folders):
    requests = requests_of(name)
    with torch.inference_mode():
        got = rh.run_steps(runners(name, dtype), rh.portions(requests, seed=7))
    assert len(got) == sum(len(t) for t in requests.values())
    rh.compare(got, rh.oracle(model_folders[name], requests, dtype), dtype, what=f"portions {name}")


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", sorted(TINY_CONFIGS))
def test_mixed_batches_with_scarce_pages(name, dtype, model_folders):
    """Up to four live requests, portions beside single tokens, and a pool exactly as
    large as the peak demand, so that pages of finished requests are taken again."""
    requests = requests_of(name)
    steps = rh.mixed(requests, seed=11)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len(e["tokens"]) == 1 for s in steps for e in s["entries"])
    page = PAGE_SIZES[name]
    pages = peak_pages(steps, page)
    assert pages * page < sum(len(t) for t in requests.values())     # the pool is used more than once
    runner = make_runner(model_folders[name], dtype, page, pages, max_requests=4)
    with torch.inference_mode():
        got = rh.run_steps(runner, steps)
    assert len(got) == sum(len(t) for t in requests.values())
    for pool in runner.manager.pools:
        assert pool.free_count == pool.num_pages
    rh.compare(got, rh.oracle(model_folders[name], requests, dtype), dtype, what=f"mixed {name}")


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_cutting_does_not_change_float_bits_beyond_rounding(dtype, runners, model_folders):
    """Whole against portions against mixed, engine against engine: the rows agree to rounding."""
    name = "b"
    requests = requests_of(name)
    runner = runners(name, dtype)
    with torch.inference_mode():
        base = rh.run_steps(runner, rh.whole(requests))
        cut = rh.run_steps(runner, rh.portions(requests, seed=3))
        mix = rh.run_steps(runner, rh.mixed(requests, seed=5))
    limit = 1e-5 if dtype == torch.float32 else 3e-2
    for key, row in base.items():
        scale = row.abs().max().item()
        assert (cut[key] - row).abs().max().item() <= limit * scale, key
        assert (mix[key] - row).abs().max().item() <= limit * scale, key


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_trace_run_program(dtype_name, model_folders, tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and 'done' lines out."""
    name = "b"
    dtype = getattr(torch, dtype_name)
    requests = {k: v for k, v in list(requests_of(name).items())[:5]}
    steps = rh.mixed(requests, seed=13)
    out_dir = tmp_path / "out"
    text = "".join(json.dumps(step) + "\n" for step in steps)
    result = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_folders[name]),
         "--dtype", dtype_name, "--out", str(out_dir), "--max-tokens", str(rh.live_token_need(steps))],
        input=text, capture_output=True, text=True, timeout=900,
        env={**os.environ, "PYTHONPATH": ""})
    assert result.returncode == 0, result.stderr[-2000:]
    assert result.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    got = rh.read_trace_output(steps, out_dir, TINY_CONFIGS[name].vocab_size)
    rh.compare(got, rh.oracle(model_folders[name], requests, dtype), dtype, what="trace_run")


def test_a_lone_long_request_is_cut_over_several_clusters(model_folders, monkeypatch):
    """From a length on (brought down to 96 tokens here) a request that decodes alone has its keys
    cut over several clusters per kv head: eagerly, and in the decode graph of one row that long
    requests have for themselves; shorter ones keep the other graph, and one that grows past the
    length changes over."""
    from tinyvllm_b200.engine.graphs import DecodeGraphs
    from tinyvllm_b200.engine.step import StepEntry
    from tinyvllm_b200.ops import attention as attention_ops
    from tinyvllm_b200.ops import kernels
    from tinyvllm_b200.sampling.params import SamplingParams

    monkeypatch.setattr(attention_ops, "FAR_FROM_KEYS", 96)
    name, dtype = "e", torch.bfloat16
    vocab = TINY_CONFIGS[name].vocab_size
    requests = {"long": random_tokens(vocab, 400, 77), "short": random_tokens(vocab, 60, 78),
                "grows": random_tokens(vocab, 104, 79)}
    tail = 24
    seen = []
    real = kernels.attention_decode

    def watched(*args, far_groups=1, **kwargs):
        seen.append(far_groups)
        return real(*args, far_groups=far_groups, **kwargs)

    monkeypatch.setattr(kernels, "attention_decode", watched)
    for use_graphs in (False, True):
        runner = make_runner(model_folders[name], dtype, PAGE_SIZES[name], 40 if use_graphs else 41)
        graphs = None
        if use_graphs:
            graphs = DecodeGraphs(runner, [1, 2], max_model_len=runner.max_model_len)
            assert graphs.far_bucket is not None
            graphs.capture()
        got = {}
        with torch.inference_mode():
            for rid, tokens in requests.items():
                runner.open(rid)
                runner.run([StepEntry(rid, tuple(tokens[:-tail]), ())])
                for step in range(tail):
                    position = len(tokens) - tail + step
                    far = position + 1 >= 96       # tokens of the request with its new one
                    entries = [StepEntry(rid, (tokens[position],), (0,))]
                    seen.clear()
                    if graphs is None:
                        logits = runner.run(entries)
                        # every layer's launch says how it was cut
                        assert seen and all((groups > 1) == far for groups in seen)
                    else:
                        plan = runner.plan(entries)
                        prepared = graphs.prepare(plan, entries, [SamplingParams()], [0])
                        assert (prepared[0] is graphs.far_bucket) == far
                        _, logits = graphs.launch(prepared, plan)
                        runner.manager.commit(plan)
                    got[(rid, position)] = logits[0].float().cpu().clone()
                runner.close(rid)
        positions = {rid: {p for (r, p) in got if r == rid} for rid in requests}
        expected = rh.oracle(model_folders[name], requests, dtype, positions=positions)
        rh.compare(got, expected, dtype, what=f"lone long request, graphs {use_graphs}")


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_steps_replayed_as_graphs_give_the_eager_logits(dtype, model_folders):
    """A step whose signature keeps coming back is captured at its third occurrence and replayed
    from the fourth: the logits of every occurrence are those of a runner that never captures, bit
    for bit, also with other steps in between and with pages that are used again."""
    from tinyvllm_b200.engine.step import StepEntry

    name = "e"
    vocab = TINY_CONFIGS[name].vocab_size
    eager = make_runner(model_folders[name], dtype, PAGE_SIZES[name], 24, max_requests=4)
    graphed = make_runner(model_folders[name], dtype, PAGE_SIZES[name], 24, max_requests=4)
    graphed.enable_step_graphs(limit=2)
    # capture eagerly: at the second occurrence, any number of captures in a row, any graph may go
    graphed.CAPTURE_AT_OCCURRENCE, graphed.CAPTURE_EVERY_STEPS, graphed.KEEP_FOR_STEPS = 2, 0, 0
    shapes = [(150, 3), (150, 3), (40, 2), (150, 3), (150, 3), (40, 2), (40, 2), (7, 1), (150, 3), (7, 1), (7, 1)]
    for step, (count, wanted) in enumerate(shapes):
        tokens = tuple(random_tokens(vocab, count, 1000 + step))
        want = tuple(range(count - wanted, count))
        results = []
        for r in (eager, graphed):
            r.open(step)
            results.append(r.run([StepEntry(step, tokens, want)]).clone())
            # two decoded tokens behind the prompt: the cache the step left is the eager one's
            for extra in range(2):
                results.append(r.run([StepEntry(step, (tokens[extra],), (0,))]).clone())
            r.close(step)
        half = len(results) // 2
        for a, b in zip(results[:half], results[half:]):
            assert torch.equal(a, b), f"step {step}"
    assert len(graphed._step_graphs) == 2          # the limit holds: the third shape took the place of the
    assert any(sig[0][0] == 7 for sig in graphed._step_graphs)      # one unused for longest


def test_steps_are_captured_sparingly(model_folders):
    """A capture costs about two steps: a shape is captured at its third occurrence, captures keep a
    distance of some steps, and a graph in use is not thrown out for a newcomer."""
    from tinyvllm_b200.engine.step import StepEntry, StepRunner

    name = "e"
    vocab = TINY_CONFIGS[name].vocab_size
    runner = make_runner(model_folders[name], torch.bfloat16, PAGE_SIZES[name], 64, max_requests=4)
    runner.enable_step_graphs(limit=1)

    def step(count, index):
        runner.open(index)
        runner.run([StepEntry(index, tuple(random_tokens(vocab, count, index)), (count - 1,))])
        runner.close(index)

    for index in range(2):
        step(100, index)
    assert not runner._step_graphs                              # seen twice: not yet
    step(100, 2)
    assert len(runner._step_graphs) == 1                        # the third time
    (first,) = runner._step_graphs
    for index in range(3, 3 + StepRunner.CAPTURE_EVERY_STEPS + 4):
        step(50, index)                                         # another shape, again and again
    assert list(runner._step_graphs) == [first]                 # the graph was replayed too recently to go
    runner.KEEP_FOR_STEPS = 4
    for index in range(40, 46):
        step(50, index)
    assert list(runner._step_graphs) != [first] and len(runner._step_graphs) == 1
