"""The engine's loop over runs of decode steps, without a GPU: model, graphs and sampler are
stand-ins that make a request's next token a function of the request and the position, so that
what the engine does with runs (launching ahead, reading step by step, ending a run early for a
newcomer, a stop token or a cancel) can be compared with one step at a time."""

import random

import pytest

from tinyvllm_b200.cache.manager import CacheGroup, CacheManager
from tinyvllm_b200.engine.engine import Engine
from tinyvllm_b200.engine.scheduler import Scheduler
from tinyvllm_b200.sampling.params import SamplingParams

VOCAB = 50
STOP = 7


def token_at(request_id, position: int) -> int:
    """The token a request gets after the token at ``position``."""
    return (request_id * 13 + position * 7 + (position * position) % 5) % VOCAB


class Tokens:
    """Stands for a device tensor of sampled ids."""

    def __init__(self, values):
        self.values = list(values)

    def tolist(self):
        return list(self.values)


class StandInRunner:
    vocab_size = VOCAB

    def __init__(self, manager):
        self.manager = manager
        self.calls = 0
        self.fail_prepare = 0           # so many calls of prepare raise
        self.fail_launch = False

    def prepare(self, entries, plan):              # the host half: nothing runs yet
        if self.fail_prepare:
            self.fail_prepare -= 1
            raise RuntimeError("lowering failed")
        return entries, plan

    def launch(self, prepared):                    # the device half
        entries, plan = prepared
        if self.fail_launch:
            raise RuntimeError("the model failed")
        self.calls += 1
        by_id = {p.request_id: p for p in plan.entries}
        rows = [token_at(e.request_id, by_id[e.request_id].start + len(e.tokens) - 1) for e in entries if e.want]
        return Tokens(rows) if rows else None

    def forward(self, entries, plan):
        return self.launch(self.prepare(entries, plan))


class StandInSampler:
    def sample(self, logits, params, draws):
        return logits


class StandInFlight:
    def __init__(self, planned, steps, log):
        self.planned, self.steps, self.log = planned, steps, log
        self.launched = self.read_steps = 0
        self.bucket = object()

    fail_read_at = None                 # the read of this step raises

    def launch(self):
        assert self.launched < self.steps
        self.launched += 1
        self.log.append(("launch", self.launched - self.read_steps))

    def read(self):
        assert self.read_steps < self.launched
        if self.fail_read_at == self.read_steps:
            raise RuntimeError("the device did not answer")
        tokens = [token_at(p.request_id, p.start + self.read_steps) for p in self.planned]
        self.read_steps += 1
        return tokens


class StandInGraphs:
    def __init__(self, largest=8):
        self.largest = largest
        self.log = []
        self.forgotten = 0

    def bucket_for(self, rows):
        return object() if 0 < rows <= self.largest else None

    def prepare(self, plan, entries, params, draws):
        return None                     # single steps take the eager path of the stand-in runner

    def start_run(self, plan, first_tokens, params, draws, steps):
        self.log.append(("run", len(first_tokens), steps))
        return StandInFlight(plan.entries, steps, self.log)

    def forget_tables(self, bucket):
        self.forgotten += 1


def make_engine(run_steps, pages=64, seqs=4, **engine_arguments):
    cache = CacheManager([CacheGroup((0,), 1, 16, None)], 4, pages, seqs)
    scheduler = Scheduler(cache, max_num_seqs=seqs, max_num_batched_tokens=32, prefill_chunk_size=16,
                          max_model_len=96, eos_token_ids=(STOP,))
    graphs = StandInGraphs()
    engine = Engine(StandInRunner(cache), scheduler, graphs=graphs, decode_run_steps=run_steps, **engine_arguments)
    engine.sampler = StandInSampler()
    return engine, cache, graphs


def drive(engine, script, seed):
    """Run ``script`` = {call index: [("submit", id, prompt length, new tokens, ignore_eos) | ("cancel", id)]}
    to the end; outputs by request id."""
    rng = random.Random(seed)
    outputs, streamed, call = {}, {}, 0
    pending = dict(script)
    while engine.has_unfinished() or pending:
        for action in pending.pop(call, []):
            if action[0] == "submit":
                _, rid, length, new, ignore = action
                prompt = [rng.randrange(VOCAB) for _ in range(length)]
                engine.submit(prompt, SamplingParams(max_new_tokens=new, ignore_eos=ignore), request_id=rid)
            else:
                engine.cancel(action[1])
        events = engine.step()
        for rid, token in events.tokens:
            streamed.setdefault(rid, []).append(token)
        for done in events.finished:
            outputs[done.request_id] = (tuple(done.output_token_ids), done.finish_reason)
        call += 1
        assert call < 2000
    for rid, (tokens, _) in outputs.items():
        assert tuple(streamed.get(rid, ())) == tokens          # every token was also reported as an event
    return outputs


def test_runs_read_step_by_step_give_what_single_steps_give():
    reasons = set()
    for seed in range(12):
        rng = random.Random(100 + seed)
        script = {}
        for rid in range(7):
            script.setdefault(rng.randrange(0, 30), []).append(
                ("submit", rid, rng.randrange(1, 30), rng.randrange(1, 40), rng.random() < 0.5))
        results = []
        for run_steps in (1, 4, 32):
            engine, cache, graphs = make_engine(run_steps)
            results.append(drive(engine, script, seed))
            assert engine._run is None and engine.scheduler.run_in_flight is None
            cache.check()
            assert all(pool.free_count == pool.num_pages for pool in cache.pools)
            if run_steps > 1:
                assert any(entry[0] == "run" for entry in graphs.log)
                # never more than two steps launched and not read
                assert max(entry[1] for entry in graphs.log if entry[0] == "launch") <= Engine.RUN_AHEAD
            engine.close()
        assert results[0] == results[1] == results[2], seed
        reasons |= {reason for _, reason in results[0].values()}
    assert reasons == {"stop", "length"}             # both ways of ending occurred


def test_a_newcomer_and_a_cancel_end_a_run_after_what_was_launched():
    engine, cache, graphs = make_engine(32)
    engine.submit([1, 2, 3], SamplingParams(max_new_tokens=60, ignore_eos=True), request_id=0)
    engine.submit([4, 5], SamplingParams(max_new_tokens=60, ignore_eos=True), request_id=1)
    engine.step()                                   # both prompts, first tokens
    assert engine._run is None
    first = engine.step()                           # a run of 32 starts: two steps launched, one read
    assert engine._run is not None and [rid for rid, _ in first.tokens] == [0, 1]
    run, flight, _ = engine._run
    assert (run.steps, flight.launched, flight.read_steps) == (32, 2, 1)
    engine.step()
    assert (flight.launched, flight.read_steps) == (3, 2)
    engine.submit([9] * 5, SamplingParams(max_new_tokens=3, ignore_eos=True), request_id=2)
    ended = engine.step()                           # nothing more is launched; what was is read; the run ends
    assert engine._run is None and flight.launched == 3 and flight.read_steps == 3
    assert [rid for rid, _ in ended.tokens] == [0, 1]
    assert graphs.forgotten == 1
    assert cache.length(0) == 3 + 3 and cache.length(1) == 2 + 3          # the prompt and three decoded tokens written
    assert len(cache.block_table(0, 0)) == 2                               # pages for 32 more tokens went back
    mixed = engine.step()                           # the newcomer's prompt beside the others' next tokens
    assert sorted(rid for rid, _ in mixed.tokens) == [0, 1, 2]
    # a cancel inside the next run
    while engine._run is None:
        engine.step()
    run, flight, _ = engine._run
    assert engine.cancel(1)
    assert cache.is_open(1)                         # its pages stay until the run has ended
    after = engine.step()
    assert engine._run is None and not cache.is_open(1)
    assert [o.request_id for o in after.finished if o.finish_reason == "cancelled"] == [1]
    assert all(rid != 1 for rid, _ in after.tokens)
    while engine.has_unfinished():
        engine.step()
    cache.check()
    assert all(pool.free_count == pool.num_pages for pool in cache.pools)


# ---------------------------------------------------------------- failures (made on the host)
def all_pages_free(cache) -> bool:
    cache.check()
    return all(pool.free_count == pool.num_pages for pool in cache.pools)


def test_a_failure_while_lowering_gives_the_pages_back_and_the_engine_goes_on():
    """Nothing of the step was launched (tinyvllm/engine.py:354-365): the plan is rolled back, the
    requests keep their places, the next call runs them."""
    engine, cache, _ = make_engine(1)
    engine.submit(list(range(1, 20)), SamplingParams(max_new_tokens=4, ignore_eos=True), request_id=0)
    engine.runner.fail_prepare = 1
    with pytest.raises(RuntimeError, match="lowering failed"):
        engine.step()
    cache.check()
    assert cache.is_open(0) and cache.length(0) == 0 and cache.block_table(0, 0) == ()
    assert engine._failed is None
    outputs = {}
    while engine.has_unfinished():
        for done in engine.step().finished:
            outputs[done.request_id] = done
    assert outputs[0].finish_reason == "length" and len(outputs[0].output_token_ids) == 4
    stats = engine.stats()
    assert stats["lowering_failures"] == 1 and stats["prompt_tokens"] == 19 and stats["decode_tokens"] == 3
    assert stats["pages_free"] == stats["pages_total"] and stats["decoding"] == 0
    # the same tokens as an engine that never failed
    other, _, _ = make_engine(1)
    other.submit(list(range(1, 20)), SamplingParams(max_new_tokens=4, ignore_eos=True), request_id=0)
    expected = {}
    while other.has_unfinished():
        for done in other.step().finished:
            expected[done.request_id] = done
    assert outputs[0].output_token_ids == expected[0].output_token_ids
    assert all_pages_free(cache)


def test_a_failure_after_launch_stops_the_engine_and_loses_no_page():
    """The model raised (tinyvllm/engine.py:367-387, :543-564): fail-stop."""
    engine, cache, _ = make_engine(1)
    engine.submit([1, 2, 3], SamplingParams(max_new_tokens=8, ignore_eos=True), request_id=0)
    engine.step()
    engine.submit([4] * 9, SamplingParams(max_new_tokens=8, ignore_eos=True), request_id=1)
    engine.runner.fail_launch = True
    with pytest.raises(RuntimeError, match="the model failed"):
        engine.step()
    assert engine._failed is not None and "the model failed" in engine._failed
    assert all_pages_free(cache) and cache.open_requests() == ()
    for call in (engine.step, lambda: engine.submit([1], None), lambda: engine.cancel(0),
                 lambda: engine.generate([])):
        with pytest.raises(RuntimeError, match="stopped after a failed step"):
            call()


def test_a_failed_read_inside_a_run_stops_the_engine_and_loses_no_page():
    engine, cache, graphs = make_engine(32)
    engine.submit([1, 2, 3], SamplingParams(max_new_tokens=60, ignore_eos=True), request_id=0)
    engine.submit([4, 5], SamplingParams(max_new_tokens=60, ignore_eos=True), request_id=1)
    engine.step()
    engine.step()                                    # the run starts
    _, flight, _ = engine._run
    flight.fail_read_at = 2
    engine.step()
    with pytest.raises(RuntimeError, match="did not answer"):
        engine.step()
    assert engine._failed is not None and engine._run is None and engine.scheduler.run_in_flight is None
    assert all_pages_free(cache) and cache.open_requests() == ()
    with pytest.raises(RuntimeError, match="stopped after a failed step"):
        engine.step()


def test_a_run_that_cannot_start_is_rolled_back():
    engine, cache, graphs = make_engine(32)
    engine.submit([1, 2, 3], SamplingParams(max_new_tokens=60, ignore_eos=True), request_id=0)
    engine.step()
    held = len(cache.block_table(0, 0))

    def refuse(*arguments):
        raise RuntimeError("no pinned memory")

    graphs.start_run, start_run = refuse, graphs.start_run
    with pytest.raises(RuntimeError, match="no pinned memory"):
        engine.step()
    cache.check()
    assert engine._failed is None and len(cache.block_table(0, 0)) == held
    graphs.start_run = start_run
    while engine.has_unfinished():
        engine.step()
    assert all_pages_free(cache)


# ------------------------------------------------------------------- arrivals and the clock
class Clock:
    def __init__(self):
        self.now = 0
        self.slept = []

    def __call__(self):
        return self.now

    def sleep(self, seconds):
        self.slept.append(seconds)
        self.now += int(round(seconds * 1e9))


def test_requests_take_part_from_their_arrival_time_on():
    clock = Clock()
    engine, cache, _ = make_engine(1, clock=clock, sleep=clock.sleep)
    ms = 1_000_000
    for rid in range(4):                             # 20 ms apart, submitted all at once
        engine.submit([rid + 1] * 5, SamplingParams(max_new_tokens=3, ignore_eos=True), request_id=rid,
                      arrival_ns=rid * 20 * ms)
    assert engine.scheduler.next_arrival_ns == 20 * ms
    first = engine.step(now_ns=0)
    assert [rid for rid, _ in first.tokens] == [0]
    assert engine.scheduler.requests[1].status.value == "pending"
    events = engine.step(now_ns=20 * ms)
    with pytest.raises(ValueError, match="backwards"):
        engine.step(now_ns=19 * ms)
    assert sorted(rid for rid, _ in events.tokens) == [0, 1]
    assert engine.cancel(3) and engine.scheduler.next_arrival_ns == 40 * ms
    done = {}
    now = 20 * ms
    while engine.has_unfinished():
        now += 10 * ms
        for output in engine.step(now_ns=now).finished:
            done[output.request_id] = output
    assert sorted(done) == [0, 1, 2, 3] and done[3].finish_reason == "cancelled"
    assert done[2].admitted_ns >= 40 * ms and done[2].arrival_ns == 40 * ms
    assert done[1].first_token_ns == 20 * ms
    assert all_pages_free(cache)


def test_generate_sleeps_until_the_next_arrival():
    from tinyvllm_b200.engine.engine import GenerateRequest

    clock = Clock()
    engine, cache, _ = make_engine(1, clock=clock, sleep=clock.sleep)
    sampling = SamplingParams(max_new_tokens=2, ignore_eos=True)
    outputs = engine.generate([GenerateRequest((1, 2, 3), sampling, arrival_ns=0),
                               GenerateRequest((4, 5), sampling, arrival_ns=50_000_000)])
    assert [len(o.output_token_ids) for o in outputs] == [2, 2]
    assert clock.slept and abs(sum(clock.slept) - 0.05) < 1e-9      # idle once, until the second arrived
    assert outputs[1].admitted_ns >= 50_000_000
    assert all_pages_free(cache)
