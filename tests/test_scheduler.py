"""The scheduler's decisions, with the model replaced by a function that makes up tokens.  No GPU."""

import random

import pytest

from tinyvllm_b200.cache.manager import CacheGroup, CacheManager
from tinyvllm_b200.engine.scheduler import Request, RequestStatus, Scheduler
from tinyvllm_b200.sampling.params import SamplingParams


def make(pages=64, page_size=4, seqs=4, budget=32, chunk=16, max_len=128, window=None, eos=(),
         reserve=(0, 0)):
    groups = [CacheGroup((0,), 1, 16, None)]
    if window is not None:
        groups.append(CacheGroup((1,), 1, 16, window))
    cache = CacheManager(groups, page_size, pages, seqs)
    scheduler = Scheduler(cache, max_num_seqs=seqs, max_num_batched_tokens=budget,
                          prefill_chunk_size=chunk, max_model_len=max_len, eos_token_ids=eos,
                          prefill_reserve_tokens=reserve[0], prefill_reserve_requests=reserve[1])
    return scheduler, cache


def request(rid, prompt_len, new=4, **sampling):
    return Request(rid, tuple(range(1, prompt_len + 1)), SamplingParams(max_new_tokens=new, **sampling))


def run_step(scheduler, token_of=lambda rid: 100 + rid):
    step = scheduler.schedule()
    if step is None:
        return None, []
    events = scheduler.commit(step, {i.request_id: token_of(i.request_id) for i in step.items if i.sample})
    scheduler.cache.check()
    return step, events


def drain(scheduler, token_of=lambda rid: 100 + rid, limit=10_000):
    steps = []
    while scheduler.has_unfinished():
        step, _ = run_step(scheduler, token_of)
        assert step is not None, "requests are unfinished but nothing can be scheduled"
        steps.append(step)
        assert len(steps) < limit
    return steps


def test_prompt_is_cut_under_the_chunk_and_token_budget():
    scheduler, _ = make(budget=20, chunk=8)
    scheduler.add(request(0, 19, new=2))
    counts = []
    while scheduler.has_unfinished():
        step, _ = run_step(scheduler)
        counts.append([(i.start, i.count, i.sample) for i in step.items])
    assert counts == [[(0, 8, False)], [(8, 8, False)], [(16, 3, True)], [(19, 1, True)]]
    done = scheduler.take_finished()
    assert len(done) == 1 and done[0].output_token_ids == [100, 100] and done[0].finish_reason == "length"
    assert done[0].computed_tokens == 20          # the last sampled token is never written


def test_decodes_come_first_and_share_the_step_with_prefill():
    scheduler, _ = make(budget=12, chunk=8, seqs=3)
    scheduler.add(request(0, 3, new=10))
    run_step(scheduler)                            # request 0 now decodes
    scheduler.add(request(1, 30, new=2))
    step, _ = run_step(scheduler)
    assert [(i.request_id, i.count) for i in step.items] == [(0, 1), (1, 8)]
    assert step.num_tokens <= 12
    step, _ = run_step(scheduler)
    assert [(i.request_id, i.start, i.count) for i in step.items] == [(0, 4, 1), (1, 8, 8)]


def test_token_budget_limits_the_whole_step():
    scheduler, _ = make(budget=10, chunk=10, seqs=4)
    for rid in range(3):
        scheduler.add(request(rid, 7, new=3))
    step, _ = run_step(scheduler)
    assert [(i.request_id, i.count) for i in step.items] == [(0, 7), (1, 3)]
    step, _ = run_step(scheduler)
    assert step.num_tokens <= 10 and step.items[0].request_id == 0 and step.items[0].count == 1


def test_finish_reasons_and_eos():
    scheduler, _ = make(eos=(7,))
    scheduler.add(request(0, 3, new=5))
    scheduler.add(request(1, 3, new=5, ignore_eos=True))
    scheduler.add(request(2, 3, new=0))
    assert [r.request_id for r in scheduler.take_finished()] == [2]        # nothing to generate
    tokens = iter([5, 7, 7, 9, 9, 9, 9, 9, 9, 9])
    while scheduler.has_unfinished():
        run_step(scheduler, token_of=lambda rid: 7 if rid == 0 and next(tokens) else 7)
    done = {r.request_id: r for r in scheduler.take_finished()}
    assert done[0].finish_reason == "stop" and done[0].output_token_ids == [7]
    assert done[1].finish_reason == "length" and len(done[1].output_token_ids) == 5
    assert done[0].status is RequestStatus.FINISHED


def test_max_model_len_stops_generation_and_refuses_long_prompts():
    scheduler, _ = make(max_len=12, pages=16)
    scheduler.add(request(0, 10, new=50))
    drain(scheduler)
    done = scheduler.take_finished()[0]
    assert len(done.prompt_token_ids) + len(done.output_token_ids) == 12
    with pytest.raises(ValueError, match="max_model_len"):
        scheduler.add(request(1, 13))
    with pytest.raises(ValueError, match="at least one token"):
        scheduler.add(request(2, 0))
    scheduler.add(request(3, 12, new=5))            # a prompt that fills the context ends at once
    assert scheduler.take_finished()[0].output_token_ids == []


def test_request_that_can_never_fit_is_refused_when_submitted():
    scheduler, _ = make(pages=4, page_size=4)
    with pytest.raises(ValueError, match="pages"):
        scheduler.add(request(0, 20, new=4))
    scheduler.add(request(1, 10, new=7))            # 10 + 7 - 1 = 16 tokens = 4 pages: fits exactly
    drain(scheduler)


def test_when_pages_run_out_requests_wait_and_nothing_is_preempted():
    """Admission promises a request its whole lifetime, so a running request never lacks a page."""
    scheduler, cache = make(pages=8, page_size=4, seqs=4, budget=64, chunk=64)
    for rid in range(3):
        scheduler.add(request(rid, 9, new=8))       # 16 written tokens = 4 pages each
    step, _ = run_step(scheduler)
    assert [i.request_id for i in step.items] == [0, 1]          # the third does not fit yet
    assert list(scheduler.waiting) == [2]
    seen_running = set()
    while 2 in scheduler.waiting:
        step, _ = run_step(scheduler)
        if 2 in scheduler.waiting:
            seen_running |= {i.request_id for i in step.items}
    assert seen_running == {0, 1}
    drain(scheduler)
    done = {r.request_id: r for r in scheduler.take_finished()}
    assert all(len(done[rid].output_token_ids) == 8 for rid in range(3))
    assert cache.free_pages(0) == 8


def test_a_large_waiter_does_not_block_smaller_ones():
    scheduler, _ = make(pages=8, page_size=4, seqs=4, budget=64, chunk=64)
    scheduler.add(request(0, 17, new=4))            # 20 tokens = 5 pages
    scheduler.add(request(1, 17, new=4))            # does not fit beside request 0
    scheduler.add(request(2, 5, new=4))             # 8 tokens = 2 pages: fits
    step, _ = run_step(scheduler)
    assert [i.request_id for i in step.items] == [0, 2]
    assert list(scheduler.waiting) == [1]
    drain(scheduler)
    assert sorted(r.request_id for r in scheduler.take_finished()) == [0, 1, 2]


def test_windowed_group_is_promised_less_than_a_full_one():
    scheduler, cache = make(pages=6, page_size=4, window=6, chunk=4, budget=16, seqs=2, max_len=64)
    probe = request(0, 10, new=12)                  # 21 written tokens: 6 pages in the full group
    assert scheduler.lifetime_pages(probe) == (6, 4)
    scheduler.add(probe)
    drain(scheduler)
    assert cache.free_pages(0) == 6 and cache.free_pages(1) == 6


def test_cancel_gives_everything_back():
    scheduler, cache = make()
    scheduler.add(request(0, 20, new=8))
    scheduler.add(request(1, 5, new=8))
    run_step(scheduler)
    assert scheduler.cancel(0) and not scheduler.cancel(0) and not scheduler.cancel(99)
    done = scheduler.take_finished()
    assert done[0].status is RequestStatus.ABORTED and done[0].finish_reason == "cancelled"
    drain(scheduler)
    assert cache.free_pages(0) == 64 and cache.slots.free_count == 4


def test_aborted_step_returns_its_pages():
    scheduler, cache = make()
    scheduler.add(request(0, 10, new=2))
    step = scheduler.schedule()
    assert cache.free_pages(0) < 64
    scheduler.abort_step(step)
    assert cache.free_pages(0) == 64
    cache.check()


def test_prefill_reservation_holds_room_back_from_decodes():
    scheduler, _ = make(seqs=4, budget=8, chunk=6, reserve=(4, 1))
    for rid in range(3):
        scheduler.add(request(rid, 1, new=20))
    run_step(scheduler)                             # three one-token prompts, all decode afterwards
    scheduler.add(request(3, 30, new=2))
    step, _ = run_step(scheduler)
    kinds = [(i.request_id, i.count) for i in step.items]
    assert kinds[:3] == [(0, 1), (1, 1), (2, 1)] and kinds[3][0] == 3 and kinds[3][1] >= 4


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_with_every_token_accounted_for(seed):
    rng = random.Random(seed)
    scheduler, cache = make(pages=rng.randrange(24, 60), page_size=rng.choice([2, 4, 8]),
                            seqs=rng.randrange(2, 6), budget=rng.randrange(8, 40), chunk=8,
                            window=rng.choice([None, 5, 12]), max_len=96)
    expected = {}
    submitted = 0
    steps = 0
    while submitted < 25 or scheduler.has_unfinished():
        if submitted < 25 and rng.random() < 0.4:
            prompt, new = rng.randrange(1, 40), rng.randrange(0, 20)
            try:
                scheduler.add(request(submitted, prompt, new=new))
                expected[submitted] = min(new, 96 - prompt)
            except ValueError:
                pass
            submitted += 1
        step, _ = run_step(scheduler)
        if step is not None:
            assert step.num_tokens <= scheduler.max_num_batched_tokens
            assert len(step.items) <= scheduler.max_num_seqs
            ids = [i.request_id for i in step.items]
            assert len(ids) == len(set(ids))
        steps += 1
        assert steps < 5000
    done = {}
    for r in scheduler.take_finished():
        done[r.request_id] = r
    # requests finished earlier were already taken by nobody: collect them from the loop above
    assert all(pool.free_count == pool.num_pages for pool in cache.pools)
    assert cache.slots.free_count == cache.slots.num_slots


# ------------------------------------------------------------------ decode runs
def test_decode_run_only_when_nothing_waits_and_as_long_as_every_request_may_go():
    scheduler, cache = make(pages=64, page_size=4, seqs=3, budget=32, chunk=16, max_len=40)
    scheduler.add(request(0, 5, new=10))
    scheduler.add(request(1, 7, new=3))
    assert scheduler.schedule_decode_run(4) is None            # nothing decodes yet
    run_step(scheduler)                                         # both prompts in one step, first tokens
    assert scheduler.decoding == [0, 1] and not scheduler.prefilling
    run = scheduler.schedule_decode_run(4)
    # request 1 has 2 of its 3 tokens left: the run is 2 steps long, one plan of 2 tokens each
    assert run is not None and run.steps == 2
    assert [(i.request_id, i.start, i.count) for i in run.items] == [(0, 5, 2), (1, 7, 2)]
    events = scheduler.commit_run(run, [{0: 50, 1: 60}, {0: 51, 1: 61}])
    cache.check()
    assert events == [(0, 50), (1, 60), (0, 51), (1, 61)]
    done = scheduler.take_finished()
    assert [r.request_id for r in done] == [1] and done[0].output_token_ids == [101, 60, 61]
    assert scheduler.requests[0].computed_tokens == 7 and scheduler.requests[0].output_token_ids == [100, 50, 51]
    # a newcomer waits: no run while it does, a plain step takes it in
    scheduler.add(request(2, 4, new=2))
    assert scheduler.schedule_decode_run(4) is None
    step, _ = run_step(scheduler)
    assert {i.request_id for i in step.items} == {0, 2}
    # the context limit bounds a run like the token limit does
    scheduler2, _ = make(max_len=12)
    scheduler2.add(request(0, 8, new=50))
    run_step(scheduler2)
    run = scheduler2.schedule_decode_run(8)
    assert run.steps == 3                                       # 9 tokens now, 12 at most
    scheduler2.commit_run(run, [{0: 1}, {0: 2}, {0: 3}])
    assert scheduler2.take_finished()[0].finish_reason == "length"
    assert scheduler2.schedule_decode_run(8) is None


def test_stop_token_inside_a_run_ends_the_request_there_and_frees_its_pages():
    scheduler, cache = make(pages=16, page_size=4, seqs=2, eos=(9,))
    scheduler.add(request(0, 6, new=20))
    scheduler.add(request(1, 3, new=20, ignore_eos=True))
    run_step(scheduler)
    free_before = cache.free_pages(0)
    run = scheduler.schedule_decode_run(4)
    assert run.steps == 4
    events = scheduler.commit_run(run, [{0: 5, 1: 9}, {0: 9, 1: 9}, {0: 7, 1: 9}, {0: 8, 1: 9}])
    cache.check()
    # request 0 stops at its second token; what the run made for it afterwards is dropped
    assert [e for e in events if e[0] == 0] == [(0, 5), (0, 9)]
    assert [e for e in events if e[1] == 9 and e[0] == 1] == [(1, 9)] * 4      # ignore_eos goes on
    done = scheduler.take_finished()
    assert [r.request_id for r in done] == [0] and done[0].finish_reason == "stop"
    assert done[0].output_token_ids == [100, 5, 9]
    assert not cache.is_open(0) and cache.is_open(1)
    assert cache.free_pages(0) >= free_before - 1               # request 0's pages are back
    with pytest.raises(ValueError, match="a run of"):
        run2 = scheduler.schedule_decode_run(3)
        scheduler.commit_run(run2, [{1: 1}])


def test_runs_and_single_steps_produce_the_same_requests():
    """Random workloads drained with and without runs: same outputs, no page lost."""
    for seed in range(6):
        outputs = []
        for run_steps in (1, 4):
            rng = random.Random(seed)
            scheduler, cache = make(pages=40, page_size=4, seqs=3, budget=24, chunk=8, max_len=64, eos=(7,))
            for rid in range(6):
                scheduler.add(request(rid, rng.randrange(1, 20), new=rng.randrange(1, 12)))
            counters = {}

            def token_of(rid):
                counters[rid] = counters.get(rid, 0) + 1
                return (rid * 31 + counters[rid] * 5) % 11          # sometimes the stop token 7

            guard = 0
            while scheduler.has_unfinished():
                run = scheduler.schedule_decode_run(run_steps) if run_steps > 1 else None
                if run is not None:
                    rows = [{i.request_id: token_of(i.request_id) for i in run.items} for _ in range(run.steps)]
                    scheduler.commit_run(run, rows)
                else:
                    run_step(scheduler, token_of)
                cache.check()
                guard += 1
                assert guard < 1000
            outputs.append({r.request_id: (tuple(r.output_token_ids), r.finish_reason)
                            for r in scheduler.take_finished()})
            assert all(pool.free_count == pool.num_pages for pool in cache.pools)
        # the made-up tokens depend on how often a request was asked, which a run does beyond a
        # request's end too: compare what does not (lengths up to the first stop token)
        for rid in outputs[0]:
            a, b = outputs[0][rid], outputs[1][rid]
            assert a[1] == b[1] and len(a[0]) == len(b[0]), (seed, rid, a, b)


def test_a_run_read_step_by_step_keeps_ended_requests_pages_until_it_ends():
    """begin_run / commit_run_step / end_run: the tokens of commit_run, but a request that ends
    inside the run (stop token, cancel) keeps its pages while later steps may still write them."""
    scheduler, cache = make(pages=32, page_size=4, seqs=3, eos=(9,))
    scheduler.add(request(0, 6, new=20))
    scheduler.add(request(1, 3, new=20, ignore_eos=True))
    scheduler.add(request(2, 5, new=20))
    run_step(scheduler)
    run = scheduler.schedule_decode_run(4)
    assert run.steps == 4
    scheduler.begin_run(run)
    with pytest.raises(RuntimeError, match="in flight"):
        scheduler.schedule()
    with pytest.raises(RuntimeError, match="in flight"):
        scheduler.schedule_decode_run(4)
    pages_of_0 = cache.block_table(0, 0)
    free = cache.free_pages(0)
    assert scheduler.commit_run_step(run, {0: 5, 1: 9, 2: 4}) == [(0, 5), (1, 9), (2, 4)]
    assert scheduler.commit_run_step(run, {0: 9, 1: 9, 2: 4}) == [(0, 9), (1, 9), (2, 4)]     # request 0 stops here
    assert scheduler.decoding == [1, 2] and run.closing == [0]
    assert cache.is_open(0) and cache.block_table(0, 0) == pages_of_0 and cache.free_pages(0) == free
    assert scheduler.cancel(2)                                       # cancelled while the run is in flight
    assert run.closing == [0, 2] and cache.is_open(2)
    done = scheduler.take_finished()                                 # reported at once all the same
    assert sorted((r.request_id, r.finish_reason) for r in done) == [(0, "stop"), (2, "cancelled")]
    assert scheduler.commit_run_step(run, {0: 1, 1: 9, 2: 1}) == [(1, 9)]                     # a third step was launched
    scheduler.end_run(run)                                           # the fourth never was
    cache.check()
    assert not cache.is_open(0) and not cache.is_open(2) and cache.is_open(1)
    assert cache.length(1) == 3 + 3 and scheduler.requests[1].computed_tokens == 6
    assert len(cache.block_table(1, 0)) == 2                         # 6 tokens: the page taken for the 7th went back
    assert cache.free_pages(0) == 32 - 2
    assert scheduler.run_in_flight is None
    step, _ = run_step(scheduler)
    assert [i.request_id for i in step.items] == [1]
    with pytest.raises(RuntimeError):
        scheduler.commit_run_step(run, {1: 1})


def test_runs_read_step_by_step_and_cut_short_produce_the_same_requests():
    """Random workloads drained with runs that are read step by step and cut short at random,
    against single steps: same lengths and reasons, no page lost."""
    for seed in range(8):
        outputs = []
        for streamed in (False, True):
            rng = random.Random(seed)
            cut = random.Random(seed + 100)
            scheduler, cache = make(pages=40, page_size=4, seqs=3, budget=24, chunk=8, max_len=64, eos=(7,),
                                    window=6 if seed % 2 else None)
            for rid in range(6):
                scheduler.add(request(rid, rng.randrange(1, 20), new=rng.randrange(1, 12)))
            counters = {}

            def token_of(rid):
                counters[rid] = counters.get(rid, 0) + 1
                return (rid * 31 + counters[rid] * 5) % 11          # sometimes the stop token 7

            guard = 0
            while scheduler.has_unfinished():
                run = scheduler.schedule_decode_run(6) if streamed else None
                if run is not None:
                    scheduler.begin_run(run)
                    launched = cut.randrange(1, run.steps + 1)
                    for _ in range(launched):
                        live = [i.request_id for i in run.items
                                if i.request_id in scheduler.requests and not scheduler.requests[i.request_id].status.terminal]
                        tokens = {i.request_id: 0 for i in run.items}
                        tokens.update({rid: token_of(rid) for rid in live})
                        scheduler.commit_run_step(run, tokens)
                    scheduler.end_run(run)
                else:
                    run_step(scheduler, token_of)
                cache.check()
                guard += 1
                assert guard < 1000
            outputs.append({r.request_id: (tuple(r.output_token_ids), r.finish_reason)
                            for r in scheduler.take_finished()})
            assert all(pool.free_count == pool.num_pages for pool in cache.pools)
        assert outputs[0] == outputs[1], seed


# ------------------------------------------------------------------------- arrivals
def arriving(rid, prompt_len, at, new=2):
    made = request(rid, prompt_len, new=new)
    made.arrival_ns = at
    return made


def test_requests_ahead_of_the_clock_are_kept_aside_and_join_in_time_order():
    scheduler, cache = make()
    scheduler.add(arriving(0, 3, at=300), now_ns=0)
    scheduler.add(arriving(1, 3, at=100), now_ns=0)
    scheduler.add(arriving(2, 3, at=100), now_ns=0)           # same time: the one submitted first goes first
    scheduler.add(arriving(3, 3, at=0), now_ns=0)             # already there
    assert list(scheduler.waiting) == [3] and scheduler.next_arrival_ns == 100
    assert scheduler.requests[0].status is RequestStatus.PENDING and scheduler.has_unfinished()
    assert scheduler.schedule(0).items[0].request_id == 3
    assert scheduler.advance(99) == 0 and scheduler.advance(100) == 2
    assert list(scheduler.waiting) == [1, 2] and scheduler.next_arrival_ns == 300
    assert scheduler.cancel(0, 150) and scheduler.next_arrival_ns is None
    assert scheduler.advance(1000) == 0                        # the cancelled one never joins
    with pytest.raises(ValueError, match="backwards"):
        scheduler.advance(999)
    finished = {r.request_id: r for r in scheduler.take_finished()}
    assert finished[0].finish_reason == "cancelled" and finished[0].status is RequestStatus.ABORTED
    cache.check()


def test_a_request_that_can_generate_nothing_ends_when_it_arrives():
    scheduler, _ = make()
    scheduler.add(arriving(0, 3, at=50, new=0), now_ns=0)
    assert scheduler.take_finished() == [] and scheduler.has_unfinished()
    scheduler.advance(60)
    done = scheduler.take_finished()
    assert [r.finish_reason for r in done] == ["length"] and done[0].finished_ns == 60
    assert not scheduler.has_unfinished()


def test_shutdown_gives_everything_back_and_refuses_more_work():
    scheduler, cache = make()
    scheduler.add(request(0, 9, new=6))
    scheduler.add(request(1, 5, new=6))
    run_step(scheduler)
    scheduler.add(arriving(2, 3, at=10**9), now_ns=0)
    step = scheduler.schedule()                                 # an open plan
    scheduler.shutdown(step.cache_plan)
    cache.check()
    assert cache.open_requests() == () and all(p.free_count == p.num_pages for p in cache.pools)
    assert not scheduler.has_unfinished() and scheduler.stopped
    with pytest.raises(RuntimeError, match="shut down"):
        scheduler.schedule()
    with pytest.raises(RuntimeError, match="shut down"):
        scheduler.add(request(5, 2))


def test_two_requests_with_one_id_differ_in_their_opening():
    _, cache = make()
    cache.open("a")
    first = cache.plan([("a", 3)])
    cache.commit(first)
    cache.close("a")
    cache.open("a")
    second = cache.plan([("a", 3)])
    assert first.entries[0].request_id == second.entries[0].request_id
    assert first.entries[0].opening != second.entries[0].opening
