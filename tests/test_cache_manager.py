"""The cache manager under random orders of requests: no page lost, held twice or freed twice;
pages come back when a request ends or a window has passed them, and are used again.  No GPU."""

import random

import pytest

from tinyvllm_b200.cache.manager import CacheError, CacheGroup, CacheManager, PagePool, SlotPool


def manager(pages=16, page_size=4, slots=4, window=None, groups=None):
    groups = groups or [CacheGroup((0, 1), 2, 16, window)]
    return CacheManager(groups, page_size, pages, slots)


def test_pool_take_give_and_double_free():
    pool = PagePool(4)
    a = pool.take(3, "x")
    assert sorted(a) == [0, 1, 2] and pool.free_count == 1
    assert pool.take(2, "y") is None and pool.free_count == 1          # nothing changes
    pool.give(a[:1], "x")
    with pytest.raises(CacheError, match="freed twice"):
        pool.give(a[:1], "x")
    with pytest.raises(CacheError, match="held by"):
        pool.give(a[1:2], "y")
    assert pool.take(1, "z") == a[:1]                                  # the last freed page is reused first
    pool.check()


def test_slots():
    slots = SlotPool(2)
    a, b = slots.take(), slots.take()
    assert {a, b} == {0, 1} and slots.take() is None
    slots.give(a)
    with pytest.raises(CacheError):
        slots.give(a)
    assert slots.take() == a


def test_plan_commit_tables_and_slots():
    m = manager(pages=8, page_size=4)
    m.open("r")
    plan = m.plan([("r", 6)])
    entry = plan.entries[0]
    assert entry.start == 0 and entry.count == 6 and entry.fresh_state
    table = list(entry.tables[0])                   # a copy: the plan hands out the live table
    assert len(table) == 2
    assert entry.slots[0] == tuple(table[p // 4] * 4 + p % 4 for p in range(6))
    assert m.length("r") == 0                       # not yet committed
    m.commit(plan)
    assert m.length("r") == 6
    plan = m.plan([("r", 3)])                       # 6..8: second page has room for 6, 7; 8 needs a new one
    assert len(plan.entries[0].tables[0]) == 3 and not plan.entries[0].fresh_state
    assert plan.entries[0].tables[0][:2] == table
    m.commit(plan)
    m.check()
    m.close("r")
    assert m.free_pages(0) == 8
    m.check()


def test_the_next_request_gets_neighbouring_pages_in_rising_order():
    """A fresh pool hands out rising page numbers, and what a request gives back (at its end, or
    when a plan is rolled back) comes out again in the same order: the prefill attention copies
    neighbouring pages several at a time."""
    m = manager(pages=12, page_size=4)
    m.open("a")
    plan = m.plan([("a", 22)])
    first = list(plan.entries[0].tables[0])
    assert first == list(range(first[0], first[0] + 6))
    m.commit(plan)
    m.open("b")
    planned = m.plan([("b", 9)])
    held = list(planned.entries[0].tables[0])
    m.rollback(planned)
    planned = m.plan([("b", 9)])
    assert list(planned.entries[0].tables[0]) == held == list(range(held[0], held[0] + 3))
    m.commit(planned)
    m.close("a")
    m.open("c")
    plan = m.plan([("c", 24)])
    assert list(plan.entries[0].tables[0]) == first
    m.check()


def test_commit_of_what_was_written_gives_the_rest_back():
    """A plan for several tokens per request (a run of decode steps) that ended early."""
    m = manager(pages=12, page_size=4)
    m.open("a"), m.open("b")
    m.commit(m.plan([("a", 7), ("b", 2)]))
    plan = m.plan([("a", 6), ("b", 6)])              # a: 7..12 (two more pages), b: 2..7 (one more)
    assert m.free_pages(0) == 12 - 4 - 2
    kept = m.block_table("a", 0)[:3]
    with pytest.raises(CacheError, match="more tokens than were planned"):
        m.commit(plan, written=7)
    m.commit(plan, written=2)                        # a: 9 tokens = 3 pages, b: 4 tokens = 1 page
    assert m.length("a") == 9 and m.length("b") == 4
    assert m.block_table("a", 0) == kept and len(m.block_table("b", 0)) == 1
    assert m.free_pages(0) == 12 - 3 - 1
    m.check()
    m.commit(m.plan([("a", 1), ("b", 1)]))           # and on it goes
    assert m.length("a") == 10 and len(m.block_table("b", 0)) == 2
    m.close("a"), m.close("b")
    m.check()
    assert m.free_pages(0) == 12


def test_all_or_nothing_and_rollback():
    m = manager(pages=4, page_size=4)
    m.open("a"), m.open("b")
    before = m.free_pages(0)
    assert m.plan([("a", 9), ("b", 8)]) is None     # 3 + 2 pages > 4
    assert m.free_pages(0) == before and m.block_table("a", 0) == ()
    plan = m.plan([("a", 9)])
    assert m.free_pages(0) == 1
    with pytest.raises(CacheError, match="has not ended"):
        m.plan([("a", 1)])
    with pytest.raises(CacheError, match="has not ended"):
        m.close("a")
    m.rollback(plan)
    assert m.free_pages(0) == 4 and m.length("a") == 0 and m.block_table("a", 0) == ()
    with pytest.raises(CacheError):
        m.commit(plan)
    m.check()


def test_errors():
    m = manager(slots=1)
    m.open("a")
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    with pytest.raises(CacheError, match="no state slot"):
        m.open("b")
    with pytest.raises(CacheError, match="not open"):
        m.plan([("zz", 1)])
    with pytest.raises(CacheError, match="twice"):
        m.plan([("a", 1), ("a", 1)])
    with pytest.raises(CacheError, match="at least one"):
        m.plan([("a", 0)])
    m.close("a")
    with pytest.raises(CacheError, match="not open"):
        m.close("a")


def test_window_gives_pages_back_and_keeps_what_queries_need():
    window, size = 6, 4
    m = manager(pages=8, page_size=size, window=window)
    m.open("r")
    length = 0
    for count in (5, 1, 1, 7, 1, 1, 1, 2, 9):
        plan = m.plan([("r", count)])
        assert plan is not None
        m.commit(plan)
        length += count
        table = m.block_table("r", 0)
        first_needed = max(0, length - window + 1)      # the next query stands at `length`
        for index, page in enumerate(table):
            covered_end = (index + 1) * size
            if covered_end <= first_needed:
                assert page == -1, (length, index)
            else:
                assert page >= 0, (length, index)
        m.check()
    held = sum(1 for page in m.block_table("r", 0) if page >= 0)
    assert held <= m.peak_pages(0, length, 9)
    assert m.free_pages(0) == 8 - held
    m.close("r")
    assert m.free_pages(0) == 8


def test_peak_pages_bounds_every_schedule():
    rng = random.Random(0)
    for _ in range(200):
        size = rng.choice([1, 3, 4, 8, 16])
        window = rng.choice([1, 2, 5, 16, 40])
        chunk = rng.choice([1, 2, 7, 32])
        m = manager(pages=200, page_size=size, window=window)
        m.open("r")
        total = rng.randrange(1, 150)
        done, worst = 0, 0
        while done < total:
            count = min(rng.randrange(1, chunk + 1), total - done)
            plan = m.plan([("r", count)])
            worst = max(worst, sum(1 for p in m.block_table("r", 0) if p >= 0))
            m.commit(plan)
            done += count
        assert worst <= m.peak_pages(0, total, chunk), (size, window, chunk, total)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    groups = [CacheGroup((0, 2), 2, 16, None), CacheGroup((1,), 2, 16, rng.choice([3, 9, 20]))]
    m = CacheManager(groups, rng.choice([2, 4, 8]), [rng.randrange(6, 30), rng.randrange(6, 30)], 5)
    live: dict[int, int] = {}
    next_id = 0
    reused, seen_pages = False, set()
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            m.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.85 and live:
            chosen = rng.sample(sorted(live), rng.randrange(1, len(live) + 1))
            appends = [(rid, rng.randrange(1, 12)) for rid in chosen]
            free_before = [m.free_pages(g) for g in range(2)]
            plan = m.plan(appends)
            if plan is None:
                assert [m.free_pages(g) for g in range(2)] == free_before
                victim = rng.choice(sorted(live))          # make room: a request ends
                m.close(victim)
                del live[victim]
            elif rng.random() < 0.15:
                m.rollback(plan)
                assert [m.free_pages(g) for g in range(2)] == free_before
            elif rng.random() < 0.2:
                # a run of steps cut short: every entry wrote only its first tokens
                written = rng.randrange(0, min(count for _, count in appends) + 1)
                m.commit(plan, written=written)
                for rid, _ in appends:
                    live[rid] += written
                    assert m.length(rid) == live[rid]
                    assert len(m.block_table(rid, 0)) == -(-live[rid] // m.page_size)
                if written == 0:
                    assert [m.free_pages(g) for g in range(2)] == free_before
            else:
                for entry in plan.entries:
                    for table in entry.tables:
                        for page in table[-2:]:
                            if page >= 0:
                                reused |= page in seen_pages
                                seen_pages.add(page)
                m.commit(plan)
                for rid, count in appends:
                    live[rid] += count
                    assert m.length(rid) == live[rid]
        elif live:
            victim = rng.choice(sorted(live))
            m.close(victim)
            del live[victim]
        m.check()
    for rid in list(live):
        m.close(rid)
    m.check()
    assert all(pool.free_count == pool.num_pages for pool in m.pools)
    assert m.slots.free_count == 5
    assert reused
