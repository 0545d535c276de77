"""Host side of the cache: pages, block tables and state slots.

Keys and values live in pages of ``page_size`` tokens.  Runs of the model with
the same need (heads, head size, window) form a *group*; a group has a page
pool of its own and every request has one block table per group, which all
runs of the group share.  A group with a window gives a page back as soon as
every token in it lies before the window of all queries still to come; its
block-table entry then reads -1.  Every request also holds one *state slot*,
an index into per-run arenas of fixed-size state (empty for dense attention).

A step is a transaction: :meth:`CacheManager.plan` takes the pages that all
entries of the step need or changes nothing and returns ``None``;
:meth:`commit` makes the new lengths count and releases pages a window has
passed; :meth:`rollback` undoes a plan that did not run.

The reference keeps one group, block states with generations and a
reserve/commit protocol (tinyvllm/cache.py:52-231, :431-463, :466-587,
:639-673); released blocks go to the front of its free list (:151-154), here
the free list is a stack, which reuses them as early.
"""

from __future__ import annotations

from dataclasses import dataclass, field


class CacheError(RuntimeError):
    """The cache was asked for something that breaks its bookkeeping."""


@dataclass(frozen=True)
class CacheGroup:
    """Runs that share page geometry and block tables."""

    runs: tuple[int, ...]
    num_kv_heads: int
    head_dim: int
    window: int | None = None


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


class PagePool:
    """Pages 0..n-1, each either free or held by exactly one owner."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 0:
            raise ValueError("num_pages must not be negative")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # stack: last freed, first taken
        self._owner: list[object | None] = [None] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self, count: int, owner) -> list[int] | None:
        """``count`` pages for ``owner``, or None (and no change) if too few are free."""
        if owner is None:
            raise CacheError("a page needs an owner")
        if count > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            if self._owner[page] is not None:
                raise CacheError(f"page {page} was on the free list while held")
            self._owner[page] = owner
        return pages

    def give(self, pages, owner) -> None:
        """Return pages; in the order given, so the last one is reused first.  The manager hands
        a block table back last page first: the next request then gets the same pages in the same
        (from a fresh pool: rising) order, and the prefill attention copies neighbouring pages
        several at a time."""
        for page in pages:
            if not 0 <= page < self.num_pages:
                raise CacheError(f"page {page} does not exist")
            if self._owner[page] is None:
                raise CacheError(f"page {page} is freed twice")
            if self._owner[page] != owner:
                raise CacheError(f"page {page} is held by {self._owner[page]!r}, not {owner!r}")
            self._owner[page] = None
            self._free.append(page)

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is free or held, never both and never lost."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for page in range(self.num_pages):
            held = self._owner[page] is not None
            if held == (page in free):
                raise CacheError(f"page {page} is {'held and free' if held else 'lost'}")


class SlotPool:
    """State slots 0..n-1 for the live requests."""

    def __init__(self, num_slots: int) -> None:
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held: set[int] = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int | None:
        if not self._free:
            return None
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def give(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"state slot {slot} is freed twice")
        self._held.remove(slot)
        self._free.append(slot)


@dataclass
class _Request:
    state_slot: int
    length: int = 0                                   # tokens whose keys are written
    tables: list[list[int]] = field(default_factory=list)   # per group, -1 = given back
    planned: bool = False
    opening: int = 0                                  # which call of open() made it (ids may come again)


@dataclass(frozen=True)
class PlannedEntry:
    """What one entry of a step reads and writes."""

    request_id: object
    start: int                                # tokens in the cache before the step
    count: int                                # tokens the step adds
    state_slot: int
    fresh_state: bool                         # first tokens of the request: state starts at zero
    slots: tuple[tuple[int, ...], ...]        # per group: cache slot of each new token
    tables: tuple                             # per group: the request's block table (the live list:
                                              # read it before the step is committed, do not change it)
    opening: int = 0                          # number of the open() that admitted the request: two
                                              # requests with one id, one after the other, differ in it


@dataclass
class StepCachePlan:
    entries: tuple[PlannedEntry, ...]
    taken: list[tuple[int, object, list[int]]]        # (group, request, pages) taken by this plan
    state: str = "planned"                            # planned -> committed | rolled_back


class CacheManager:
    def __init__(self, groups, page_size: int, pages_per_group, num_state_slots: int) -> None:
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.groups: tuple[CacheGroup, ...] = tuple(groups)
        if isinstance(pages_per_group, int):
            pages_per_group = [pages_per_group] * len(self.groups)
        if len(pages_per_group) != len(self.groups):
            raise ValueError("one page count per group is needed")
        self.page_size = page_size
        self.pools = [PagePool(count) for count in pages_per_group]
        self.slots = SlotPool(num_state_slots)
        self._requests: dict[object, _Request] = {}
        self._openings = 0

    # ------------------------------------------------------------ requests
    def open(self, request_id) -> int:
        """Admit a request: it gets a state slot and empty block tables."""
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already open")
        slot = self.slots.take()
        if slot is None:
            raise CacheError("no state slot is free")
        self._openings += 1
        self._requests[request_id] = _Request(slot, 0, [[] for _ in self.groups], False, self._openings)
        return slot

    def close(self, request_id) -> None:
        """Give back everything the request holds."""
        request = self._requests.get(request_id)
        if request is None:
            raise CacheError(f"request {request_id!r} is not open")
        if request.planned:
            raise CacheError(f"request {request_id!r} is part of a step that has not ended")
        del self._requests[request_id]
        for group, table in enumerate(request.tables):
            self.pools[group].give([p for p in reversed(table) if p >= 0], request_id)
        self.slots.give(request.state_slot)

    def is_open(self, request_id) -> bool:
        return request_id in self._requests

    def length(self, request_id) -> int:
        return self._requests[request_id].length

    def state_slot(self, request_id) -> int:
        return self._requests[request_id].state_slot

    def block_table(self, request_id, group: int) -> tuple[int, ...]:
        return tuple(self._requests[request_id].tables[group])

    def open_requests(self) -> tuple:
        return tuple(self._requests)

    # -------------------------------------------------------------- demand
    def first_needed(self, group: int, next_position: int) -> int:
        """First key position any query at or after ``next_position`` reads."""
        window = self.groups[group].window
        return 0 if window is None else max(0, next_position - window + 1)

    def new_pages(self, request_id, group: int, count: int) -> int:
        """Pages group ``group`` must take to add ``count`` tokens to the request."""
        request = self._requests[request_id]
        return ceil_div(request.length + count, self.page_size) - len(request.tables[group])

    def peak_pages(self, group: int, total_tokens: int, max_step_tokens: int) -> int:
        """Most pages a request of ``total_tokens`` written tokens ever holds in
        ``group`` when no step adds more than ``max_step_tokens`` to it."""
        full = ceil_div(total_tokens, self.page_size)
        window = self.groups[group].window
        if window is None:
            return full
        span = window - 1 + max(1, max_step_tokens)
        return min(full, ceil_div(span, self.page_size) + 1)

    def free_pages(self, group: int) -> int:
        return self.pools[group].free_count

    # ---------------------------------------------------------------- steps
    def plan(self, appends) -> StepCachePlan | None:
        """Take pages for ``appends`` = [(request_id, count), ...], all or nothing."""
        appends = list(appends)
        seen = set()
        for request_id, count in appends:
            if request_id not in self._requests:
                raise CacheError(f"request {request_id!r} is not open")
            if request_id in seen:
                raise CacheError(f"request {request_id!r} appears twice in one step")
            if self._requests[request_id].planned:
                raise CacheError(f"request {request_id!r} is part of a step that has not ended")
            if type(count) is not int or count <= 0:
                raise CacheError("an entry must add at least one token")
            seen.add(request_id)
        for group in range(len(self.groups)):
            need = sum(self.new_pages(rid, group, count) for rid, count in appends)
            if need > self.pools[group].free_count:
                return None
        taken: list[tuple[int, object, list[int]]] = []
        entries = []
        size = self.page_size
        for request_id, count in appends:
            request = self._requests[request_id]
            slots, tables = [], []
            for group in range(len(self.groups)):
                pages = self.pools[group].take(self.new_pages(request_id, group, count), request_id)
                assert pages is not None
                if pages:
                    taken.append((group, request_id, pages))
                    request.tables[group].extend(pages)
                table = request.tables[group]
                if count == 1:
                    p = request.length
                    if table[p // size] < 0:
                        raise CacheError("a token would be written to a page already given back")
                    row = (table[p // size] * size + p % size,)
                else:
                    positions = range(request.length, request.length + count)
                    row = tuple(table[p // size] * size + p % size for p in positions)
                    if any(table[p // size] < 0 for p in positions):
                        raise CacheError("a token would be written to a page already given back")
                slots.append(row)
                tables.append(table)
            request.planned = True
            entries.append(PlannedEntry(
                request_id, request.length, count, request.state_slot,
                request.length == 0, tuple(slots), tuple(tables), request.opening))
        return StepCachePlan(tuple(entries), taken)

    def commit(self, plan: StepCachePlan, written: int | None = None) -> None:
        """The step ran: lengths advance, windows let go of what they passed.  ``written``: every
        entry wrote only its first ``written`` tokens (a run of decode steps that was cut short);
        the pages taken for the rest go back."""
        if plan.state != "planned":
            raise CacheError(f"the plan is already {plan.state}")
        if written is not None and not (type(written) is int and 0 <= written
                                        and all(written <= entry.count for entry in plan.entries)):
            raise CacheError("an entry cannot have written more tokens than were planned for it")
        plan.state = "committed"
        size = self.page_size
        for entry in plan.entries:
            request = self._requests[entry.request_id]
            request.planned = False
            request.length = entry.start + (entry.count if written is None else written)
            if written is not None and written < entry.count:
                for group, table in enumerate(request.tables):
                    keep = ceil_div(request.length, size)
                    extra = table[keep:]
                    if extra:
                        del table[keep:]
                        self.pools[group].give([p for p in reversed(extra) if p >= 0], entry.request_id)
            for group, table in enumerate(request.tables):
                first = self.first_needed(group, request.length)
                passed = [i for i in range(min(len(table), first // size)) if table[i] >= 0]
                if passed:
                    self.pools[group].give([table[i] for i in passed], entry.request_id)
                    for i in passed:
                        table[i] = -1

    def rollback(self, plan: StepCachePlan) -> None:
        """The step did not run: its pages go back, lengths stay."""
        if plan.state != "planned":
            raise CacheError(f"the plan is already {plan.state}")
        plan.state = "rolled_back"
        for group, request_id, pages in reversed(plan.taken):
            table = self._requests[request_id].tables[group]
            del table[len(table) - len(pages):]
            self.pools[group].give(list(reversed(pages)), request_id)
        for entry in plan.entries:
            self._requests[entry.request_id].planned = False

    # ------------------------------------------------------------ checking
    def check(self) -> None:
        """No page lost, held twice or held by a request that does not list it."""
        for group, pool in enumerate(self.pools):
            pool.check()
            listed: dict[int, object] = {}
            for request_id, request in self._requests.items():
                for page in request.tables[group]:
                    if page < 0:
                        continue
                    if page in listed:
                        raise CacheError(f"page {page} of group {group} is in two block tables")
                    listed[page] = request_id
            for page in range(pool.num_pages):
                owner = pool.owner_of(page)
                if owner != listed.get(page):
                    raise CacheError(
                        f"page {page} of group {group}: pool says {owner!r}, "
                        f"tables say {listed.get(page)!r}")
