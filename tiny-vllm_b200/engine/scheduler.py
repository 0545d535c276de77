"""Continuous batching with chunked prefill over the cache manager.

A request whose arrival time lies ahead is kept aside until the clock reaches it.
Requests then wait in arrival order, are admitted while a state slot is free and
their whole lifetime fits into the page pools, run as prompt portions under a
token budget and then as single decoded tokens, and give everything back when
they finish or are cancelled.

What happens when pages run out is decided at admission: a request enters only
if the pages it can ever hold (prompt plus the tokens it may still generate;
for a windowed group the most its window and one step can span) fit into what
is free after the promises made to the requests already running.  A running
request therefore never lacks a page, nothing is preempted or recomputed, and a
request that does not fit yet stays waiting without blocking later, smaller
ones.  A request that could never fit is refused when it is submitted.

Policy and limits follow tinyvllm/scheduler.py: limits :92-150, up-front
refusal :241-269, lifetime demand and skipping admission :758-866, decodes
first :449-459, prefill reservation :427-447, portions :461-501 and :898-951,
commit and finish reasons :617-699, cancel :954-1000, immediate finish
:1058-1066, arrivals ahead of the clock :226-236 and :1045-1069, giving
everything up after a failed step :702-729.  The cache transaction is
``CacheManager.plan/commit/rollback``.
"""

from __future__ import annotations

import heapq
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Sequence

from ..cache.manager import CacheManager, StepCachePlan
from ..sampling.params import SamplingParams


class RequestStatus(Enum):
    PENDING = "pending"          # its arrival time has not come yet
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"

    @property
    def terminal(self) -> bool:
        return self in (RequestStatus.FINISHED, RequestStatus.ABORTED)


@dataclass
class Request:
    request_id: int
    prompt_token_ids: tuple[int, ...]
    sampling: SamplingParams
    arrival_ns: int = 0
    output_token_ids: list[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    computed_tokens: int = 0            # tokens whose keys and values are in the cache
    finish_reason: str | None = None    # "stop" | "length" | "cancelled"
    admitted_ns: int | None = None
    first_token_ns: int | None = None
    finished_ns: int | None = None
    promised: tuple[int, ...] = ()      # pages per group promised at admission

    @property
    def total_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def remaining_new_tokens(self) -> int:
        return self.sampling.max_new_tokens - len(self.output_token_ids)

    @property
    def decoding(self) -> bool:
        """All known tokens but the last are computed: the next step is a single token."""
        return bool(self.output_token_ids) and self.computed_tokens == self.total_tokens - 1

    def tokens(self, start: int, end: int) -> tuple[int, ...]:
        prompt = len(self.prompt_token_ids)
        if end <= prompt:
            return tuple(self.prompt_token_ids[start:end])
        if start >= prompt:
            return tuple(self.output_token_ids[start - prompt:end - prompt])
        return tuple(self.prompt_token_ids[start:]) + tuple(self.output_token_ids[:end - prompt])


@dataclass(frozen=True)
class WorkItem:
    request_id: int
    start: int
    count: int
    sample: bool          # the last token of the item produces the request's next token


@dataclass
class ScheduledStep:
    items: tuple[WorkItem, ...]
    cache_plan: StepCachePlan

    @property
    def num_tokens(self) -> int:
        return sum(item.count for item in self.items)


@dataclass
class ScheduledRun:
    """Several decode steps of the same requests, planned at once: item.count tokens each."""

    items: tuple[WorkItem, ...]
    cache_plan: StepCachePlan
    steps: int
    # while the run is read step by step (begin_run .. end_run):
    steps_read: int = 0
    closing: list = field(default_factory=list)      # requests that ended meanwhile; their pages go back at the end


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk_size: int, max_model_len: int, prefill_reserve_tokens: int = 0,
                 prefill_reserve_requests: int = 0, eos_token_ids=()) -> None:
        if prefill_chunk_size > max_num_batched_tokens:
            raise ValueError(f"a prompt portion of {prefill_chunk_size} tokens does not fit into a step "
                             f"of {max_num_batched_tokens} tokens")
        if bool(prefill_reserve_tokens) != bool(prefill_reserve_requests):
            raise ValueError("room is kept for prefills either in tokens and in requests, or in neither "
                             f"(got {prefill_reserve_tokens} tokens, {prefill_reserve_requests} requests)")
        if max_num_seqs > cache.slots.num_slots:
            raise ValueError("max_num_seqs exceeds the state slots of the cache")
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.prefill_chunk_size = prefill_chunk_size
        self.max_model_len = max_model_len
        self.prefill_reserve_tokens = prefill_reserve_tokens
        self.prefill_reserve_requests = prefill_reserve_requests
        self.eos_token_ids = frozenset(eos_token_ids)
        self.requests: dict[int, Request] = {}
        self.waiting: deque[int] = deque()
        self.prefilling: list[int] = []
        self.decoding: list[int] = []
        self.finished: list[Request] = []
        self.run_in_flight: ScheduledRun | None = None
        self._prefer_waiting = False
        self._ahead: list[tuple[int, int, int]] = []      # heap of (arrival_ns, order of submission, request id)
        self._submitted = 0
        self._now_ns: int | None = None
        self.stopped = False                              # shutdown() was called: nothing is scheduled any more

    # -------------------------------------------------------------- demand
    def _written_tokens(self, request: Request) -> int:
        """Tokens the request ever writes to the cache: the last sampled one is not written."""
        prompt = len(request.prompt_token_ids)
        new = min(request.sampling.max_new_tokens, self.max_model_len - prompt)
        return prompt + max(new, 1) - 1

    def lifetime_pages(self, request: Request) -> tuple[int, ...]:
        written = self._written_tokens(request)
        return tuple(self.cache.peak_pages(g, written, self.prefill_chunk_size)
                     for g in range(len(self.cache.groups)))

    def _outstanding(self, group: int) -> int:
        """Pages promised to running requests that they have not taken yet."""
        total = 0
        for request_id in self.prefilling + self.decoding:
            request = self.requests[request_id]
            held = sum(1 for page in self.cache.block_table(request_id, group) if page >= 0)
            total += max(0, request.promised[group] - held)
        return total

    # ------------------------------------------------------------ commands
    def validate(self, prompt_token_ids, sampling: SamplingParams) -> None:
        if not isinstance(sampling, SamplingParams):
            raise TypeError("sampling must be SamplingParams")
        if len(prompt_token_ids) == 0:
            raise ValueError("the prompt must hold at least one token")
        if len(prompt_token_ids) > self.max_model_len:
            raise ValueError(f"the prompt has {len(prompt_token_ids)} tokens, "
                             f"max_model_len is {self.max_model_len}")
        probe = Request(-1, tuple(prompt_token_ids), sampling)
        for group, pages in enumerate(self.lifetime_pages(probe)):
            if pages > self.cache.pools[group].num_pages:
                raise ValueError(f"the request needs {pages} pages of cache group {group}, "
                                 f"the pool has {self.cache.pools[group].num_pages}")

    def add(self, request: Request, now_ns: int = 0) -> None:
        """Take a request in.  With ``request.arrival_ns`` later than ``now_ns`` it is kept aside
        and joins the waiting queue when :meth:`advance` is told a time at or past its arrival."""
        self._refuse_if_stopped()
        if request.request_id in self.requests:
            raise ValueError(f"request id {request.request_id} is in use")
        self.validate(request.prompt_token_ids, request.sampling)
        self.requests[request.request_id] = request
        self._submitted += 1
        if request.arrival_ns > now_ns:
            request.status = RequestStatus.PENDING
            heapq.heappush(self._ahead, (request.arrival_ns, self._submitted, request.request_id))
            return
        self._arrive(request, now_ns)

    def _arrive(self, request: Request, now_ns: int) -> None:
        if request.sampling.max_new_tokens == 0 or len(request.prompt_token_ids) == self.max_model_len:
            self._finish(request, "length", now_ns)     # nothing can be generated
            return
        request.status = RequestStatus.WAITING
        self.waiting.append(request.request_id)

    def _still_ahead(self, entry: tuple[int, int, int]) -> bool:
        request = self.requests.get(entry[2])
        return (request is not None and request.status is RequestStatus.PENDING
                and request.arrival_ns == entry[0])

    @property
    def next_arrival_ns(self) -> int | None:
        """Arrival time of the earliest request still kept aside (cancelled ones do not count)."""
        while self._ahead and not self._still_ahead(self._ahead[0]):
            heapq.heappop(self._ahead)
        return self._ahead[0][0] if self._ahead else None

    def advance(self, now_ns: int) -> int:
        """The clock reads ``now_ns`` (it never runs backwards): requests whose time has come join
        the waiting queue in the order of their arrival times.  Returns how many did."""
        if type(now_ns) is not int or now_ns < 0:
            raise ValueError("now_ns must be a non-negative int")
        if self._now_ns is not None and now_ns < self._now_ns:
            raise ValueError(f"the clock ran backwards: {now_ns} after {self._now_ns}")
        self._now_ns = now_ns
        arrived = 0
        while self._ahead and self._ahead[0][0] <= now_ns:
            entry = heapq.heappop(self._ahead)
            if self._still_ahead(entry):
                self._arrive(self.requests[entry[2]], now_ns)
                arrived += 1
        return arrived

    def cancel(self, request_id: int, now_ns: int = 0) -> bool:
        request = self.requests.get(request_id)
        if request is None or request.status.terminal:
            return False
        if request_id in self.waiting:
            self.waiting.remove(request_id)
        self._finish(request, "cancelled", now_ns)       # one kept aside: its heap entry is skipped later
        return True

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.prefilling or self.decoding or self.next_arrival_ns is not None)

    def _refuse_if_stopped(self) -> None:
        if self.stopped:
            raise RuntimeError("the scheduler was shut down after a failed step")

    def shutdown(self, open_plan: StepCachePlan | None = None) -> None:
        """Give everything up after a step that failed on the device: the plan that was open is
        rolled back, every request lets go of its pages and slot, all queues are emptied and
        nothing is scheduled any more.  What the requests had produced is lost with them."""
        self.stopped = True
        run, self.run_in_flight = self.run_in_flight, None
        for plan in (open_plan, run.cache_plan if run is not None else None):
            if plan is not None and plan.state == "planned":
                self.cache.rollback(plan)
        for request_id in list(self.cache.open_requests()):
            self.cache.close(request_id)
        self.requests.clear()
        self.waiting.clear()
        self.prefilling.clear()
        self.decoding.clear()
        self.finished.clear()
        self._ahead.clear()

    def take_finished(self) -> list[Request]:
        done, self.finished = self.finished, []
        for request in done:
            self.requests.pop(request.request_id, None)
        return done

    # ------------------------------------------------------------ planning
    def _admit(self, now_ns: int) -> list[int]:
        """Waiting requests that fit now, in arrival order; those that do not are skipped."""
        admitted = []
        if not self.waiting:
            return admitted
        groups = range(len(self.cache.groups))
        room = [self.cache.free_pages(g) - self._outstanding(g) for g in groups]
        slots = min(self.cache.slots.free_count,
                    self.max_num_seqs - len(self.prefilling) - len(self.decoding))
        for request_id in list(self.waiting):
            if slots <= 0:
                break
            request = self.requests[request_id]
            demand = self.lifetime_pages(request)
            if all(demand[g] <= room[g] for g in groups):
                for g in groups:
                    room[g] -= demand[g]
                slots -= 1
                request.promised = demand
                admitted.append(request_id)
        return admitted

    def schedule(self, now_ns: int = 0) -> ScheduledStep | None:
        """The next step, with its pages taken; None when there is nothing to run."""
        self._refuse_if_stopped()
        if self.run_in_flight is not None:
            raise RuntimeError("a run of decode steps is in flight: end it before the next step is planned")
        admitted = self._admit(now_ns)
        active_prefills = list(self.prefilling)
        candidates = (admitted + active_prefills) if self._prefer_waiting else (active_prefills + admitted)
        rows, tokens = self.max_num_seqs, self.max_num_batched_tokens
        reserve_rows = reserve_tokens = 0
        if candidates and self.decoding:
            reserve_rows = min(self.prefill_reserve_requests, len(candidates))
            reserve_tokens = self.prefill_reserve_tokens if reserve_rows else 0
        decode_count = max(0, min(len(self.decoding), rows - reserve_rows, tokens - reserve_tokens))
        items: list[WorkItem] = []
        for request_id in self.decoding[:decode_count]:
            request = self.requests[request_id]
            items.append(WorkItem(request_id, request.computed_tokens, 1, True))
        rows -= decode_count
        tokens -= decode_count
        chosen_waiters = []
        for request_id in candidates:
            if rows <= 0 or tokens <= 0:
                break
            request = self.requests[request_id]
            left = request.total_tokens - request.computed_tokens
            count = min(left, self.prefill_chunk_size, tokens)
            end = request.computed_tokens + count
            sample = end == request.total_tokens and end < self.max_model_len + 1
            items.append(WorkItem(request_id, request.computed_tokens, count, sample))
            if request_id in admitted:
                chosen_waiters.append(request_id)
            rows -= 1
            tokens -= count
        # decodes that were held back for prefills that did not come take the room left
        extra = min(len(self.decoding) - decode_count, rows, tokens)
        for request_id in self.decoding[decode_count:decode_count + max(0, extra)]:
            request = self.requests[request_id]
            items.insert(decode_count, WorkItem(request_id, request.computed_tokens, 1, True))
            decode_count += 1
        if not items:
            return None
        for request_id in chosen_waiters:
            self.cache.open(request_id)
        plan = self.cache.plan([(item.request_id, item.count) for item in items])
        if plan is None:
            for request_id in chosen_waiters:
                self.cache.close(request_id)
            raise RuntimeError("admitted requests exceeded their page budget")
        for request_id in chosen_waiters:
            request = self.requests[request_id]
            self.waiting.remove(request_id)
            self.prefilling.append(request_id)
            request.status = RequestStatus.RUNNING
            request.admitted_ns = now_ns
        had_both = bool(decode_count) and len(items) > decode_count
        if had_both:
            self._prefer_waiting = not self._prefer_waiting
        return ScheduledStep(tuple(items), plan)

    def schedule_decode_run(self, max_steps: int, now_ns: int = 0) -> ScheduledRun | None:
        """Up to ``max_steps`` decode steps of all decoding requests as one plan, or None.

        Only when nothing waits and nothing is being prefilled (a newcomer would wait for the whole
        run), and only as many steps as every request may still take: none reaches its token limit
        or the context limit before the run's last step.  A request that meets a stop token inside
        the run ends there; what the run computed for it beyond is dropped with its pages."""
        self._refuse_if_stopped()
        if self.run_in_flight is not None:
            raise RuntimeError("a run of decode steps is in flight: end it before the next is planned")
        if max_steps < 2 or not self.decoding or self.waiting or self.prefilling:
            return None
        if len(self.decoding) > min(self.max_num_seqs, self.max_num_batched_tokens):
            return None
        steps = max_steps
        for request_id in self.decoding:
            request = self.requests[request_id]
            steps = min(steps, request.remaining_new_tokens, self.max_model_len - request.total_tokens)
        if steps < 2:
            return None
        while steps >= 2:                    # a shorter run if the pool has no pages for the whole one
            items = tuple(WorkItem(request_id, self.requests[request_id].computed_tokens, steps, True)
                          for request_id in self.decoding)
            plan = self.cache.plan([(item.request_id, item.count) for item in items])
            if plan is not None:
                return ScheduledRun(items, plan, steps)
            steps //= 2
        return None

    def commit_run(self, run: ScheduledRun, sampled: Sequence[dict[int, int]], now_ns: int = 0) -> list[tuple[int, int]]:
        """The run ran.  ``sampled[i]`` maps request id to the token of the run's i-th step.
        Returns (request id, token) in step order; a request that ended inside the run has no
        tokens after its end."""
        if len(sampled) != run.steps:
            raise ValueError(f"a run of {run.steps} steps came back with {len(sampled)}")
        for tokens in sampled:
            for item in run.items:
                if item.request_id not in tokens:
                    raise ValueError(f"no token was sampled for request {item.request_id}")
        self.cache.commit(run.cache_plan)
        events = []
        for index, tokens in enumerate(sampled):
            for item in run.items:
                request = self.requests[item.request_id]
                if request.status.terminal:          # ended earlier in this run, or cancelled
                    continue
                request.computed_tokens = item.start + index + 1
                token = int(tokens[item.request_id])
                request.output_token_ids.append(token)
                events.append((item.request_id, token))
                if token in self.eos_token_ids and not request.sampling.ignore_eos:
                    self._finish(request, "stop", now_ns)
                elif request.remaining_new_tokens <= 0 or request.total_tokens >= self.max_model_len:
                    self._finish(request, "length", now_ns)
        return events

    # A run can also be read step by step while its later steps still execute: begin_run, then
    # commit_run_step for every step that ran (in order), then end_run.  A request that ends at a
    # step (stop token, limit, cancel) leaves the queues at once, but keeps its pages until
    # end_run: steps launched ahead may still write to them.
    def begin_run(self, run: ScheduledRun) -> None:
        if self.run_in_flight is not None:
            raise RuntimeError("a run of decode steps is already in flight")
        self.run_in_flight = run

    def commit_run_step(self, run: ScheduledRun, tokens: dict[int, int], now_ns: int = 0) -> list[tuple[int, int]]:
        """The run's next step ran; ``tokens`` maps request id to its token.  Returns (request id,
        token) of the requests that had not ended before."""
        if run is not self.run_in_flight or run.steps_read >= run.steps:
            raise RuntimeError("no such step of a run in flight")
        for item in run.items:
            if item.request_id not in tokens:
                raise ValueError(f"no token was sampled for request {item.request_id}")
        index = run.steps_read
        run.steps_read += 1
        events = []
        for item in run.items:
            request = self.requests.get(item.request_id)
            if request is None or request.status.terminal:       # ended earlier in this run, or cancelled
                continue
            request.computed_tokens = item.start + index + 1
            token = int(tokens[item.request_id])
            request.output_token_ids.append(token)
            events.append((item.request_id, token))
            if token in self.eos_token_ids and not request.sampling.ignore_eos:
                self._finish(request, "stop", now_ns)
            elif request.remaining_new_tokens <= 0 or request.total_tokens >= self.max_model_len:
                self._finish(request, "length", now_ns)
        return events

    def end_run(self, run: ScheduledRun) -> None:
        """Every launched step of the run has been read (``run.steps_read`` of them): the cache
        keeps what they wrote, the rest of the plan and the pages of ended requests go back."""
        if run is not self.run_in_flight:
            raise RuntimeError("the run is not in flight")
        self.run_in_flight = None
        self.cache.commit(run.cache_plan, written=run.steps_read)
        for request_id in run.closing:
            if self.cache.is_open(request_id):
                self.cache.close(request_id)
        run.closing.clear()

    # ------------------------------------------------------------- results
    def abort_step(self, step: ScheduledStep) -> None:
        """The step did not run: its pages go back; requests keep their places."""
        self.cache.rollback(step.cache_plan)

    def commit(self, step: ScheduledStep, sampled: dict[int, int], now_ns: int = 0) -> list[tuple[int, int]]:
        """The step ran.  ``sampled`` maps request id to its new token for every item
        with ``sample``.  Returns (request id, token) in item order."""
        for item in step.items:
            if item.sample and item.request_id not in sampled:
                raise ValueError(f"no token was sampled for request {item.request_id}")
        self.cache.commit(step.cache_plan)
        events = []
        for item in step.items:
            request = self.requests[item.request_id]
            if request.status.terminal:          # cancelled while the step ran
                continue
            request.computed_tokens = item.start + item.count
            if not item.sample:
                continue
            token = int(sampled[item.request_id])
            request.output_token_ids.append(token)
            events.append((item.request_id, token))
            if request.first_token_ns is None:
                request.first_token_ns = now_ns
            if item.request_id in self.prefilling:
                self.prefilling.remove(item.request_id)
                self.decoding.append(item.request_id)
            if token in self.eos_token_ids and not request.sampling.ignore_eos:
                self._finish(request, "stop", now_ns)
            elif request.remaining_new_tokens <= 0 or request.total_tokens >= self.max_model_len:
                self._finish(request, "length", now_ns)
        return events

    def _finish(self, request: Request, reason: str, now_ns: int) -> None:
        request_id = request.request_id
        for queue in (self.prefilling, self.decoding):
            if request_id in queue:
                queue.remove(request_id)
        if self.cache.is_open(request_id):
            run = self.run_in_flight
            if run is not None and any(item.request_id == request_id for item in run.items):
                run.closing.append(request_id)           # steps launched ahead may still write its pages
            else:
                self.cache.close(request_id)
        request.status = RequestStatus.ABORTED if reason == "cancelled" else RequestStatus.FINISHED
        request.finish_reason = reason
        request.finished_ns = now_ns
        self.finished.append(request)
