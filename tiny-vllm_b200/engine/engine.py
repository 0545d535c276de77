"""The engine: model, cache, step function, scheduler and sampler behind one lifecycle.

``Engine.from_config`` reads the model folder, loads (or draws) the weights,
sizes the page pools from the byte budget, captures the decode graphs and
returns an engine; ``submit``/``step``/``generate``/``cancel``/``close`` are the
token-level API.  Start-up follows tinyvllm/bootstrap.py:59-208 (KV sizing
:19-56, :109-145), the step follows tinyvllm/engine.py:303-387 and
tinyvllm/executor.py:125-141: plan, lower, run, sample, one device-to-host read
of the sampled ids, commit.  A step fails in one of two ways
(tinyvllm/engine.py:354-387, :543-564): while it is lowered on the host, before
anything of it was launched, its pages go back and the engine stays usable;
once it has been launched, the engine stops for good (fail-stop): every request
is dropped with its pages and later calls are refused.  Requests may carry an
arrival time ahead of the clock and ``step`` may be told the time
(tinyvllm/engine.py:179-256, :303-306, :426-435).
"""

from __future__ import annotations

import contextlib
import logging
import os
import time
from dataclasses import dataclass
from typing import Sequence

import torch

from ..config.engine import EngineConfig
from ..ops import kernels
from ..config.registry import read_model_config
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .graphs import DecodeGraphs
from .model import Model
from .scheduler import Request, RequestStatus, ScheduledStep, Scheduler
from .step import StepEntry, StepRunner

log = logging.getLogger("tinyvllm_b200")

# TINYVLLM_B200_NVTX=1: every call of Engine.step and its phases (schedule, lower, launch and read,
# commit; a decode run's launches and reads) are NVTX ranges, for a timeline in Nsight Systems
NVTX = os.environ.get("TINYVLLM_B200_NVTX", "0") == "1"


@contextlib.contextmanager
def _range(name: str):
    if not NVTX:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


@dataclass(frozen=True)
class GenerateRequest:
    prompt_token_ids: tuple[int, ...]
    sampling: SamplingParams
    request_id: int | None = None
    arrival_ns: int | None = None         # None: it arrives when it is submitted

    def __post_init__(self) -> None:
        object.__setattr__(self, "prompt_token_ids", tuple(self.prompt_token_ids))


@dataclass(frozen=True)
class RequestOutput:
    request_id: int
    output_token_ids: tuple[int, ...]
    prompt_token_count: int
    finish_reason: str                    # "stop" | "length" | "cancelled"
    status: RequestStatus
    arrival_ns: int
    admitted_ns: int | None
    first_token_ns: int | None
    finished_ns: int | None

    @staticmethod
    def of(request: Request) -> "RequestOutput":
        return RequestOutput(
            request.request_id, tuple(request.output_token_ids), len(request.prompt_token_ids),
            request.finish_reason or "length", request.status, request.arrival_ns,
            request.admitted_ns, request.first_token_ns, request.finished_ns)


@dataclass(frozen=True)
class StepEvents:
    tokens: tuple[tuple[int, int], ...]          # (request id, new token)
    finished: tuple[RequestOutput, ...]


def plan_pages(kv_cache_memory_bytes: int, bytes_per_page: int, free_bytes: int, total_bytes: int,
               used_bytes: int, utilization: float) -> int:
    """Pages per group from the byte budget, refused if they do not fit under the ceiling
    (tinyvllm/bootstrap.py:19-56)."""
    pages = kv_cache_memory_bytes // bytes_per_page
    if pages <= 0:
        raise ValueError(f"kv_cache_memory_bytes={kv_cache_memory_bytes} holds no page "
                         f"of {bytes_per_page} bytes")
    room = min(free_bytes, int(total_bytes * utilization) - used_bytes)
    if pages * bytes_per_page > room:
        raise ValueError(
            f"the cache of {pages * bytes_per_page} bytes does not fit: {room} bytes are left "
            f"under gpu_memory_utilization={utilization}")
    return pages


def check_memory_ceiling(used_bytes: int, total_bytes: int, utilization: float) -> None:
    """After everything is set up (cache, graphs and their pools, library work areas): the device
    must not hold more than its allowed share (tinyvllm/bootstrap.py:171-185)."""
    allowed = int(total_bytes * utilization)
    if used_bytes > allowed:
        raise ValueError(
            f"the engine holds {used_bytes} bytes of the device after start-up, more than the {allowed} "
            f"that gpu_memory_utilization={utilization} allows: lower kv_cache_memory_bytes, set "
            "enforce_eager, or free device memory")


@dataclass
class _LoweredStep:
    """A scheduled step after its host half: what the device half needs."""

    sample_ids: list
    params: list
    draws: list
    bucket: object = None                 # (bucket, rows) of a decode graph, or
    prepared: object = None               # a PreparedStep of the step runner


class Engine:
    def __init__(self, runner: StepRunner, scheduler: Scheduler, *, graphs: DecodeGraphs | None = None,
                 clock=time.monotonic_ns, decode_run_steps: int = 1, sleep=time.sleep) -> None:
        self.runner = runner
        self.scheduler = scheduler
        self.graphs = graphs
        self.decode_run_steps = decode_run_steps if graphs is not None else 1
        self.sampler = Sampler()
        self._clock = clock
        self._sleep = sleep
        self._next_id = 0
        self._closed = False
        self._failed: str | None = None
        self._last_now: int | None = None
        self.steps_run = 0
        self.graph_steps = 0
        self.prompt_tokens = 0          # tokens of prompt portions run so far
        self.decode_tokens = 0          # single tokens run so far (one per request and decode step)
        self.lowering_failures = 0      # steps that failed before launch and were rolled back
        self._run = None            # (scheduled run, run in flight on the graphs, request ids) between calls

    # ---------------------------------------------------------- construction
    @classmethod
    def from_config(cls, config: EngineConfig) -> "Engine":
        if not torch.cuda.is_available():
            raise RuntimeError("the engine runs CUDA kernels and needs a GPU; none is visible")
        device = torch.device(config.device)
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[config.dtype]
        torch.backends.cuda.matmul.allow_tf32 = False
        model_config = read_model_config(config.model)
        spec = model_config.to_spec()
        if config.max_model_len > spec.max_positions:
            raise ValueError(f"max_model_len={config.max_model_len} exceeds the model's "
                             f"{spec.max_positions} positions")
        with torch.inference_mode():
            model = Model(spec, device=device, dtype=dtype)
            if config.weights == "random":
                model.init_random(config.seed)
            else:
                model.load(config.model)
            page_bytes = StepRunner.bytes_per_token(model, dtype) * config.kv_block_size
            free, total = torch.cuda.mem_get_info(device)
            pages = plan_pages(config.kv_cache_memory_bytes, page_bytes, free, total, total - free,
                               config.gpu_memory_utilization)
            runner = StepRunner(model, page_size=config.kv_block_size, num_pages=pages,
                                max_requests=config.max_num_seqs, max_model_len=config.max_model_len)
            scheduler = Scheduler(
                runner.manager, max_num_seqs=config.max_num_seqs,
                max_num_batched_tokens=config.max_num_batched_tokens,
                prefill_chunk_size=config.prefill_chunk_size, max_model_len=config.max_model_len,
                prefill_reserve_tokens=config.prefill_reserve_tokens,
                prefill_reserve_requests=config.prefill_reserve_requests,
                eos_token_ids=spec.eos_token_ids)
            graphs = None
            if not config.enforce_eager:
                sizes = [s for s in config.graph_batch_sizes if s <= config.max_num_seqs]
                if config.max_num_seqs not in sizes and config.max_num_seqs <= 256:
                    sizes.append(config.max_num_seqs)
                graphs = DecodeGraphs(runner, sizes, max_model_len=config.max_model_len)
                graphs.capture()
                runner.enable_step_graphs()       # prefill and mixed steps whose shape comes back
            # graph pools and library work areas exist now: measure again
            torch.cuda.synchronize(device)
            torch.cuda.empty_cache()
            free, total = torch.cuda.mem_get_info(device)
            check_memory_ceiling(total - free, total, config.gpu_memory_utilization)
        log.info("engine ready: %s, %s, %d pages of %d tokens per group, %.1f MiB of weights",
                 spec.architecture, config.dtype, pages, config.kv_block_size,
                 model.weight_bytes() / 2**20)
        return cls(runner, scheduler, graphs=graphs, decode_run_steps=config.decode_run_steps)

    # ------------------------------------------------------------- requests
    def _check_usable(self) -> None:
        if self._closed:
            raise RuntimeError("the engine is closed")
        if self._failed:
            raise RuntimeError(f"the engine stopped after a failed step: {self._failed}")

    def submit(self, prompt_token_ids: Sequence[int], sampling: SamplingParams | None = None,
               *, request_id: int | None = None, arrival_ns: int | None = None) -> int:
        """Hand a request to the engine.  With ``arrival_ns`` ahead of the clock it is kept aside
        and takes part from the first step whose time is at or past it."""
        self._check_usable()
        sampling = sampling if sampling is not None else SamplingParams()
        prompt = tuple(prompt_token_ids)
        for token in prompt:
            if type(token) is not int or not 0 <= token < self.runner.vocab_size:
                raise ValueError(f"{token!r} is not a token id below {self.runner.vocab_size}")
        if request_id is None:
            request_id = self._next_id
        if type(request_id) is not int or request_id < 0:
            raise ValueError("request_id must be a non-negative int")
        now = self._now(None)
        if arrival_ns is None:
            arrival_ns = now
        elif type(arrival_ns) is not int or arrival_ns < 0:
            raise ValueError("arrival_ns must be a non-negative int")
        self.scheduler.add(Request(request_id, prompt, sampling, arrival_ns=arrival_ns), now)
        self._next_id = max(self._next_id, request_id + 1)
        return request_id

    def cancel(self, request_id: int) -> bool:
        self._check_usable()
        return self.scheduler.cancel(request_id, self._now(None))

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    def stats(self) -> dict:
        """Counters since the engine was made, and what the cache holds now."""
        manager = self.runner.manager
        runner = self.runner
        return {
            "steps": self.steps_run, "decode_graph_steps": self.graph_steps,
            "prompt_tokens": self.prompt_tokens, "decode_tokens": self.decode_tokens,
            "lowering_failures": self.lowering_failures,
            "step_graphs": len(getattr(runner, "_step_graphs", ())),
            "waiting": len(self.scheduler.waiting), "prefilling": len(self.scheduler.prefilling),
            "decoding": len(self.scheduler.decoding),
            "pages_free": [pool.free_count for pool in manager.pools],
            "pages_total": [pool.num_pages for pool in manager.pools],
            "state_slots_free": manager.slots.free_count,
        }

    @property
    def in_run(self) -> bool:
        """Whether a run of decode steps is in flight (its remaining steps are read by ``step``)."""
        return self._run is not None

    def _now(self, now_ns: int | None) -> int:
        """The time of a call: the caller's, else the clock's, never earlier than the last one the
        scheduler was told (a caller that passes times drives the clock alone)."""
        if now_ns is None:
            now_ns = self._clock()
            if self._last_now is not None:
                now_ns = max(now_ns, self._last_now)
        elif type(now_ns) is not int or now_ns < 0:
            raise ValueError("now_ns must be a non-negative int")
        self._last_now = now_ns
        return now_ns

    # ----------------------------------------------------------------- step
    def step(self, now_ns: int | None = None) -> StepEvents:
        """Run one step of whatever the scheduler picks; tokens and finished requests.  ``now_ns``
        sets the time of the step (arrivals up to it take part, timestamps read it); without it the
        engine's clock is read."""
        self._check_usable()
        now = self._now(now_ns)
        explicit = now_ns is not None
        self.scheduler.advance(now)
        if self._run is not None:
            return self._continue_run(now if explicit else None)
        if self.decode_run_steps > 1 and self.graphs.bucket_for(len(self.scheduler.decoding)) is not None:
            run = self.scheduler.schedule_decode_run(self.decode_run_steps, now)
            if run is not None:
                self._start_run(run)
                return self._continue_run(now if explicit else None)
        with _range("schedule"):
            scheduled = self.scheduler.schedule(now)
        if scheduled is None:
            return StepEvents((), tuple(RequestOutput.of(r) for r in self.scheduler.take_finished()))
        try:
            with _range("lower"):
                lowered = self._lower(scheduled)
        except BaseException:
            # nothing of the step was launched: its pages go back, the requests keep their places
            # and the next call plans them again
            self.scheduler.abort_step(scheduled)
            self.lowering_failures += 1
            raise
        try:
            with _range("launch and read"):
                sampled = self._launch(scheduled, lowered)
            with _range("commit"):
                events = self.scheduler.commit(scheduled, sampled, now if explicit else self._now(None))
        except BaseException as exc:
            self._fail_stop(exc, scheduled.cache_plan)
            raise
        self.steps_run += 1
        for item in scheduled.items:
            if item.count == 1 and item.sample and item.start > 0:
                self.decode_tokens += 1
            else:
                self.prompt_tokens += item.count
        finished = tuple(RequestOutput.of(r) for r in self.scheduler.take_finished())
        return StepEvents(tuple(events), finished)

    def _fail_stop(self, cause: BaseException, open_plan=None) -> None:
        """A step failed after it was launched: what it left in the cache cannot be trusted.  The
        engine keeps the reason as text (not the exception: its traceback would hold tensors), drops
        every request with its pages and refuses all later calls."""
        self._failed = f"{type(cause).__name__}: {cause}"
        self._run = None
        try:
            self.scheduler.shutdown(open_plan)
        except BaseException as cleanup:          # noqa: BLE001 (the first failure is the one reported)
            cause.add_note(f"giving the cache back failed too: {cleanup!r}")

    # A run of decode steps is planned at once and read step by step: a call of step() launches
    # steps until RUN_AHEAD of them are not read yet, waits for the oldest and returns its tokens,
    # so the GPU works on the next step while the caller has this one.  The run ends early when a
    # request of it ends or a newcomer waits (what was launched is still read and counted); the
    # pages of requests that ended inside it go back when it ends.
    RUN_AHEAD = 2

    def _start_run(self, run) -> None:
        requests = self.scheduler.requests
        ids = [item.request_id for item in run.items]
        try:
            first = [requests[i].tokens(item.start, item.start + 1)[0] for i, item in zip(ids, run.items)]
            params = [requests[i].sampling for i in ids]
            draws = [len(requests[i].output_token_ids) for i in ids]
            flight = self.graphs.start_run(run.cache_plan, first, params, draws, run.steps)
            if flight is None:
                raise RuntimeError("no decode graph holds the rows of the run")
        except BaseException:
            # host work only so far: the plan goes back and the engine stays usable
            if run.cache_plan.state == "planned":
                self.scheduler.cache.rollback(run.cache_plan)
            raise
        self.scheduler.begin_run(run)
        self._run = (run, flight, ids)

    def _continue_run(self, fixed_now: int | None = None) -> StepEvents:
        run, flight, ids = self._run
        scheduler = self.scheduler
        events: list = []
        try:
            def must_stop() -> bool:
                return bool(run.closing or scheduler.waiting or scheduler.prefilling)

            def read_one() -> None:
                with _range("read a step of the run"):
                    tokens = flight.read()
                kernels.check_finished_launches()
                when = fixed_now if fixed_now is not None else self._now(None)
                got = scheduler.commit_run_step(run, dict(zip(ids, tokens)), when)
                events.extend(got)
                self.steps_run += 1
                self.graph_steps += 1
                self.decode_tokens += len(got)

            while flight.launched < run.steps and not must_stop() and flight.launched < flight.read_steps + self.RUN_AHEAD:
                with _range("launch a step of the run"):
                    flight.launch()
            if flight.read_steps < flight.launched:
                read_one()
            if flight.launched == run.steps or must_stop():
                while flight.read_steps < flight.launched:       # what was launched ahead still counts
                    read_one()
                scheduler.end_run(run)
                if flight.launched < run.steps:
                    self.graphs.forget_tables(flight.bucket)
                self._run = None
        except BaseException as exc:
            self._fail_stop(exc)
            raise
        finished = tuple(RequestOutput.of(r) for r in scheduler.take_finished())
        return StepEvents(tuple(events), finished)

    @torch.inference_mode()
    def _lower(self, scheduled: ScheduledStep) -> _LoweredStep:
        """The host half of a step: entries from the requests' tokens, sampling arguments, and the
        step's fields lowered into pinned memory (of a decode graph if one holds the step)."""
        requests = self.scheduler.requests
        entries, params, draws, sample_ids = [], [], [], []
        for item in scheduled.items:
            request = requests[item.request_id]
            tokens = request.tokens(item.start, item.start + item.count)
            entries.append(StepEntry(item.request_id, tokens, (item.count - 1,) if item.sample else ()))
            if item.sample:
                params.append(request.sampling)
                draws.append(len(request.output_token_ids))
                sample_ids.append(item.request_id)
        lowered = _LoweredStep(sample_ids, params, draws)
        decode_only = all(item.count == 1 and item.sample for item in scheduled.items)
        if decode_only and self.graphs is not None:
            lowered.bucket = self.graphs.prepare(scheduled.cache_plan, entries, params, draws)
        if lowered.bucket is None:
            lowered.prepared = self.runner.prepare(entries, scheduled.cache_plan)
        return lowered

    @torch.inference_mode()
    def _launch(self, scheduled: ScheduledStep, lowered: _LoweredStep) -> dict[int, int]:
        """The device half: run the step, sample, read the tokens (the step's one device-to-host read)."""
        tokens_device = None
        if lowered.bucket is not None:
            tokens_device = self.graphs.launch(lowered.bucket, scheduled.cache_plan)[0]
            self.graph_steps += 1
        else:
            logits = self.runner.launch(lowered.prepared)
            if logits is not None:
                tokens_device = self.sampler.sample(logits, lowered.params, lowered.draws)
        if tokens_device is None:
            return {}
        host = tokens_device.tolist()
        kernels.check_finished_launches()
        return dict(zip(lowered.sample_ids, host))

    # ------------------------------------------------------------- generate
    def generate(self, requests: Sequence[GenerateRequest]) -> list[RequestOutput]:
        """Run ``requests`` to the end; outputs in the order given.  While nothing can run because
        every request left arrives later, the engine sleeps until the next arrival."""
        self._check_usable()
        if self.has_unfinished():
            raise RuntimeError("generate() needs an idle engine")
        ids = [self.submit(r.prompt_token_ids, r.sampling, request_id=r.request_id, arrival_ns=r.arrival_ns)
               for r in requests]
        outputs: dict[int, RequestOutput] = {}
        while True:
            events = self.step()
            for output in events.finished:
                outputs[output.request_id] = output
            if not self.has_unfinished():
                for request in self.scheduler.take_finished():
                    outputs[request.request_id] = RequestOutput.of(request)
                break
            scheduler = self.scheduler
            if not (events.tokens or scheduler.waiting or scheduler.prefilling or scheduler.decoding):
                ahead = scheduler.next_arrival_ns
                if ahead is not None:
                    delay = (ahead - self._clock()) / 1e9
                    if delay > 0:
                        self._sleep(delay)
        return [outputs[i] for i in ids]

    def close(self) -> None:
        if self._run is not None:                  # steps in flight still write to the cache
            torch.cuda.synchronize()
            self._run = None
        self._closed = True
        self.graphs = None
        drop = getattr(self.runner, "drop_graphs", None)
        if drop is not None:
            drop()
