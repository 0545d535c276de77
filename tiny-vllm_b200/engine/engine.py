"""The engine: model, cache, step function, scheduler and sampler behind one lifecycle.

``Engine.from_config`` reads the model folder, loads (or draws) the weights,
sizes the page pools from the byte budget, captures the decode graphs and
returns an engine; ``submit``/``step``/``generate``/``cancel``/``close`` are the
token-level API.  Start-up follows tinyvllm/bootstrap.py:59-208 (KV sizing
:19-56, :109-145), the step follows tinyvllm/engine.py:303-387 and
tinyvllm/executor.py:125-141: plan, lower, run, sample, one device-to-host read
of the sampled ids, commit.  A failure after the pages of a step are taken
stops the engine for good (fail-stop, tinyvllm/engine.py:367-387, :543-564).
"""

from __future__ import annotations

import logging
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


@dataclass(frozen=True)
class GenerateRequest:
    prompt_token_ids: tuple[int, ...]
    sampling: SamplingParams
    request_id: int | None = None

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


class Engine:
    def __init__(self, runner: StepRunner, scheduler: Scheduler, *, graphs: DecodeGraphs | None = None,
                 clock=time.monotonic_ns, decode_run_steps: int = 1) -> None:
        self.runner = runner
        self.scheduler = scheduler
        self.graphs = graphs
        self.decode_run_steps = decode_run_steps if graphs is not None else 1
        self.sampler = Sampler()
        self._clock = clock
        self._next_id = 0
        self._closed = False
        self._failed: str | None = None
        self.steps_run = 0
        self.graph_steps = 0
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
               *, request_id: int | None = None) -> int:
        self._check_usable()
        sampling = sampling if sampling is not None else SamplingParams()
        prompt = tuple(prompt_token_ids)
        for token in prompt:
            if type(token) is not int or not 0 <= token < self.runner.vocab_size:
                raise ValueError(f"{token!r} is not a token id below {self.runner.vocab_size}")
        if request_id is None:
            request_id = self._next_id
        self._next_id = max(self._next_id, request_id + 1)
        now = self._clock()
        self.scheduler.add(Request(request_id, prompt, sampling, arrival_ns=now), now)
        return request_id

    def cancel(self, request_id: int) -> bool:
        self._check_usable()
        return self.scheduler.cancel(request_id, self._clock())

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ----------------------------------------------------------------- step
    def step(self) -> StepEvents:
        """Run one step of whatever the scheduler picks; tokens and finished requests."""
        self._check_usable()
        if self._run is not None:
            return self._continue_run()
        now = self._clock()
        if self.decode_run_steps > 1 and self.graphs.bucket_for(len(self.scheduler.decoding)) is not None:
            run = self.scheduler.schedule_decode_run(self.decode_run_steps, now)
            if run is not None:
                self._start_run(run)
                return self._continue_run()
        scheduled = self.scheduler.schedule(now)
        if scheduled is None:
            return StepEvents((), tuple(RequestOutput.of(r) for r in self.scheduler.take_finished()))
        try:
            sampled = self._execute(scheduled)
            events = self.scheduler.commit(scheduled, sampled, self._clock())
        except BaseException as exc:
            self._failed = repr(exc)
            if scheduled.cache_plan.state == "planned":
                self.scheduler.abort_step(scheduled)
            raise
        self.steps_run += 1
        finished = tuple(RequestOutput.of(r) for r in self.scheduler.take_finished())
        return StepEvents(tuple(events), finished)

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
            self.scheduler.begin_run(run)
        except BaseException as exc:
            self._failed = repr(exc)
            if run.cache_plan.state == "planned":
                self.scheduler.cache.rollback(run.cache_plan)
            raise
        self._run = (run, flight, ids)

    def _continue_run(self) -> StepEvents:
        run, flight, ids = self._run
        scheduler = self.scheduler
        events: list = []
        try:
            def must_stop() -> bool:
                return bool(run.closing or scheduler.waiting or scheduler.prefilling)

            def read_one() -> None:
                tokens = flight.read()
                kernels.check_finished_launches()
                events.extend(scheduler.commit_run_step(run, dict(zip(ids, tokens)), self._clock()))
                self.steps_run += 1
                self.graph_steps += 1

            while flight.launched < run.steps and not must_stop() and flight.launched < flight.read_steps + self.RUN_AHEAD:
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
            self._failed = repr(exc)
            raise
        finished = tuple(RequestOutput.of(r) for r in scheduler.take_finished())
        return StepEvents(tuple(events), finished)

    @torch.inference_mode()
    def _execute(self, scheduled: ScheduledStep) -> dict[int, int]:
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
        decode_only = all(item.count == 1 and item.sample for item in scheduled.items)
        tokens_device = None
        if decode_only and self.graphs is not None:
            replayed = self.graphs.run(scheduled.cache_plan, entries, params, draws)
            if replayed is not None:
                tokens_device = replayed[0]
                self.graph_steps += 1
        if tokens_device is None:
            logits = self.runner.forward(entries, scheduled.cache_plan)
            if logits is not None:
                tokens_device = self.sampler.sample(logits, params, draws)
        if tokens_device is None:
            return {}
        host = tokens_device.tolist()              # the step's one device-to-host read
        kernels.check_finished_launches()
        return dict(zip(sample_ids, host))

    # ------------------------------------------------------------- generate
    def generate(self, requests: Sequence[GenerateRequest]) -> list[RequestOutput]:
        """Run ``requests`` to the end; outputs in the order given."""
        self._check_usable()
        if self.has_unfinished():
            raise RuntimeError("generate() needs an idle engine")
        ids = [self.submit(r.prompt_token_ids, r.sampling, request_id=r.request_id) for r in requests]
        outputs: dict[int, RequestOutput] = {}
        while True:
            events = self.step()
            for output in events.finished:
                outputs[output.request_id] = output
            if not self.has_unfinished():
                for request in self.scheduler.take_finished():
                    outputs[request.request_id] = RequestOutput.of(request)
                break
        return [outputs[i] for i in ids]

    def close(self) -> None:
        if self._run is not None:                  # steps in flight still write to the cache
            torch.cuda.synchronize()
            self._run = None
        self._closed = True
        self.graphs = None
