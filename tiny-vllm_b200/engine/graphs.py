"""Decode steps as CUDA graphs.

A step in which every entry is one decoded token runs the same kernels with the
same shapes every time, so for a list of batch sizes the whole step (embedding to
sampled tokens) is captured once and replayed; a step takes the smallest captured
size that holds it, the spare rows being padding (row -1, slot -1: they write
nothing and attend nothing).  The step's metadata and sampling arguments go up
in one copy from pinned memory into the buffers the graph reads.

The reference captures sizes {1, 2, 4, 8, 12, 16} the same way
(tinyvllm/runtime/graphs.py:36-140, padding tinyvllm/runtime/inputs.py:94-98),
sampling outside the graph.
"""

from __future__ import annotations

import numpy as np
import torch

from ..ops import attention as attention_ops
from ..ops import kernels
from ..sampling.sampler import ROW_WORDS, pack_rows, sample_packed
from .capture import capture
from .step import StepContext


class _Bucket:
    """Buffers and graph of one batch size."""

    def __init__(self, runner, size: int, blocks: list[int], far: bool = False) -> None:
        groups = len(runner.manager.groups)
        self.size = size
        self.far = far                    # the graph of a lone request with a long context
        self.blocks = blocks
        sizes = [size, size, size, size, size, size + 1]
        for g in range(groups):
            sizes += [size, size * blocks[g]]
        sizes.append(ROW_WORDS * size)
        self.sizes = sizes
        self.offsets = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])]).astype(np.int64)
        total = int(self.offsets[-1])
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.device = torch.zeros(total, dtype=torch.int32, device=runner.device)
        self.tokens = torch.zeros(size, dtype=torch.int32, device=runner.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits = None
        self.launches = 0
        self.guarded = (False, False)     # kernels with bounded waits inside the graph (gemm_tc, attention_prefill_tc)
        # per group and row: (request and the open() that admitted it, entries written, leading
        # entries given back) of the last step
        self.row_tables = [[None] * size for _ in range(groups)]
        self.copied: torch.cuda.Event | None = None      # the last upload has left the pinned buffer
        self.history: torch.Tensor | None = None         # pinned [steps, size]: the tokens of a run's steps

    def host_view(self, i: int) -> np.ndarray:
        return self.host_np[self.offsets[i]:self.offsets[i] + self.sizes[i]]

    def device_view(self, i: int) -> torch.Tensor:
        return self.device[int(self.offsets[i]):int(self.offsets[i]) + self.sizes[i]]


class DecodeGraphs:
    def __init__(self, runner, batch_sizes, *, max_model_len: int) -> None:
        self.runner = runner
        self.max_model_len = max_model_len
        page = runner.page_size
        self.blocks = [-(-max_model_len // page) for _ in runner.manager.groups]
        chunk = kernels.attention_chunk_keys()
        self.split_chunks = -(-max_model_len // chunk) if max_model_len > chunk else 0
        self.buckets = [_Bucket(runner, size, self.blocks) for size in sorted(set(batch_sizes))]
        # A lone request with a long context has a graph of its own, in which the decode attention
        # cuts it over several clusters a kv head (``ops.attention.far_plan``); which of the two
        # graphs of one row a step replays follows from the request's length, which the host knows.
        self.far_bucket = None
        if 1 in set(batch_sizes) and max_model_len >= attention_ops.FAR_FROM_KEYS:
            self.far_bucket = _Bucket(runner, 1, self.blocks, far=True)
        self._pool = None

    @property
    def largest(self) -> int:
        return self.buckets[-1].size if self.buckets else 0

    def _context(self, bucket: _Bucket) -> StepContext:
        groups = len(self.runner.manager.groups)
        size = bucket.size
        return StepContext(
            storage=self.runner.storage, num_tokens=size, num_rows=size, num_wanted=size,
            token_ids=bucket.device_view(0), positions=bucket.device_view(1),
            token_row=bucket.device_view(2), want_rows=bucket.device_view(3),
            state_slots=bucket.device_view(4), row_starts=bucket.device_view(5),
            slots=[bucket.device_view(6 + 2 * g) for g in range(groups)],
            block_tables=[bucket.device_view(7 + 2 * g).view(size, bucket.blocks[g])
                          for g in range(groups)],
            cache_sources=self.runner.cache_sources, max_position=self.max_model_len - 1,
            split_chunks=self.split_chunks, workspace_of=self.runner._workspace_of,
            decode_only=True, decode_splits=attention_ops.decode_splits(self.max_model_len, size),
            decode_far=bucket.far, max_context=self.max_model_len)

    def _fill_padding(self, bucket: _Bucket) -> None:
        bucket.host_np[:] = 0
        bucket.host_view(1)[:] = -1                     # positions
        bucket.host_view(2)[:] = -1                     # rows
        bucket.host_view(3)[:] = np.arange(bucket.size)  # every row's logits are produced
        bucket.host_view(5)[:] = np.arange(bucket.size + 1)
        for g in range(len(self.runner.manager.groups)):
            bucket.host_view(6 + 2 * g)[:] = -1         # slots: write nothing
        packed = bucket.host_view(len(bucket.sizes) - 1).reshape(ROW_WORDS, bucket.size)
        packed[1] = np.ones(bucket.size, dtype=np.float32).view(np.int32)   # top_p = 1

    def capture(self) -> None:
        """Capture every batch size (largest first, so the graphs share one memory pool)."""
        if self.split_chunks:
            # scratch the blocks' kernels may ask for must exist before anything is recorded
            need = max((block.scratch_floats(self.largest, self.split_chunks)
                        for block in self.runner.model.blocks), default=0)
            if need > 0:
                self.runner.reserve_workspace(need)
        stream = torch.cuda.Stream(device=self.runner.device)
        for bucket in list(reversed(self.buckets)) + ([self.far_bucket] if self.far_bucket is not None else []):
            self._fill_padding(bucket)
            bucket.device.copy_(bucket.host)
            ctx = self._context(bucket)
            packed = bucket.device_view(len(bucket.sizes) - 1).view(ROW_WORDS, bucket.size)
            torch.cuda.synchronize()
            with torch.cuda.stream(stream):
                for _ in range(2):                                   # load kernels, settle allocations
                    sample_packed(self.runner.model.forward(ctx), packed, out=bucket.tokens)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            launched = kernels.launch_count()
            guarded = kernels.guarded_launch_counts()
            with capture(graph, pool=self._pool, stream=stream):
                bucket.logits = self.runner.model.forward(ctx)
                sample_packed(bucket.logits, packed, out=bucket.tokens)
                # the sampled tokens are the next step's input where the host does not upload others
                # (inside a run of steps)
                bucket.device_view(0).copy_(bucket.tokens)
            bucket.launches = kernels.launch_count() - launched
            now = kernels.guarded_launch_counts()
            bucket.guarded = (now[0] > guarded[0], now[1] > guarded[1])
            if self._pool is None:
                self._pool = graph.pool()
            bucket.graph = graph
        torch.cuda.synchronize()

    def launches_per_step(self, rows: int) -> int:
        """Kernels of this package inside the graph that a step of ``rows`` rows replays
        (library matrix products are not counted)."""
        bucket = self.bucket_for(rows)
        return bucket.launches if bucket is not None else 0

    def bucket_for(self, rows: int, longest: int = 0) -> _Bucket | None:
        """The graph of the smallest size that holds ``rows``; ``longest``: tokens of the longest
        request of the step (with its new one)."""
        if (rows == 1 and self.far_bucket is not None and self.far_bucket.graph is not None
                and longest >= attention_ops.FAR_FROM_KEYS):
            return self.far_bucket
        for bucket in self.buckets:
            if bucket.size >= rows and bucket.graph is not None:
                return bucket
        return None

    def _fill(self, bucket: _Bucket, planned, rows: int, tokens, offset: int, params, draws) -> None:
        """Write the fields of one decode step into the bucket's pinned buffer.  ``offset``: how
        many tokens of the plan lie before this step (0 for a plain step); ``tokens`` None leaves
        the token ids as they are (they come from the step before, on the device)."""
        if bucket.copied is not None:
            bucket.copied.synchronize()
        groups = len(self.runner.manager.groups)
        # per-row fields, one array assignment each; rows past the step are padding
        size = bucket.size
        if tokens is not None:
            bucket.host_view(0)[:rows] = tokens
            bucket.host_view(0)[rows:] = 0
        bucket.host_view(1)[:rows] = [p.start + offset for p in planned]
        bucket.host_view(1)[rows:] = -1
        bucket.host_view(2)[:rows] = np.arange(rows)
        bucket.host_view(2)[rows:] = -1
        bucket.host_view(4)[:rows] = [p.state_slot for p in planned]
        for g in range(groups):
            bucket.host_view(6 + 2 * g)[:rows] = [p.slots[g][offset] for p in planned]
            bucket.host_view(6 + 2 * g)[rows:] = -1
            # block tables stay in the buffer from step to step: a row whose request is the one of
            # the step before only gets the entries that were added or given back since
            tables = bucket.host_view(7 + 2 * g).reshape(size, bucket.blocks[g])
            known = bucket.row_tables[g]
            for r, p in enumerate(planned):
                table = p.tables[g]
                before = known[r]
                who = (p.request_id, p.opening)       # an id may come again for another request
                if before is None or before[0] != who or before[1] > len(table):
                    tables[r, :len(table)] = table
                    first_live = 0
                else:
                    tables[r, before[1]:len(table)] = table[before[1]:]
                    first_live = before[2]
                # pages a window gave back read -1 from the first live entry backwards
                while first_live < len(table) and table[first_live] < 0:
                    tables[r, first_live] = -1
                    first_live += 1
                known[r] = (who, len(table), first_live)
            for r in range(rows, size):
                known[r] = None
        packed = bucket.host_view(len(bucket.sizes) - 1).reshape(ROW_WORDS, size)
        packed[:] = pack_rows(params, draws, capacity=size)

    def prepare(self, plan, entries, params, draws) -> "tuple[_Bucket, int] | None":
        """Lower a step of single tokens into the pinned buffer of the smallest graph that holds it
        (host work only); None if no graph does."""
        rows = len(entries)
        bucket = self.bucket_for(rows, max((p.start + 1 for p in plan.entries), default=0))
        if bucket is None:
            return None
        self._fill(bucket, plan.entries, rows, [entry.tokens[0] for entry in entries], 0, params, draws)
        return bucket, rows

    @torch.inference_mode()
    def launch(self, prepared, plan) -> tuple[torch.Tensor, torch.Tensor]:
        """Upload what :meth:`prepare` wrote and replay the graph: (tokens, logits) views of the
        step's rows, valid until the next replay."""
        bucket, rows = prepared
        self.runner.storage.clear_state([p.state_slot for p in plan.entries if p.fresh_state])
        bucket.device.copy_(bucket.host, non_blocking=True)
        bucket.copied = torch.cuda.Event()
        bucket.copied.record()
        bucket.graph.replay()
        kernels.note_guarded_launches(*bucket.guarded)
        return bucket.tokens[:rows], bucket.logits[:rows]

    def run(self, plan, entries, params, draws) -> tuple[torch.Tensor, torch.Tensor] | None:
        """:meth:`prepare` and :meth:`launch` in one call; None if no graph holds the step."""
        prepared = self.prepare(plan, entries, params, draws)
        return None if prepared is None else self.launch(prepared, plan)

    @torch.inference_mode()
    def start_run(self, plan, first_tokens, params, draws, steps: int) -> "RunInFlight | None":
        """``steps`` decode steps of the same requests back to back: the plan holds ``steps`` tokens
        per request, step i runs its i-th.  The tokens a step samples are the next step's input on
        the device (the host only uploads positions, slots and sampling arguments, which it knows
        in advance) and are copied to pinned memory after every step.  The caller launches steps
        (:meth:`RunInFlight.launch`) ahead of the ones it reads (:meth:`RunInFlight.read`), so the
        GPU does not wait for the host between two steps, nor between the last step the host has
        seen and the next.  None if no graph holds the rows."""
        rows = len(first_tokens)
        bucket = self.bucket_for(rows, max((p.start + 1 for p in plan.entries), default=0))
        if bucket is None:
            return None
        self.runner.storage.clear_state([p.state_slot for p in plan.entries if p.fresh_state])
        if bucket.history is None or bucket.history.shape[0] < steps:
            bucket.history = torch.zeros((steps, bucket.size), dtype=torch.int32, pin_memory=True)
        return RunInFlight(self, bucket, plan.entries, rows, list(first_tokens), list(params), list(draws), steps)

    def run_many(self, plan, first_tokens, params, draws, steps: int) -> list[list[int]] | None:
        """All steps of a run launched, then all read: the tokens [steps][rows], or None if no
        graph holds the rows."""
        run = self.start_run(plan, first_tokens, params, draws, steps)
        if run is None:
            return None
        for _ in range(steps):
            run.launch()
        return [run.read() for _ in range(steps)]

    def forget_tables(self, bucket: _Bucket) -> None:
        """The next step uploads every row's block table whole (after a run that was cut short,
        whose last pages went back and may come again in another order)."""
        for known in bucket.row_tables:
            for r in range(len(known)):
                known[r] = None


class RunInFlight:
    """A run of decode steps on one bucket's graph: ``launch`` enqueues the next step, ``read``
    waits for the oldest step not read yet and returns its tokens."""

    def __init__(self, graphs: DecodeGraphs, bucket: _Bucket, planned, rows: int, first_tokens, params, draws,
                 steps: int) -> None:
        self.graphs, self.bucket, self.planned, self.rows = graphs, bucket, planned, rows
        self.first_tokens, self.params, self.draws, self.steps = first_tokens, params, draws, steps
        self.launched = 0
        self.read_steps = 0
        self.done: list[torch.cuda.Event] = []

    @torch.inference_mode()
    def launch(self) -> None:
        if self.launched >= self.steps:
            raise RuntimeError("every step of the run has been launched")
        bucket, index = self.bucket, self.launched
        self.graphs._fill(bucket, self.planned, self.rows, self.first_tokens if index == 0 else None, index,
                          self.params, [d + index for d in self.draws])
        if index == 0:
            bucket.device.copy_(bucket.host, non_blocking=True)
        else:
            ids_end = int(bucket.offsets[1])            # the token ids are there: the graph left them
            bucket.device[ids_end:].copy_(bucket.host[ids_end:], non_blocking=True)
        bucket.copied = torch.cuda.Event()
        bucket.copied.record()
        bucket.graph.replay()
        kernels.note_guarded_launches(*bucket.guarded)
        bucket.history[index].copy_(bucket.tokens, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self.done.append(done)
        self.launched += 1

    def read(self) -> list[int]:
        if self.read_steps >= self.launched:
            raise RuntimeError("no launched step is left to read")
        self.done[self.read_steps].synchronize()
        tokens = self.bucket.history[self.read_steps, :self.rows].tolist()
        self.read_steps += 1
        return tokens
