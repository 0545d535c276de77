"""The step function: one flat batch through the model, from the cache.

A step is a list of entries (request, its next tokens, the places among them
whose logits are wanted).  Portions of prompts stand beside single decoded
tokens, cut anywhere.  The step runs only the tokens it is given, writes their
keys and values into the pages the cache manager assigns, and returns the
logits at the wanted places as float32 ``[wanted, vocab]``.

Counterparts in the reference: the flat batch of tinyvllm/batch.py:100-136, the
device inputs of tinyvllm/runtime/contracts.py:47-145 and
tinyvllm/runtime/inputs.py:14-137, the checks of tinyvllm/runtime/runner.py:101-193
and ``ModelRunner.run`` (:196-246).  Differences: metadata is int32 and goes up
in one copy for every kind of batch; logits can be wanted at any place of an
entry, not only its last token; there is no per-request loop on the host.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, StepCachePlan
from ..cache.storage import CacheStorage, bytes_per_page, group_runs
from ..ops import attention as attention_ops
from ..ops import kernels
from .capture import capture

log = logging.getLogger("tinyvllm_b200")


class StepError(ValueError):
    """A step was asked for something the engine cannot run."""


class OutOfPages(RuntimeError):
    """The page pool cannot hold the tokens of this step."""


@dataclass(frozen=True)
class StepEntry:
    request_id: object
    tokens: tuple[int, ...]
    want: tuple[int, ...] = ()          # places among ``tokens`` whose logits are wanted


@dataclass
class StepContext:
    """Everything a part may read about the running step (device tensors are int32)."""

    storage: CacheStorage
    num_tokens: int
    num_rows: int
    num_wanted: int
    token_ids: torch.Tensor              # [tokens]
    positions: torch.Tensor              # [tokens] absolute position of each token
    token_row: torch.Tensor              # [tokens] index of the token's entry, -1 for padding
    want_rows: torch.Tensor              # [wanted] flat token index of each wanted place
    state_slots: torch.Tensor            # [rows] state slot of each entry
    row_starts: torch.Tensor             # [rows + 1] first flat token of each entry
    slots: list[torch.Tensor]            # per group [tokens]: cache slot each token is written to
    block_tables: list[torch.Tensor]     # per group [rows, blocks]
    cache_sources: tuple                 # per run: the run whose cache it reads, or None
    max_position: int                    # largest position in the step (bounds the split of attention)
    split_chunks: int                    # 0: walk the keys per row; n: spread n chunks over the grid
    workspace_of: object = None          # callable(floats) -> float32 scratch tensor
    decode_only: bool = False            # every entry is a single token
    decode_splits: int = 0               # pieces the fused decode attention cuts a context into
    decode_far: bool = False             # a lone request with a long context: several clusters a kv head
    max_context: int = 0                 # no request grows beyond this many tokens
    tile_row: torch.Tensor | None = None     # tiles of consecutive query tokens for the tile kernel:
    tile_first: torch.Tensor | None = None   # request row, first flat token and token count of each
    tile_count: torch.Tensor | None = None
    tile_tc_row: torch.Tensor | None = None      # the same for the tcgen05 tile kernel (tiles of up to 128
    tile_tc_first: torch.Tensor | None = None    # tokens, longest context first); a token is in one of the
    tile_tc_count: torch.Tensor | None = None    # two sets
    # host copies, for parts that plan on the host (and for tests)
    host_rows: tuple = ()                # (request_id, first position, count, state_slot, fresh) per entry
    single_runs: tuple = ()              # (first flat token, count) of runs of single-token entries beside
                                         # prompt portions: not in the tile lists, the row kernel takes them
    signature: tuple = ()                # sizes and flags that fix the step's launches (two steps with the
                                         # same signature differ in the contents of their tensors only)
    arena: torch.Tensor | None = None    # the int32 tensor all the fields above are views of

    def writes_cache(self, run: int) -> bool:
        return self.cache_sources[run] is None

    def workspace(self, floats: int) -> torch.Tensor:
        return self.workspace_of(floats)



# block-table widths are multiples of this many pages
TABLE_WIDTH_GRAIN = 8


@dataclass
class _StepGraph:
    """A captured step: the graph, the tensor its fields are copied into, its logits."""

    graph: object
    arena: torch.Tensor
    logits: torch.Tensor | None
    ctx: StepContext                      # keeps the views the graph reads alive
    last_used: int = 0                    # step count at its last replay
    guarded: tuple = (False, False)       # kernels with bounded waits inside (gemm_tc, attention_prefill_tc)


@dataclass
class PreparedStep:
    """A lowered step: its context on the device, the graph that replays it (if one was captured
    for its signature) and whether it is to be captured after it has run."""

    ctx: StepContext
    graph: _StepGraph | None = None
    capture: bool = False


class StepRunner:
    """Model + cache + the step function that generation, replay and tests all use."""

    def __init__(self, model, *, page_size: int, num_pages, max_requests: int,
                 max_model_len: int | None = None) -> None:
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.page_size = page_size
        self.max_model_len = min(max_model_len or model.spec.max_positions, model.spec.max_positions)
        needs = model.cache_needs()
        self.cache_sources = tuple(model.cache_sources())
        groups, where = group_runs(needs, list(self.cache_sources))
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(groups)
        self.manager = CacheManager(groups, page_size, list(num_pages), max_requests)
        self.storage = CacheStorage(groups, where, needs, page_size=page_size,
                                    pages_per_group=list(num_pages), num_state_slots=max_requests,
                                    dtype=self.dtype, device=self.device)
        self.vocab_size = model.spec.vocab_size
        self._pinned: torch.Tensor | None = None
        self._pinned_free: torch.cuda.Event | None = None
        self._workspace: torch.Tensor | None = None
        self._retired_workspaces: list[torch.Tensor] = []
        self._step_graph_limit = 0
        self._step_graphs: dict[tuple, _StepGraph] = {}
        self._step_seen: dict[tuple, int] = {}
        self._step_graph_pool = None
        self._step_graph_stream = None
        self._step_count = 0
        self._last_capture_at = -(1 << 30)
        self.decode_splits = attention_ops.decode_splits(self.max_model_len)
        # prefill tiles are cut for the tcgen05 attention kernel if every block says it takes them
        blocks = getattr(model, "blocks", ())
        self.tensor_memory_tiles = self.dtype == torch.bfloat16 and len(blocks) > 0 and all(
            getattr(block, "takes_tensor_memory_tiles", lambda page: False)(page_size)
            for block in blocks)

    # ------------------------------------------------------------- sizing
    @staticmethod
    def bytes_per_token(model, dtype: torch.dtype) -> int:
        """Cache bytes one token takes in all groups (windows count as full here)."""
        needs = model.cache_needs()
        groups, _ = group_runs(needs, model.cache_sources())
        return sum(bytes_per_page(g, 1, torch.empty((), dtype=dtype).element_size()) for g in groups)

    # ----------------------------------------------------------- requests
    def open(self, request_id) -> int:
        return self.manager.open(request_id)

    def close(self, request_id) -> None:
        self.manager.close(request_id)

    # ------------------------------------------------------------ scratch
    def _workspace_of(self, floats: int) -> torch.Tensor:
        if self._workspace is None or self._workspace.numel() < floats:
            if torch.cuda.is_current_stream_capturing():
                raise StepError("scratch memory must be sized before a graph is captured")
            if self._workspace is not None:
                self._retired_workspaces.append(self._workspace)      # captured graphs may still name it
            self._workspace = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=self.device)
        return self._workspace

    def reserve_workspace(self, floats: int) -> None:
        self._workspace_of(floats)

    # --------------------------------------------------------------- steps
    def validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        for entry in entries:
            if not entry.tokens:
                raise StepError(f"request {entry.request_id!r}: an entry needs at least one token")
            if not self.manager.is_open(entry.request_id):
                raise StepError(f"request {entry.request_id!r} is not open")
            for token in entry.tokens:
                if type(token) is not int or not 0 <= token < self.vocab_size:
                    raise StepError(f"request {entry.request_id!r}: {token!r} is not a token id "
                                    f"below {self.vocab_size}")
            for place in entry.want:
                if type(place) is not int or not 0 <= place < len(entry.tokens):
                    raise StepError(f"request {entry.request_id!r}: wanted place {place!r} is not "
                                    f"among its {len(entry.tokens)} tokens")
            end = self.manager.length(entry.request_id) + len(entry.tokens)
            if end > self.max_model_len:
                raise StepError(f"request {entry.request_id!r} would reach {end} tokens, "
                                f"the limit is {self.max_model_len}")

    def plan(self, entries: Sequence[StepEntry]) -> StepCachePlan | None:
        """Check the entries and take their pages; None when pages run out."""
        self.validate(entries)
        return self.manager.plan([(e.request_id, len(e.tokens)) for e in entries])

    def build_context(self, entries: Sequence[StepEntry], plan: StepCachePlan,
                      *, split_chunks: int | None = None, arena_of=None) -> StepContext:
        """Lower entries + cache plan to device tensors (one pinned buffer, one copy).

        ``arena_of(signature, count)`` may name the int32 device tensor the step's fields are
        copied into (a captured graph reads its own); else a new one is allocated."""
        rows = len(entries)
        counts = [len(e.tokens) for e in entries]
        tokens = sum(counts)
        wanted = sum(len(e.want) for e in entries)
        groups = len(self.manager.groups)
        # block tables as wide as the longest, rounded up so that steps of growing requests share a shape
        blocks = [-(-max(1, max(len(p.tables[g]) for p in plan.entries)) // TABLE_WIDTH_GRAIN) * TABLE_WIDTH_GRAIN
                  for g in range(groups)]
        decode_only = all(count == 1 for count in counts)
        # only the bfloat16 tile kernel reads tile lists; the 32-bit path walks rows
        tiled = not decode_only and self.storage.dtype == torch.bfloat16
        if tiled:
            tc_lists, tile_lists, single_runs = attention_ops.prefill_tiles(
                counts, [p.start for p in plan.entries], tensor_memory=self.tensor_memory_tiles,
                singles_apart=True)
        else:
            tc_lists, tile_lists, single_runs = ([], [], []), ([], [], []), ()
        sizes = [tokens, tokens, tokens, wanted, rows, rows + 1]
        for g in range(groups):
            sizes += [tokens, rows * blocks[g]]
        tiles_at = len(sizes)
        sizes += [len(tile_lists[0])] * 3 + [len(tc_lists[0])] * 3
        offsets = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])
        host = np.zeros(int(offsets[-1]), dtype=np.int32)

        def view(i):
            return host[offsets[i]:offsets[i] + sizes[i]]

        cursor, wanted_cursor, max_position = 0, 0, 0
        row_starts = view(5)
        for r, (entry, planned) in enumerate(zip(entries, plan.entries)):
            n = counts[r]
            view(0)[cursor:cursor + n] = entry.tokens
            view(1)[cursor:cursor + n] = np.arange(planned.start, planned.start + n, dtype=np.int32)
            view(2)[cursor:cursor + n] = r
            for place in entry.want:
                view(3)[wanted_cursor] = cursor + place
                wanted_cursor += 1
            view(4)[r] = planned.state_slot
            row_starts[r] = cursor
            for g in range(groups):
                view(6 + 2 * g)[cursor:cursor + n] = planned.slots[g]
                table = planned.tables[g]
                view(7 + 2 * g)[r * blocks[g]:r * blocks[g] + len(table)] = table
            max_position = max(max_position, planned.start + n - 1)
            cursor += n
        row_starts[rows] = cursor
        for i in range(3):
            view(tiles_at + i)[:] = tile_lists[i]
            view(tiles_at + 3 + i)[:] = tc_lists[i]

        if split_chunks is None:
            split_chunks = attention_ops.choose_split(tokens, max_position)
        # all that decides which kernels a step launches and with which sizes
        decode_far = decode_only and rows == 1 and max_position + 1 >= attention_ops.FAR_FROM_KEYS
        signature = (tuple(sizes), decode_only, split_chunks, single_runs, decode_far)
        device = self._upload(host, None if arena_of is None else arena_of(signature, host.shape[0]))

        def dview(i):
            return device[int(offsets[i]):int(offsets[i]) + sizes[i]]

        fresh = [p.state_slot for p in plan.entries if p.fresh_state]
        self.storage.clear_state(fresh)
        return StepContext(
            storage=self.storage, num_tokens=tokens, num_rows=rows, num_wanted=wanted,
            token_ids=dview(0), positions=dview(1), token_row=dview(2), want_rows=dview(3),
            state_slots=dview(4), row_starts=dview(5),
            slots=[dview(6 + 2 * g) for g in range(groups)],
            block_tables=[dview(7 + 2 * g).view(rows, blocks[g]) for g in range(groups)],
            cache_sources=self.cache_sources, max_position=max_position, split_chunks=split_chunks,
            workspace_of=self._workspace_of, decode_only=decode_only,
            decode_splits=attention_ops.decode_splits(self.max_model_len, rows), max_context=self.max_model_len,
            decode_far=decode_far,
            tile_row=dview(tiles_at) if tiled else None,
            tile_first=dview(tiles_at + 1) if tiled else None,
            tile_count=dview(tiles_at + 2) if tiled else None,
            tile_tc_row=dview(tiles_at + 3) if tiled else None,
            tile_tc_first=dview(tiles_at + 4) if tiled else None,
            tile_tc_count=dview(tiles_at + 5) if tiled else None,
            host_rows=tuple((p.request_id, p.start, p.count, p.state_slot, p.fresh_state)
                            for p in plan.entries),
            signature=signature, arena=device, single_runs=single_runs,
        )

    def _upload(self, host: np.ndarray, device: torch.Tensor | None = None) -> torch.Tensor:
        count = host.shape[0]
        if self._pinned is None or self._pinned.numel() < count:
            if self._pinned_free is not None:
                self._pinned_free.synchronize()
            self._pinned = torch.empty(max(count, 1 << 16), dtype=torch.int32, pin_memory=True)
            self._pinned_free = None
        if self._pinned_free is not None:
            self._pinned_free.synchronize()          # the previous step's copy has left the buffer
        self._pinned[:count].numpy()[:] = host
        if device is None:
            device = torch.empty(count, dtype=torch.int32, device=self.device)
        device.copy_(self._pinned[:count], non_blocking=True)
        self._pinned_free = torch.cuda.Event()
        self._pinned_free.record()
        return device

    def execute(self, ctx: StepContext) -> torch.Tensor | None:
        return self.model.forward(ctx)

    # ------------------------------------------------- steps as CUDA graphs
    # A capture costs about two eager steps (the step runs once more on the capture stream, then
    # its launches are recorded and the graph is instantiated), a replay saves about half of one:
    # a shape is captured when it has come CAPTURE_AT_OCCURRENCE times, at most one capture in
    # CAPTURE_EVERY_STEPS steps, and a graph that was replayed within the last KEEP_FOR_STEPS steps
    # is not thrown out for a newcomer.
    CAPTURE_AT_OCCURRENCE = 3
    CAPTURE_EVERY_STEPS = 8
    KEEP_FOR_STEPS = 64

    def enable_step_graphs(self, limit: int = 16) -> None:
        """Steps whose signature (token, row, block and tile counts) keeps coming back are captured
        as CUDA graphs (at their third occurrence) and replayed from then on: the host then issues
        one launch instead of some ten a layer.  At most ``limit`` graphs are kept (one that has not
        been replayed for a while makes room); they share one memory pool.  Only for models whose
        parts do all per-step work in kernels (no host-side planning from ``host_rows``)."""
        self._step_graph_limit = limit
        self._last_capture_at = -(1 << 30)

    @torch.inference_mode()
    def prepare(self, entries: Sequence[StepEntry], plan: StepCachePlan) -> "PreparedStep":
        """Lower a step: its fields go into pinned memory and up to the device, and a captured graph
        is looked up.  No kernel that touches the cache or the model is launched here, so a failure
        in this half leaves nothing to undo but the cache plan."""
        if self._step_graph_limit <= 0:
            return PreparedStep(self.build_context(entries, plan), None, False)
        chosen = {}

        def arena_of(signature, count):
            self._step_count += 1
            graph = self._step_graphs.get(signature)
            if graph is not None:
                graph.last_used = self._step_count
                chosen["graph"] = graph
                return graph.arena
            seen = self._step_seen.get(signature, 0) + 1
            if len(self._step_seen) > 4096:
                self._step_seen.clear()
            self._step_seen[signature] = seen
            if seen < self.CAPTURE_AT_OCCURRENCE or self._step_count - self._last_capture_at < self.CAPTURE_EVERY_STEPS:
                return None
            if len(self._step_graphs) >= self._step_graph_limit:
                # the graph that has waited longest for its shape to come back makes room, unless
                # even that one was replayed a moment ago
                oldest = min(self._step_graphs, key=lambda key: self._step_graphs[key].last_used)
                if self._step_count - self._step_graphs[oldest].last_used < self.KEEP_FOR_STEPS:
                    return None
                del self._step_graphs[oldest]
                if not self._step_graphs:
                    self._step_graph_pool = None      # the pool went with its last graph
            self._last_capture_at = self._step_count
            chosen["capture"] = True
            return torch.empty(count, dtype=torch.int32, device=self.device)

        ctx = self.build_context(entries, plan, arena_of=arena_of)
        return PreparedStep(ctx, chosen.get("graph"), bool(chosen.get("capture")))

    @torch.inference_mode()
    def launch(self, prepared: "PreparedStep") -> torch.Tensor | None:
        """Run a prepared step: the logits at its wanted places (None if there are none)."""
        graph = prepared.graph
        if graph is not None:
            graph.graph.replay()
            # the replay launched the kernels with bounded waits behind the back of their wrappers
            kernels.note_guarded_launches(*graph.guarded)
            return graph.logits
        logits = self.execute(prepared.ctx)
        if prepared.capture and self._step_graph_limit > 0:
            self._capture_step(prepared.ctx)
        return logits

    def forward(self, entries: Sequence[StepEntry], plan: StepCachePlan) -> torch.Tensor | None:
        """The step's logits, through a captured graph if this kind of step has one."""
        return self.launch(self.prepare(entries, plan))

    def _capture_step(self, ctx: StepContext) -> None:
        """Record the launches of a step that has just run eagerly on ``ctx``.  The step runs once
        more, on the capture stream, before it is recorded (libraries settle their per-stream
        work areas outside the capture; the same keys and values go to the same cache slots), and
        nothing runs while it is recorded.  Graphs are an optimisation: if the capture fails, the
        runner stays eager from then on and the step's eager logits stand."""
        if self._step_graph_stream is None:
            self._step_graph_stream = torch.cuda.Stream(device=self.device)
        stream = self._step_graph_stream
        before = kernels.guarded_launch_counts()
        try:
            stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(stream):
                self.model.forward(ctx)
            stream.synchronize()
            after = kernels.guarded_launch_counts()
            graph = torch.cuda.CUDAGraph()
            with capture(graph, pool=self._step_graph_pool, stream=stream):
                logits = self.model.forward(ctx)
        except Exception as failure:                      # noqa: BLE001 (whatever a part or CUDA raises)
            self._step_graph_limit = 0
            self._step_graphs.clear()
            self._step_graph_pool = None
            log.warning("a step could not be captured as a CUDA graph (%r); steps run eagerly from now on",
                        failure)
            try:
                torch.cuda.synchronize(self.device)
            except Exception:                             # noqa: BLE001 (reported by the next real call)
                pass
            return
        if self._step_graph_pool is None:
            self._step_graph_pool = graph.pool()
        guarded = (after[0] > before[0], after[1] > before[1])      # what one pass of the step launched
        ctx.workspace_of = None       # a replay asks for no scratch; without it the graph does not hold the runner
        self._step_graphs[ctx.signature] = _StepGraph(graph, ctx.arena, logits, ctx, self._step_count, guarded)

    def drop_graphs(self) -> None:
        """Forget every captured step (their device memory goes back to the allocator)."""
        self._step_graphs.clear()
        self._step_graph_pool = None
        self._step_seen.clear()

    @torch.inference_mode()
    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Plan, run and commit one step; raises :class:`OutOfPages` if it does not fit."""
        entries = list(entries)
        plan = self.plan(entries)
        if plan is None:
            raise OutOfPages(
                "the page pool is too small for this step: "
                + ", ".join(f"group {g} has {self.manager.free_pages(g)} free pages"
                            for g in range(len(self.manager.groups))))
        try:
            logits = self.forward(entries, plan)
        except BaseException:
            self.manager.rollback(plan)
            raise
        self.manager.commit(plan)
        return logits
