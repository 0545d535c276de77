"""Interfaces of the parts a model is put together from.

A part is built from the parameters of its :class:`PartSpec` plus the build
context (device, storage dtype, checkpoint prefix).  It declares its tensors
as :class:`ParamSpec` (checkpoint names, shapes, packing), what cache it needs,
and runs on the tensors of one step.  No part knows the model it is in.

Kinds of parts and what each must offer
---------------------------------------
norm            ``forward(x) -> y`` and ``add(x, residual) -> (y, new_residual)``,
                optionally ``add_rows(x, residual, rows) -> y`` on chosen rows.  A norm
                that is y = x * rsqrt(mean(x^2) + eps) * weight with attributes
                ``weight`` [width] and ``eps`` may set ``folds_into_product = True``:
                a projection right behind it may then apply it inside its own kernel
position        built by the mixer that names it in its spec; ``finalize()`` makes its
                tables.  One whose tables the fused q/k kernels are to apply has
                float32 ``cos`` and ``sin`` [positions, head_dim / 2] and declares
                ``pairing = "half_split"``; any other pairing is refused by those
                kernels with a clear error (it needs a kernel, or a mixer, of its own)
mixer           ``cache_need() -> KVNeed | StateNeed | None`` and
                ``forward(x, ctx, run) -> y`` where ``ctx`` is the step's
                :class:`StepContext` and ``run`` the index in the run list;
                optionally ``forward_normed(hidden, residual, norm, ctx, run)
                -> (y, new_residual)`` (takes its pre-norm into its first
                projection; ``hidden`` is None when the part before added its
                output to the residual itself, and ``y`` may be None for the
                same reason), ``streamed_weights()`` (the large weights in the
                order a step reads them), ``takes_tensor_memory_tiles(page_size)``
                and ``scratch_floats(rows, chunks) -> int`` (float32 scratch its
                kernels may ask of ``ctx.workspace`` for a step of ``rows`` single
                tokens whose keys are cut into ``chunks`` chunks; it is set aside
                before decode steps are captured as graphs)
feed_forward    ``forward(x, ctx) -> y``, optionally ``forward_normed`` and
                ``streamed_weights`` as above
block           ``forward(hidden, residual, ctx, run) -> (hidden, residual)``;
                ``residual`` is None for the first block, ``hidden`` is None
                (on the way in or out) when it is in the residual already.
                The engine asks the block, never its insides: ``cache_need()``
                (one per run of the block), ``takes_tensor_memory_tiles(page_size)``
                and ``scratch_floats(rows, chunks)``; :class:`Block` answers them
                from an attribute ``mixer``, a block arranged otherwise answers
                them itself
embedding       ``forward(token_ids) -> hidden``
head            ``forward(hidden_rows) -> logits`` (float32)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class ParamSource:
    """One checkpoint tensor and the rows of the destination it fills."""

    name: str
    row_start: int
    rows: int


@dataclass(frozen=True)
class ParamSpec:
    """One device tensor of a part.

    ``sources`` lists the checkpoint tensors that are packed along the first
    dimension.  ``role``: "matrix" and "table" tensors take the storage dtype;
    a "vector" that the file stores in 32-bit stays in 32-bit; "integer"
    tensors become int32.  ``init`` is the law of the random-weights mode:
    "normal" draws N(0, 0.02), "around_one" draws 1 + U(-0.1, 0.1).
    """

    attr: str
    shape: tuple[int, ...]
    sources: tuple[ParamSource, ...]
    role: str = "matrix"
    init: str = "normal"

    @staticmethod
    def single(attr: str, name: str, shape: tuple[int, ...], *, role: str = "matrix",
               init: str = "normal") -> "ParamSpec":
        return ParamSpec(attr, shape, (ParamSource(name, 0, shape[0]),), role, init)

    @staticmethod
    def packed(attr: str, names_rows: list[tuple[str, int]], cols: int) -> "ParamSpec":
        sources, start = [], 0
        for name, rows in names_rows:
            sources.append(ParamSource(name, start, rows))
            start += rows
        return ParamSpec(attr, (start, cols), tuple(sources))


@dataclass(frozen=True)
class KVNeed:
    """A growing cache of keys and values, ``window`` keys long if given."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, zero when a request starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class BuildContext:
    """What every part constructor receives besides its own parameters."""

    device: torch.device
    dtype: torch.dtype          # storage dtype: torch.bfloat16 or torch.float32
    prefix: str = ""            # checkpoint prefix of the layer, "" for top-level parts
    build: Callable[..., Any] | None = None   # build(kind_group, PartSpec, ctx) for nested parts

    def child(self, name: str) -> "BuildContext":
        prefix = f"{self.prefix}.{name}" if self.prefix else name
        return BuildContext(self.device, self.dtype, prefix, self.build)


class Part:
    """Base of all parts: tensors by declaration, nested parts by listing."""

    def param_specs(self) -> list[ParamSpec]:
        return []

    def children(self) -> list["Part"]:
        return []

    def bind(self, attr: str, tensor: torch.Tensor) -> None:
        setattr(self, attr, tensor)

    def all_parts(self) -> list["Part"]:
        found = [self]
        for child in self.children():
            found.extend(child.all_parts())
        return found


class Block(Part):
    """Base of block arrangements.  The engine talks to a block only through these methods and
    ``forward``; the defaults pass the questions on to ``self.mixer``."""

    mixer = None

    def cache_need(self):
        """What one run of this block needs of the cache: KVNeed, StateNeed or None."""
        return self.mixer.cache_need() if self.mixer is not None else None

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        """Whether prompt portions of this block may be cut into the tile lists of the
        tensor-memory attention kernel (a block without attention does not care: True)."""
        if self.mixer is None:
            return True
        asked = getattr(self.mixer, "takes_tensor_memory_tiles", None)
        return bool(asked(page_size)) if asked is not None else False

    def scratch_floats(self, rows: int, chunks: int) -> int:
        asked = getattr(self.mixer, "scratch_floats", None) if self.mixer is not None else None
        return int(asked(rows, chunks)) if asked is not None else 0
