"""The description of a model as data.

A :class:`ModelSpec` names, layer by layer, which mixer, feed-forward, norm and
block arrangement to build and with which sizes and constants, and in which
order the layers run.  An architecture is a function from its typed
configuration to such a spec; nothing below the spec knows the architecture.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part to build: a registry key and the keyword arguments of its class."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **more: Any) -> "PartSpec":
        return PartSpec(self.kind, {**self.params, **more})


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its checkpoint prefix, its arrangement and its parts."""

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec


@dataclass(frozen=True)
class RunStep:
    """One entry of the run list.

    ``layer`` indexes :attr:`ModelSpec.layers`; the same layer may be named by
    several entries, each run then has a cache of its own.  ``cache_from``
    names an earlier entry of the run list whose cache this run reads instead
    of writing one.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.order:
            raise ValueError("the run list is empty")
        for index, step in enumerate(self.order):
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"run {index} names layer {step.layer}, which does not exist")
            if step.cache_from is not None:
                if not 0 <= step.cache_from < index:
                    raise ValueError(
                        f"run {index} reads the cache of run {step.cache_from}, "
                        "which is not an earlier run"
                    )
                if self.order[step.cache_from].cache_from is not None:
                    raise ValueError(
                        f"run {index} reads the cache of run {step.cache_from}, "
                        "which has no cache of its own"
                    )
