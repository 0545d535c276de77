"""Weights by tensor name from safetensors files.

The model hands over the (part, ParamSpec) pairs it is made of; every
checkpoint tensor is copied into the rows of the device tensor it belongs to
(q/k/v and gate/up are packed that way), in the storage dtype, and bound to
the part.  Everything that is wrong with a folder is reported in ONE
:class:`WeightsError`: missing tensors, unexpected tensors and wrong shapes.

Shard discovery and the by-name loop follow tinyvllm/checkpoint.py:25-81 and
:84-143; the name routes follow tinyvllm/models/qwen3.py:569-648.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable

import torch

from ..parts.base import ParamSpec, Part


class WeightsError(RuntimeError):
    """A model folder does not hold the tensors the model needs."""

    def __init__(self, folder, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.wrong_shape = tuple(wrong_shape)
        self.other = tuple(other)
        lines = [f"cannot load weights from {folder}:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        lines.extend(f"  {text}" for text in self.other)
        super().__init__("\n".join(lines))


def shard_files(folder: Path) -> list[Path]:
    """The safetensors files of a folder: those an index names, else all."""
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        try:
            names = sorted(set(json.loads(index.read_text(encoding="utf-8"))["weight_map"].values()))
        except (OSError, ValueError, KeyError, AttributeError, TypeError) as exc:
            raise WeightsError(folder, other=[f"invalid index {index.name}: {exc}"]) from exc
        files = [folder / name for name in names]
        absent = [p.name for p in files if not p.is_file()]
        if absent:
            raise WeightsError(folder, other=["index names absent files: " + ", ".join(absent)])
        return files
    files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise WeightsError(folder, other=["no .safetensors file in the folder"])
    return files


def storage_dtype_of(spec: ParamSpec, stored: torch.dtype, dtype: torch.dtype) -> torch.dtype:
    """Device dtype of a tensor: integers int32; a vector stored in 32-bit stays
    32-bit; everything else takes the storage dtype."""
    if spec.role == "integer" or not stored.is_floating_point:
        return torch.int32
    if spec.role == "vector" and stored == torch.float32:
        return torch.float32
    return dtype


def _routes(targets: Iterable[tuple[Part, ParamSpec]]):
    routes = {}
    for part, spec in targets:
        for source in spec.sources:
            if source.name in routes:
                raise ValueError(f"two parts claim the checkpoint tensor {source.name}")
            routes[source.name] = (part, spec, source)
    return routes


def bind_tensors(targets, named_tensors, *, dtype, device, folder="<memory>",
                 optional: Iterable[str] = (), aliases: dict[str, str] | None = None) -> None:
    """Fill and bind every declared tensor from ``named_tensors`` (name -> CPU or
    device tensor, or an iterable of such pairs).  ``optional`` names may be
    present without being used.  ``aliases`` maps a name a file may use to the
    declared name it stands for: the tensor fills the declared one (the one that
    comes later in the file wins if both are there) and the declared one counts
    as present.  A tied head stored as ``lm_head.weight`` fills the embedding that
    way, as the reference does (tinyvllm/models/qwen3.py:637-641, :682-686)."""
    targets = list(targets)
    routes = _routes(targets)
    optional = set(optional)
    aliases = dict(aliases or {})
    destinations: dict[tuple[int, str], torch.Tensor] = {}
    in_file, seen, unexpected, wrong = set(), set(), [], []
    items = named_tensors.items() if hasattr(named_tensors, "items") else named_tensors
    for name, tensor in items:
        if name in in_file:
            raise WeightsError(folder, other=[f"tensor {name} appears twice"])
        in_file.add(name)
        if name in aliases and aliases[name] in routes:
            name = aliases[name]
        seen.add(name)
        route = routes.get(name)
        if route is None:
            if name not in optional:
                unexpected.append(name)
            continue
        part, spec, source = route
        want = (source.rows,) + tuple(spec.shape[1:])
        if tuple(tensor.shape) != want:
            wrong.append((name, want, tuple(tensor.shape)))
            continue
        key = (id(part), spec.attr)
        if key not in destinations:
            destinations[key] = torch.empty(
                spec.shape, dtype=storage_dtype_of(spec, tensor.dtype, dtype), device=device)
        destinations[key][source.row_start:source.row_start + source.rows].copy_(tensor)
    missing = sorted(name for name in routes if name not in seen)
    if missing or unexpected or wrong:
        raise WeightsError(folder, missing, sorted(unexpected), wrong)
    for part, spec in targets:
        part.bind(spec.attr, destinations[(id(part), spec.attr)])


def load_checkpoint(targets, folder, *, dtype, device, optional=(), aliases=None) -> None:
    """Read every shard of ``folder`` and bind the tensors to their parts."""
    from safetensors import safe_open

    folder = Path(folder)

    def stream():
        for path in shard_files(folder):
            with safe_open(str(path), framework="pt", device="cpu") as shard:
                for name in shard.keys():
                    yield name, shard.get_tensor(name)

    bind_tensors(targets, stream(), dtype=dtype, device=device, folder=folder, optional=optional,
                 aliases=aliases)
