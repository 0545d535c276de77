"""Registries of part classes, one for each kind of part.

``register_part("mixer", "gqa_attention", cls)`` makes the class buildable from
``PartSpec("gqa_attention", {...})``; code outside the package (a test, a
plug-in) registers its own parts the same way.
"""

from __future__ import annotations

from typing import Any

from ..config.spec import PartSpec
from .base import BuildContext

GROUPS = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")

_PARTS: dict[str, dict[str, type]] = {group: {} for group in GROUPS}


def register_part(group: str, kind: str, cls: type) -> None:
    if group not in _PARTS:
        raise KeyError(f"unknown part group {group!r}; groups: {', '.join(GROUPS)}")
    _PARTS[group][kind] = cls


def part_kinds(group: str) -> tuple[str, ...]:
    return tuple(sorted(_PARTS[group]))


def build_part(group: str, spec: PartSpec, ctx: BuildContext, **extra: Any):
    """Instance of the class registered for ``spec.kind`` in ``group``."""
    try:
        cls = _PARTS[group][spec.kind]
    except KeyError:
        known = ", ".join(part_kinds(group)) or "none"
        raise KeyError(f"no {group} part named {spec.kind!r}; registered: {known}") from None
    if ctx.build is None:
        ctx.build = build_part
    return cls(ctx, **dict(spec.params), **extra)
