"""The parts a model is put together from, and their registries."""

from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (they register themselves)
from .base import Block, BuildContext, KVNeed, ParamSource, ParamSpec, Part, StateNeed
from .registry import build_part, part_kinds, register_part

__all__ = ["Block", "BuildContext", "KVNeed", "ParamSource", "ParamSpec", "Part", "StateNeed",
           "build_part", "part_kinds", "register_part"]
