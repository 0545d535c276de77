"""Architectures of the package; importing a module registers its architecture."""

from . import qwen3  # noqa: F401
from .qwen3 import Qwen3Config

__all__ = ["Qwen3Config"]
