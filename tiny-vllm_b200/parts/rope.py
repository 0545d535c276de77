"""Rotary position encoding, half-split pairing.

inv_freq_j = theta^(-2j/d) and the angle p * inv_freq_j are float32; cos and sin
are tabulated in float32 for every position up to ``max_positions``
(tinyvllm/layers.py:167-226).  The rotation itself is part of the mixer's fused
q/k kernel, which reads these tables at the step's positions (the reference
gathers and casts them per step, tinyvllm/layers.py:229-245).
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import BuildContext, Part
from .registry import register_part

_TABLES: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


class RopeHalfSplit(Part):
    # How the fused q/k kernels pair the elements of a head: element j of the first half with
    # element j of the second, rotated by position * inv_freq_j read from the float32 tables
    # ``cos`` and ``sin``.  A position part with another pairing must not hand its tables to them.
    pairing = "half_split"

    def __init__(self, ctx: BuildContext, *, head_dim: int, theta: float, max_positions: int) -> None:
        if head_dim % 2:
            raise ValueError("rotary encoding needs an even head size")
        self.head_dim = head_dim
        self.theta = float(theta)
        self.max_positions = max_positions
        self.device = ctx.device
        self.cos = self.sin = None

    def inverse_frequencies(self) -> torch.Tensor:
        """theta^(-2j/d) in float32, the reference's expression (tinyvllm/layers.py:192-205)."""
        exponent = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim
        return 1.0 / (self.theta ** exponent)

    def finalize(self) -> None:
        """Tabulate once per (sizes, device); layers with equal parameters share the tables."""
        key = (self.head_dim, self.theta, self.max_positions, str(self.device))
        if key not in _TABLES:
            inv_freq = self.inverse_frequencies().to(self.device)
            _TABLES[key] = kernels.rope_tables(inv_freq, self.max_positions)
        self.cos, self.sin = _TABLES[key]


register_part("position", "rope_half_split", RopeHalfSplit)
