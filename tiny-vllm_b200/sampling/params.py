"""Per-request sampling parameters; names, defaults and checks of tinyvllm/request.py:32-75."""

from __future__ import annotations

import math
from dataclasses import dataclass

_MAX_SEED = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 64
    temperature: float = 0.0        # 0 = greedy
    ignore_eos: bool = False
    seed: int = 0
    top_k: int = 0                  # 0 = off
    top_p: float = 1.0              # 1 = off

    def __post_init__(self) -> None:
        for name in ("max_new_tokens", "seed", "top_k"):
            value = getattr(self, name)
            if type(value) is not int or value < 0:
                raise ValueError(f"{name} must be a non-negative integer")
        if self.seed > _MAX_SEED:
            raise ValueError("seed must fit in 64 bits")
        if type(self.temperature) not in (int, float):
            raise TypeError("temperature must be a number")
        temperature = float(self.temperature)
        if not math.isfinite(temperature) or temperature < 0.0:
            raise ValueError("temperature must be finite and non-negative")
        object.__setattr__(self, "temperature", temperature)
        if type(self.top_p) not in (int, float):
            raise TypeError("top_p must be a number")
        top_p = float(self.top_p)
        if not math.isfinite(top_p) or not 0.0 < top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        object.__setattr__(self, "top_p", top_p)
        if type(self.ignore_eos) is not bool:
            raise TypeError("ignore_eos must be bool")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
