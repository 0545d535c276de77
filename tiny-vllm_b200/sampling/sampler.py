"""Next tokens from logits rows: greedy, temperature, top-k, top-p.

One kernel launch samples all rows, each with its own parameters
(``csrc/sampling.cu``).  The noise of a draw depends on the request's seed and
on how many tokens the request has drawn before, nothing else, so a request's
tokens do not change with the batch it runs in.  The reference keeps one
``torch.Generator`` per request instead (tinyvllm/sampling.py:167-185) and
samples with torch operations (:75-164).
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..ops import kernels
from .params import SamplingParams

ROW_WORDS = 7        # temperature, top_p (float bits), top_k, seed lo/hi, draw lo/hi


def pack_rows(params: Sequence[SamplingParams], draws: Sequence[int], capacity: int | None = None) -> np.ndarray:
    """Per-row arguments as one int32 array ``[7, capacity]`` (row-major by field)."""
    rows = len(params)
    capacity = capacity or rows
    packed = np.zeros((ROW_WORDS, capacity), dtype=np.int32)
    temperature = np.zeros(capacity, dtype=np.float32)
    top_p = np.ones(capacity, dtype=np.float32)
    for i, (p, draw) in enumerate(zip(params, draws)):
        temperature[i] = p.temperature
        top_p[i] = p.top_p
        packed[2, i] = min(p.top_k, 2**31 - 1)
        packed[3:7, i] = np.array([p.seed & 0xFFFFFFFF, p.seed >> 32, draw & 0xFFFFFFFF, draw >> 32],
                                  dtype=np.uint32).view(np.int32)
    packed[0] = temperature.view(np.int32)
    packed[1] = top_p.view(np.int32)
    return packed


def sample_packed(logits: torch.Tensor, packed: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Sample with per-row arguments already on the device as int32 ``[7, capacity]``."""
    return kernels.sample_rows(logits, packed, out=out)


class Sampler:
    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draws: Sequence[int]) -> torch.Tensor:
        """int32 tokens on the device, one per row; ``draws[i]`` counts the tokens
        row i's request has drawn before."""
        if logits.shape[0] != len(params) or len(params) != len(draws):
            raise ValueError("params and draws must align with the rows of logits")
        packed = torch.from_numpy(pack_rows(params, draws)).to(logits.device, non_blocking=True)
        return sample_packed(logits, packed)
