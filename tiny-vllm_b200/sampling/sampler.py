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
    packed[1] = np.ones(capacity, dtype=np.float32).view(np.int32)
    if rows == 0:
        return packed
    packed[0, :rows] = np.array([p.temperature for p in params], dtype=np.float32).view(np.int32)
    packed[1, :rows] = np.array([p.top_p for p in params], dtype=np.float32).view(np.int32)
    packed[2, :rows] = np.minimum(np.array([p.top_k for p in params], dtype=np.int64), 2**31 - 1)
    seeds = np.array([p.seed for p in params], dtype=np.uint64)
    counts = np.array(list(draws), dtype=np.uint64)
    low = np.uint64(0xFFFFFFFF)
    packed[3, :rows] = (seeds & low).astype(np.uint32).view(np.int32)
    packed[4, :rows] = (seeds >> np.uint64(32)).astype(np.uint32).view(np.int32)
    packed[5, :rows] = (counts & low).astype(np.uint32).view(np.int32)
    packed[6, :rows] = (counts >> np.uint64(32)).astype(np.uint32).view(np.int32)
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
