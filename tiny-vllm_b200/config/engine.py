"""Engine limits as one frozen, validated dataclass.

Field names, defaults and checks follow tinyvllm/config.py:15-92 where the
reference has them.  Added: ``dtype="float32"`` (a true 32-bit path),
``weights``/``seed`` (random weights instead of a checkpoint), ``graph_batch_sizes``,
``decode_run_steps`` (decode steps the engine plans at once and launches ahead of the one whose
tokens it reads; 1: every step is planned, run and read by itself).
Dropped: ``attention_backend`` (there is one backend), ``enable_prefix_caching``
(not built), float16.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path
from typing import Literal

DTYPES = ("bfloat16", "float32")


def _positive_int(name: str, value) -> None:
    if type(value) is not int or value <= 0:
        raise ValueError(f"{name} must be a positive integer, got {value!r}")


def _non_negative_int(name: str, value) -> None:
    if type(value) is not int or value < 0:
        raise ValueError(f"{name} must be a non-negative integer, got {value!r}")


@dataclass(frozen=True)
class EngineConfig:
    model: Path
    dtype: Literal["bfloat16", "float32"] = "bfloat16"
    max_model_len: int = 4096
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 4096
    gpu_memory_utilization: float = 0.9
    kv_block_size: int = 16
    kv_cache_memory_bytes: int = 2 * 1024**3
    prefill_chunk_size: int = 512
    prefill_reserve_tokens: int = 128
    prefill_reserve_requests: int = 1
    enforce_eager: bool = False
    # "checkpoint": read model.safetensors; "random": config.json only, weights drawn from ``seed``
    weights: Literal["checkpoint", "random"] = "checkpoint"
    seed: int = 0
    graph_batch_sizes: tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64)
    # While nothing waits, up to this many decode steps run back to back, each fed the step before's
    # tokens on the device; the host reads their tokens together afterwards.  1: one step a time.
    decode_run_steps: int = 32
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        model = Path(self.model).expanduser().resolve()
        object.__setattr__(self, "model", model)
        if not model.is_dir():
            raise ValueError(f"model directory does not exist: {model}")
        if self.dtype not in DTYPES:
            raise ValueError(f"unsupported dtype: {self.dtype}")
        if self.weights not in ("checkpoint", "random"):
            raise ValueError(f"unsupported weights mode: {self.weights}")
        if type(self.enforce_eager) is not bool:
            raise TypeError("enforce_eager must be bool")
        for name in ("max_model_len", "max_num_seqs", "max_num_batched_tokens",
                     "prefill_chunk_size", "kv_block_size", "kv_cache_memory_bytes", "decode_run_steps"):
            _positive_int(name, getattr(self, name))
        for name in ("prefill_reserve_tokens", "prefill_reserve_requests", "seed"):
            _non_negative_int(name, getattr(self, name))
        sizes = tuple(self.graph_batch_sizes)
        for size in sizes:
            _positive_int("graph_batch_sizes entry", size)
        object.__setattr__(self, "graph_batch_sizes", tuple(sorted(set(sizes))))

        utilization = self.gpu_memory_utilization
        if type(utilization) not in (int, float):
            raise TypeError("gpu_memory_utilization must be a number")
        if not math.isfinite(utilization) or not 0.0 < utilization < 1.0:
            raise ValueError("gpu_memory_utilization must be between 0 and 1")

        tokens, requests = self.prefill_reserve_tokens, self.prefill_reserve_requests
        if (tokens == 0) != (requests == 0):
            raise ValueError("prefill reservations must both be zero or both positive")
        if not tokens < self.max_num_batched_tokens:
            raise ValueError("prefill token reservation leaves no decode capacity")
        if not requests < self.max_num_seqs:
            raise ValueError("prefill request reservation leaves no decode capacity")
        if tokens < requests:
            raise ValueError("each reserved prefill request needs one token")
        if self.prefill_chunk_size > self.max_num_batched_tokens:
            raise ValueError("prefill chunk exceeds the step token budget")
