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
WEIGHT_MODES = ("checkpoint", "random")

# field -> smallest value it may take; all of these are plain ints (bool is not an int here)
_INT_FIELDS = {
    "max_model_len": 1, "max_num_seqs": 1, "max_num_batched_tokens": 1, "prefill_chunk_size": 1,
    "kv_block_size": 1, "kv_cache_memory_bytes": 1, "decode_run_steps": 1,
    "prefill_reserve_tokens": 0, "prefill_reserve_requests": 0, "seed": 0,
}


def _int_at_least(name: str, value, least: int) -> None:
    if type(value) is not int or value < least:
        kind = "a positive integer" if least == 1 else f"an integer of at least {least}"
        raise ValueError(f"{name} must be {kind}, got {value!r}")


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
        folder = Path(self.model).expanduser().resolve()
        if not folder.is_dir():
            raise ValueError(f"the model folder {folder} does not exist")
        object.__setattr__(self, "model", folder)
        self._check_choices()
        for name, least in _INT_FIELDS.items():
            _int_at_least(name, getattr(self, name), least)
        sizes = tuple(self.graph_batch_sizes)
        for size in sizes:
            _int_at_least("graph_batch_sizes entry", size, 1)
        object.__setattr__(self, "graph_batch_sizes", tuple(sorted(set(sizes))))
        self._check_memory_share()
        self._check_step_budget()

    def _check_choices(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype is one of {', '.join(DTYPES)}, not {self.dtype!r}")
        if self.weights not in WEIGHT_MODES:
            raise ValueError(f"weights is one of {', '.join(WEIGHT_MODES)}, not {self.weights!r}")
        if type(self.enforce_eager) is not bool:
            raise TypeError("enforce_eager must be bool")

    def _check_memory_share(self) -> None:
        share = self.gpu_memory_utilization
        if isinstance(share, bool) or not isinstance(share, (int, float)):
            raise TypeError("gpu_memory_utilization must be a number")
        if not (math.isfinite(share) and 0.0 < share < 1.0):
            raise ValueError(f"gpu_memory_utilization must lie between 0 and 1 (both excluded), got {share}")

    def _check_step_budget(self) -> None:
        """A step holds up to max_num_batched_tokens tokens of up to max_num_seqs requests.  While
        requests decode, part of that room may be kept for prompt portions: so many tokens for so
        many requests.  The part kept must leave room to decode, and a portion must fit a step."""
        kept_tokens, kept_requests = self.prefill_reserve_tokens, self.prefill_reserve_requests
        if bool(kept_tokens) != bool(kept_requests):
            raise ValueError("prefill_reserve_tokens and prefill_reserve_requests are both zero or both "
                             f"positive (got {kept_tokens} and {kept_requests})")
        if kept_tokens < kept_requests:
            raise ValueError(f"{kept_requests} requests cannot share {kept_tokens} kept tokens: "
                             "each needs at least one")
        if kept_tokens >= self.max_num_batched_tokens or kept_requests >= self.max_num_seqs:
            raise ValueError(
                f"keeping {kept_tokens} tokens and {kept_requests} requests of a step for prefills leaves "
                f"nothing of its {self.max_num_batched_tokens} tokens or {self.max_num_seqs} requests to decode with")
        if self.prefill_chunk_size > self.max_num_batched_tokens:
            raise ValueError(f"prefill_chunk_size={self.prefill_chunk_size}: a prompt portion (chunk) does not "
                             f"fit into a step of {self.max_num_batched_tokens} tokens")
