"""bfloat16 matrix products: which kernel takes which shape.

Up to 16 rows (decode) with a bfloat16 result and a weight of up to 40 MB (24 MB beyond 8 rows):
the package's weight-streaming kernel for small weights (measured against cuBLAS per shape: it
wins up to 8 rows by 20 to 50 %, is level around 16 and loses beyond, and loses on large
weights).  Up to 64 rows and a weight of 400 MB and more (the gate/up product of the largest
models): the package's stream-k tcgen05 kernel, which reads the weight faster than cuBLAS but has
a higher fixed cost per launch (figures at STREAM_MIN_WEIGHT_BYTES).  Results in float32 (the
logits: vocabulary x width) go to cuBLAS with float32 output at every row count: 53 us against
84 us (small-weight kernel) and 56 us (stream-k kernel) at 8 rows.  The packed gate/up product
with its activation at 128 rows and more (prefill): the package's tcgen05 kernel, which keeps
the accumulator in tensor memory and applies SiLU(gate) * up on the way out.  The other
products with more than 32 rows: cuBLAS through ``torch.nn.functional.linear``, the library
call the reference's engine makes for every projection (tinyvllm/layers.py:84-85).
"""

from __future__ import annotations

import os
import weakref

import torch

from . import kernels


# weight (by address) -> (that weight, the weight the model streams next in a decode step), both as
# weak references: the weight-streaming kernel asks for the next one to be brought into L2 while it
# works on its own.  Weak, so that a model that is dropped frees its memory; the first reference
# tells a weight from a later tensor that the allocator put at the same address.
_next_weight: dict[int, tuple[weakref.ref, weakref.ref]] = {}


def chain_weights(weights) -> None:
    """Declare the order in which a step streams ``weights`` (the last is followed by the first)."""
    weights = [w for w in weights if w is not None and w.is_cuda and w.dtype == torch.bfloat16]
    for key in [key for key, (current, _) in _next_weight.items() if current() is None]:
        del _next_weight[key]
    for current, following in zip(weights, weights[1:] + weights[:1]):
        _next_weight[current.data_ptr()] = (weakref.ref(current), weakref.ref(following))


def next_weight(weight: torch.Tensor) -> torch.Tensor | None:
    found = _next_weight.get(weight.data_ptr())
    if found is None or found[0]() is not weight:
        return None
    return found[1]()


# rows from which the tcgen05 kernel's tiles of 128 rows are mostly full
TC_MIN_ROWS = 128
# rows up to which the weight-streaming kernel is chosen over cuBLAS
SMALL_M_DISPATCH_ROWS = 16
# ... and the size of the weight up to which it is: the kernel is built for the latency of small
# products (many small CTAs, a cluster barrier at the end) and streams at 3 to 4 TB/s at best, while
# cuBLAS reaches 5.4 to 5.7 TB/s on weights of 100 MB and more.  Measured in CUDA graphs, weights
# rotated through more than L2 (us, this kernel / cuBLAS): 8 rows 12.6 MB 3.9 / 7.6, 33.6 MB
# 11.7 / 12.6, 50 MB 16.9 / 11.6, 84 MB 25.2 / 17.6, 201 MB 50 / 37, 524 MB 130 / 93; 16 rows
# 12.6 MB 5.3 / 7.8, 33.6 MB 16.8 / 9.3, 50 MB 22.4 / 12.8.
SMALL_M_MAX_WEIGHT_BYTES = 40 << 20
SMALL_M_MAX_WEIGHT_BYTES_OVER_8_ROWS = 24 << 20


# The stream-k tcgen05 kernel reads a large weight at 6.1 to 6.3 TB/s where cuBLAS reaches 5.5 to
# 5.8, but a launch costs about 7 us beside the stream itself (set-up, the first copies, and the
# partial sums of tiles that two CTAs share), and rows of x beyond 32 cost more than they do in
# cuBLAS.  Measured in CUDA graphs, weights rotated through more than L2 (us, this kernel / cuBLAS,
# the latter with the activation kernel behind it for gate/up): 8 rows gate/up 201 MB 41.9 / 37.1,
# 357 MB 64.2 / 63.8, 524 MB 85.6 / 93.6; 64 rows 524 MB 96.3 / 98.9; the head (311 MB, float32
# out) 56.5 / 53.7; 262 MB with k = 25,600 (every tile shared by four CTAs) 50.6 / 45.6.
STREAM_MIN_WEIGHT_BYTES = int(os.environ.get("TINYVLLM_B200_STREAM_MIN_MB", "400")) << 20
STREAM_MAX_ROWS = 64


def streamed(x: torch.Tensor, weight: torch.Tensor, mode: int) -> bool:
    """Whether the stream-k kernel takes this product."""
    return (x.shape[0] <= STREAM_MAX_ROWS and weight.numel() * weight.element_size() >= STREAM_MIN_WEIGHT_BYTES
            and kernels.gemm_stream_takes(x, weight, mode))


def small(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes this product."""
    limit = SMALL_M_MAX_WEIGHT_BYTES if x.shape[0] <= 8 else SMALL_M_MAX_WEIGHT_BYTES_OVER_8_ROWS
    return (x.shape[0] <= SMALL_M_DISPATCH_ROWS and weight.numel() * weight.element_size() <= limit
            and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0)


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, *, out_dtype: torch.dtype,
                out: torch.Tensor | None = None) -> torch.Tensor:
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise kernels.KernelError("linear_bf16 wants bfloat16 operands")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise kernels.KernelError(f"linear_bf16 cannot produce {out_dtype}")
    if out_dtype == torch.float32:
        # float32 results (logits) keep the float32 accumulator unrounded
        if streamed(x, weight, kernels.GEMM_F32) and (out is None or out.stride(1) == 1):
            return kernels.gemm_stream(x, weight, kernels.GEMM_F32, out=out)
        if x.stride(1) == 1 and weight.stride(1) == 1 and x.shape[1] % 8 == 0:
            result = torch.mm(x, weight.t(), out_dtype=torch.float32)
        elif x.shape[0] <= 256:
            return kernels.gemm_nt_simt(x, weight, out=out, out_dtype=torch.float32)
        else:
            result = torch.nn.functional.linear(x, weight).float()
        if out is not None:
            out.copy_(result)
            return out
        return result
    if small(x, weight):
        return kernels.gemm_small_m(x, weight, kernels.GEMM_BF16, out=out, prefetch=next_weight(weight))
    if streamed(x, weight, kernels.GEMM_BF16) and (out is None or out.stride(1) == 1):
        return kernels.gemm_stream(x, weight, kernels.GEMM_BF16, out=out)
    if out is not None:
        return torch.mm(x, weight.t(), out=out)
    return torch.nn.functional.linear(x, weight)


def linear_silu_bf16(x: torch.Tensor, gate_up_weight: torch.Tensor) -> torch.Tensor:
    """silu(x . gate^T) * (x . up^T) for a packed [gate | up] weight."""
    if small(x, gate_up_weight):
        return kernels.gemm_small_m(x, gate_up_weight, kernels.GEMM_SILU, prefetch=next_weight(gate_up_weight))
    if streamed(x, gate_up_weight, kernels.GEMM_SILU):
        return kernels.gemm_stream(x, gate_up_weight, kernels.GEMM_SILU)
    if x.shape[0] >= TC_MIN_ROWS and kernels.gemm_tc_takes(x, gate_up_weight, kernels.GEMM_SILU):
        return kernels.gemm_tc(x, gate_up_weight, kernels.GEMM_SILU)
    return kernels.silu_mul(torch.nn.functional.linear(x, gate_up_weight))
