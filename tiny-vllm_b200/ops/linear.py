"""x . W^T for the parts, by storage dtype.

float32: the package's own float32-core kernel (true 32-bit, ascending k).
bfloat16: the tensor-core kernels of this package where they take the shape,
else cuBLAS through ``torch.nn.functional.linear``, which is what the
reference's engine calls for every projection (tinyvllm/layers.py:84-85).
"""

from __future__ import annotations

import torch

from . import kernels


def linear(x: torch.Tensor, weight: torch.Tensor, *, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """x [m, k] times weight [n, k] transposed; the result has ``out_dtype``
    (default: the dtype of x)."""
    if not x.is_cuda:
        raise kernels.KernelError("linear runs on CUDA tensors only; there is no CPU path")
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise kernels.KernelError("a float32 product has a float32 result")
        return kernels.gemm_nt_simt(x, weight, out=out)
    from . import gemm

    return gemm.linear_bf16(x, weight, out_dtype=out_dtype, out=out)


def linear_silu(x: torch.Tensor, gate_up_weight: torch.Tensor) -> torch.Tensor:
    """round(round(silu(x . gate^T)) * (x . up^T)) for a packed [gate | up] weight, [m, inter]."""
    if not x.is_cuda:
        raise kernels.KernelError("linear_silu runs on CUDA tensors only; there is no CPU path")
    if x.dtype == torch.float32:
        return kernels.silu_mul(kernels.gemm_nt_simt(x, gate_up_weight))
    from . import gemm

    return gemm.linear_silu_bf16(x, gate_up_weight)
