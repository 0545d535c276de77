"""bfloat16 matrix products: which kernel takes which shape."""

from __future__ import annotations

import torch

from . import kernels


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, *, out_dtype: torch.dtype,
                out: torch.Tensor | None = None) -> torch.Tensor:
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise kernels.KernelError("linear_bf16 wants bfloat16 operands")
    if out_dtype == torch.bfloat16:
        if out is not None:
            return torch.mm(x, weight.t(), out=out)
        return torch.nn.functional.linear(x, weight)
    if out_dtype == torch.float32:
        # float32 results (logits) keep the float32 accumulator unrounded
        return kernels.gemm_nt_simt(x, weight, out=out, out_dtype=torch.float32)
    raise kernels.KernelError(f"linear_bf16 cannot produce {out_dtype}")
