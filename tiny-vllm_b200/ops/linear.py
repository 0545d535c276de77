"""x . W^T for the parts, by storage dtype.

float32: the package's own float32-core kernel (true 32-bit, ascending k).
bfloat16: the tensor-core kernels of this package where they take the shape,
else cuBLAS through ``torch.nn.functional.linear``, which is what the
reference's engine calls for every projection (tinyvllm/layers.py:84-85).
"""

from __future__ import annotations

import os

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


# Every CTA of the fused kernel reads all rows of the input to normalise them for itself; beyond
# a few rows those reads cost more (in L2 bandwidth) than the separate norm kernel they replace.
FUSED_NORM_MAX_ROWS = int(os.environ.get("TINYVLLM_B200_FUSED_NORM_ROWS", "2"))


# TINYVLLM_B200_STREAM_ADD=0: output projections never add to the stream themselves (the norm kernel
# runs between every two products), for comparison
STREAM_ADD = os.environ.get("TINYVLLM_B200_STREAM_ADD", "1") != "0"


def linear_into_stream(x: torch.Tensor, weight: torch.Tensor, stream: torch.Tensor):
    """A part's output projection, added to the residual stream where that saves a kernel.

    Returns (None, stream + linear(x, weight)) when the product's kernel does the addition on its
    way out (small bfloat16 batches): the new stream then carries ``row_squares``, the sums of
    squares of its rows tile by tile, with which :func:`linear_norm` applies the next pre-norm
    inside the next product, so that no norm kernel runs between the two (there the norm weight
    multiplies the stream before the product and the inverse RMS the sums after it: one rounding
    where the norm kernel has two).  Otherwise
    (linear(x, weight), stream), and the next norm adds the two as usual."""
    from . import gemm

    if (STREAM_ADD and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and stream is not None
            and stream.dtype == torch.bfloat16 and stream.is_contiguous() and gemm.small(x, weight)
            and stream.shape == (x.shape[0], weight.shape[0])):
        summed, squares = kernels.gemm_small_m(x, weight, kernels.GEMM_BF16, add_stream=stream,
                                               prefetch=gemm.next_weight(weight))
        summed.row_squares = squares
        return None, summed
    return linear(x, weight), stream


def linear_norm(hidden: torch.Tensor | None, residual: torch.Tensor | None, norm, weight: torch.Tensor, *,
                silu: bool = False):
    """(linear(norm(hidden + residual), weight), hidden + residual): a pre-norm and the
    projection behind it as one operation.  ``norm`` is a norm part (``weight``, ``eps``,
    ``forward``, ``add``).  Without a residual the stream is ``hidden`` itself; without
    ``hidden`` (None) the residual holds the sum already (:func:`linear_into_stream`).  ``silu``
    applies SiLU(gate) * up to a packed [gate | up] weight.  Small bfloat16 batches run as
    one kernel; everything else as the norm kernel and the product."""
    from . import gemm

    if hidden is None:
        squares = getattr(residual, "row_squares", None)
        if (squares is not None and weight.dtype == torch.bfloat16 and getattr(norm, "folds_into_product", False)
                and gemm.small(residual, weight) and residual.is_contiguous()
                and norm.weight.data_ptr() % 16 == 0):
            mode = kernels.GEMM_SILU if silu else kernels.GEMM_BF16
            out = kernels.gemm_small_m(residual, weight, mode, norm_weight=norm.weight, eps=norm.eps,
                                       row_squares=squares, prefetch=gemm.next_weight(weight))
            return out, residual
        x = norm.forward(residual)
        return (linear_silu(x, weight) if silu else linear(x, weight)), residual
    if (hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and hidden.is_contiguous()
            and getattr(norm, "folds_into_product", False) and gemm.small(hidden, weight)
            and hidden.shape[0] <= FUSED_NORM_MAX_ROWS
            and kernels.gemm_small_m_takes_norm(hidden.shape[0], hidden.shape[1])):
        mode = kernels.GEMM_SILU if silu else kernels.GEMM_BF16
        out, stream = kernels.gemm_small_m(hidden, weight, mode, norm_weight=norm.weight,
                                           residual=residual, eps=norm.eps,
                                           prefetch=gemm.next_weight(weight))
        return out, (hidden if residual is None else stream)
    if residual is None:
        x, stream = norm.forward(hidden), hidden
    else:
        x, stream = norm.add(hidden, residual)
    return (linear_silu(x, weight) if silu else linear(x, weight)), stream
