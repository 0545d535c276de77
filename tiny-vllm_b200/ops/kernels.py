"""Python face of the CUDA kernels: tensors in, launch on the current stream.

Every function checks shapes and dtypes, refuses what its kernel does not take
with a clear error, and raises :class:`KernelError` if the launch fails.  There
is no other implementation behind these functions: without a GPU and a built
library they raise.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 and bfloat16, not {dtype}")


def _stream() -> int:
    # the raw handle of the current stream of the current device: the same value as
    # torch.cuda.current_stream().cuda_stream without building a Stream object (this runs once a launch)
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_launches = 0

# Programmatic dependent launch for the kernels that wait for their predecessor themselves
# (griddepcontrol.wait): they may start, and fetch weights, while the kernel before them ends.
# TINYVLLM_B200_PDL=0 turns it off; a comma-separated list (gemm,norm,attention,attention_few,prefill,
# sample) keeps it for those kernels only (attention: the decode attention at every batch size;
# attention_few: with up to PDL_ATTENTION_ROWS rows and only where the launch runs as CTAs of eight
# warps that are all on the GPU at once, which find the SMs free: batch 1 to 3 gain 3 to 4 %, batch
# 4 is level and batch 6 loses 3 %, its clusters waiting for room beside the projection's CTAs; prefill: the prompt's q/k norm, rotation and cache write,
# and the tcgen05 attention).
_PDL_DEFAULT = ("gemm", "norm", "attention_few")
PDL_ATTENTION_ROWS = 3
_setting = os.environ.get("TINYVLLM_B200_PDL", "1")
PDL = frozenset() if _setting == "0" else frozenset(_PDL_DEFAULT if _setting == "1" else _setting.split(","))


def _pdl(kind: str) -> int:
    return 1 if kind in PDL else 0


def launch_count() -> int:
    """Kernels of this package launched so far by this process (graph replays not counted)."""
    return _launches


def _check(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += launches
        return
    if code < 0:
        raise KernelError(f"{what}: the kernel does not take these sizes")
    raise KernelError(f"{what}: CUDA error {code}")


def _need_cuda(*tensors: torch.Tensor) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU path")


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(library: str, name: str, argtypes, restype=c_int):
    function = _functions.get(name)
    if function is None:
        function = getattr(load_library(library), name)
        function.argtypes = argtypes
        function.restype = restype
        _functions[name] = function
    return function


def _fn_of(library: str, name: str, argtypes, restype=c_int):
    """:func:`_fn` for a function that several libraries define (one per head size and weight type)."""
    key = f"{library}:{name}"
    function = _functions.get(key)
    if function is None:
        function = getattr(load_library(library), name)
        function.argtypes = argtypes
        function.restype = restype
        _functions[key] = function
    return function


DECODE_HEAD_DIMS = (64, 128, 256)
BF16_OR_F32 = {F32: torch.float32, BF16: torch.bfloat16}


def _decode_library(head_dim: int, weight_tag: int) -> str:
    """The fused decode attention is compiled per head size and type of norm weights."""
    if head_dim not in DECODE_HEAD_DIMS:
        raise KernelError(f"attention_decode takes head sizes {DECODE_HEAD_DIMS}, not {head_dim}")
    return f"attention_decode_{head_dim}_{'f32' if weight_tag == F32 else 'bf16'}"


# ------------------------------------------------------------------ embedding
def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]]; ids int32."""
    _need_cuda(table, ids)
    if ids.dtype != torch.int32 or ids.dim() != 1 or table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embed_rows wants a contiguous [vocab, width] table and int32 ids [tokens]")
    rows, (vocab, width) = ids.shape[0], table.shape
    if out is None:
        out = torch.empty((rows, width), dtype=table.dtype, device=table.device)
    fn = _fn("pointwise", "tvb_embed_rows",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(table.data_ptr(), ids.data_ptr(), out.data_ptr(), rows, width, vocab,
              dtype_tag(table.dtype), _stream()), "embed_rows")
    return out


# -------------------------------------------------------------------- RMSNorm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, *, residual: torch.Tensor | None = None,
             rows: torch.Tensor | None = None, out: torch.Tensor | None = None,
             residual_out: torch.Tensor | None = None, want_residual: bool = True):
    """RMSNorm over the last dimension of x [tokens, width].

    With ``residual`` the rounded sum x + residual is normalised and returned as
    the second result (the new residual stream).  With ``rows`` (int32) only
    those rows are produced, in that order, and no residual is returned.
    """
    _need_cuda(x, weight, residual, rows)
    if x.dim() != 2 or not x.is_contiguous() or weight.shape != (x.shape[1],):
        raise KernelError("rms_norm wants contiguous x [tokens, width] and weight [width]")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype
                                 or not residual.is_contiguous()):
        raise KernelError("rms_norm: residual must match x")
    width = x.shape[1]
    if width * 4 > 200 * 1024:
        raise KernelError(f"rms_norm: width {width} is larger than a row buffer of shared memory holds")
    count = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("rms_norm: rows must be int32")
    if out is None:
        out = torch.empty((count, width), dtype=x.dtype, device=x.device)
    if residual is not None and rows is None and want_residual and residual_out is None:
        residual_out = torch.empty_like(x)
    if rows is not None or residual is None:
        residual_out = None
    if x.dtype == torch.bfloat16 and width % 8 == 0 and width <= 8192:     # 16-byte accesses
        fn = _fn("pointwise_bf16", "tvb_rms_norm_bf16",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                  c_int, c_int, c_void_p])
        _check(fn(x.data_ptr(), _ptr(residual), weight.data_ptr(), out.data_ptr(), _ptr(residual_out),
                  _ptr(rows), count, width, eps, dtype_tag(weight.dtype), _pdl("norm"), _stream()),
               "rms_norm")
        if residual is not None and rows is None:
            return out, residual_out
        return out
    fn = _fn("pointwise", "tvb_rms_norm",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
              c_int, c_int, c_int, c_void_p])
    _check(fn(x.data_ptr(), _ptr(residual), weight.data_ptr(), out.data_ptr(), _ptr(residual_out),
              _ptr(rows), count, width, eps, dtype_tag(x.dtype), dtype_tag(weight.dtype), _pdl("norm"),
              _stream()), "rms_norm")
    if residual is not None and rows is None:
        return out, residual_out
    return out


# ------------------------------------------------------------- SiLU(gate) * up
def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """round(round(silu(gate)) * up) of packed rows [tokens, 2 * inter]."""
    _need_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("silu_mul wants contiguous [tokens, 2 * inter]")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    if gate_up.dtype == torch.bfloat16 and inter % 8 == 0:
        fn = _fn("pointwise_bf16", "tvb_silu_mul_bf16", [c_void_p, c_void_p, c_int, c_int, c_void_p])
        _check(fn(gate_up.data_ptr(), out.data_ptr(), rows, inter, _stream()), "silu_mul")
        return out
    fn = _fn("pointwise", "tvb_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(gate_up.data_ptr(), out.data_ptr(), rows, inter, dtype_tag(gate_up.dtype), _stream()),
           "silu_mul")
    return out


# -------------------------------------------------------------- rotary tables
def rope_tables(inv_freq: torch.Tensor, positions: int) -> tuple[torch.Tensor, torch.Tensor]:
    """float32 cos and sin of position * inv_freq[j], [positions, half]."""
    _need_cuda(inv_freq)
    if inv_freq.dtype != torch.float32 or inv_freq.dim() != 1:
        raise KernelError("rope_tables wants float32 inv_freq [half]")
    half = inv_freq.shape[0]
    cos = torch.empty((positions, half), dtype=torch.float32, device=inv_freq.device)
    sin = torch.empty_like(cos)
    fn = _fn("pointwise", "tvb_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions, half, _stream()),
           "rope_tables")
    return cos, sin


# ------------------------------------ q/k norm + rotation + cache write, fused
def qk_norm_rope_store(qkv: torch.Tensor, *, num_q: int, num_kv: int, head_dim: int,
                       positions: torch.Tensor, q_weight: torch.Tensor | None,
                       k_weight: torch.Tensor | None, eps: float,
                       cos: torch.Tensor | None, sin: torch.Tensor | None,
                       slots: torch.Tensor | None, key_cache: torch.Tensor | None,
                       value_cache: torch.Tensor | None) -> None:
    """In place on the packed projection [tokens, (num_q + 2 num_kv) * head_dim]: q heads are
    normalised and rotated where they stand; k heads are normalised, rotated and written to
    ``key_cache`` at ``slots`` (page * page_size + offset); v heads are copied to
    ``value_cache``.  Caches are [pages, num_kv, page_size, head_dim]; without ``slots``
    nothing is written."""
    _need_cuda(qkv, positions, q_weight, k_weight, cos, sin, slots, key_cache, value_cache)
    tokens = qkv.shape[0]
    if qkv.dim() != 2 or not qkv.is_contiguous() or qkv.shape[1] != (num_q + 2 * num_kv) * head_dim:
        raise KernelError("qk_norm_rope_store: qkv must be contiguous [tokens, (q + 2 kv) * head_dim]")
    if head_dim % 2 or head_dim > 256:
        raise KernelError(f"qk_norm_rope_store takes even head sizes up to 256, not {head_dim}")
    if positions.dtype != torch.int32 or positions.shape != (tokens,):
        raise KernelError("qk_norm_rope_store: positions must be int32 [tokens]")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_norm_rope_store: q and k norm weights come together")
    weight_tag = dtype_tag(qkv.dtype)
    if q_weight is not None:
        if q_weight.shape != (head_dim,) or k_weight.shape != (head_dim,) or q_weight.dtype != k_weight.dtype:
            raise KernelError("qk_norm_rope_store: norm weights must be [head_dim] of one dtype")
        weight_tag = dtype_tag(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        if cos.dtype != torch.float32 or cos.shape != sin.shape or cos.shape[1] != head_dim // 2:
            raise KernelError("qk_norm_rope_store: tables must be float32 [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    if slots is not None:
        if (slots.dtype != torch.int32 or slots.shape != (tokens,) or key_cache is None
                or value_cache is None or key_cache.dim() != 4
                or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim)
                or key_cache.dtype != qkv.dtype or value_cache.shape != key_cache.shape
                or not key_cache.is_contiguous() or not value_cache.is_contiguous()):
            raise KernelError("qk_norm_rope_store: slots int32 [tokens]; caches contiguous "
                              "[pages, num_kv, page_size, head_dim] of the dtype of qkv")
    page_size = key_cache.shape[2] if slots is not None else 0
    if qkv.dtype == torch.bfloat16 and head_dim in (16, 32, 64, 128, 256):
        fn = _fn("pointwise_bf16", "tvb_qk_norm_rope_store_bf16",
                 [c_void_p] * 9 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p])
        _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
                  positions.data_ptr(), _ptr(slots), _ptr(key_cache), _ptr(value_cache), tokens, num_q,
                  num_kv, head_dim, page_size, table_positions, eps, weight_tag, _pdl("prefill"), _stream()),
               "qk_norm_rope_store")
        return
    fn = _fn("pointwise", "tvb_qk_norm_rope_store",
             [c_void_p] * 9 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p])
    _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
              positions.data_ptr(), _ptr(slots), _ptr(key_cache), _ptr(value_cache), tokens, num_q,
              num_kv, head_dim, page_size, table_positions, eps, dtype_tag(qkv.dtype), weight_tag,
              _stream()),
           "qk_norm_rope_store")


# ------------------------------------------------------------------ attention
_chunk_keys: int | None = None


def attention_chunk_keys() -> int:
    global _chunk_keys
    if _chunk_keys is None:
        _chunk_keys = _fn("attention_rows", "tvb_attention_chunk_keys", [])()
    return _chunk_keys


def attention_rows_scratch_floats(tokens: int, num_q: int, head_dim: int, max_chunks: int) -> int:
    return tokens * num_q * max_chunks * (head_dim + 2)


def attention_rows(q: torch.Tensor, q_token_stride: int, key_cache: torch.Tensor,
                   value_cache: torch.Tensor, block_tables: torch.Tensor, token_row: torch.Tensor,
                   positions: torch.Tensor, *, num_q: int, num_kv: int, head_dim: int,
                   window: int | None, scale: float, out: torch.Tensor | None = None,
                   scratch: torch.Tensor | None = None, max_chunks: int = 0) -> torch.Tensor:
    """Paged causal attention, one warp per (token, head).

    ``q`` holds the query heads of token t at ``t * q_token_stride`` elements
    (the packed projection serves as it is).  ``max_chunks > 0`` spreads the
    chunks of every row over the grid and needs ``scratch`` (float32, at least
    :func:`attention_rows_scratch_floats` long); 0 walks them in one warp."""
    _need_cuda(q, key_cache, value_cache, block_tables, token_row, positions, scratch)
    tokens = positions.shape[0]
    if head_dim > 256 or num_q % num_kv:
        raise KernelError(f"attention_rows takes head sizes up to 256 and whole groups "
                          f"(head_dim {head_dim}, {num_q} / {num_kv} heads)")
    if key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            value_cache.shape != key_cache.shape or key_cache.dtype != q.dtype or \
            not key_cache.is_contiguous() or not value_cache.is_contiguous():
        raise KernelError("attention_rows: caches must be contiguous [pages, num_kv, page_size, head_dim]")
    for name, t in (("block_tables", block_tables), ("token_row", token_row), ("positions", positions)):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention_rows: {name} must be contiguous int32")
    if block_tables.dim() != 2 or token_row.shape != (tokens,):
        raise KernelError("attention_rows: block_tables [requests, blocks], token_row [tokens]")
    if out is None:
        out = torch.empty((tokens, num_q * head_dim), dtype=q.dtype, device=q.device)
    if max_chunks > 0:
        need = attention_rows_scratch_floats(tokens, num_q, head_dim, max_chunks)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_rows: split mode needs {need} float32 of scratch")
    fn = _fn("attention_rows", "tvb_attention_rows",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(q.data_ptr(), q_token_stride, key_cache.data_ptr(), value_cache.data_ptr(),
              block_tables.data_ptr(), block_tables.shape[1], token_row.data_ptr(),
              positions.data_ptr(), out.data_ptr(), _ptr(scratch), max_chunks, tokens, num_q, num_kv,
              head_dim, key_cache.shape[2], window or 0, scale, dtype_tag(q.dtype), _stream()),
           "attention_rows", 2 if max_chunks > 0 else 1)
    return out


# ----------------------------------------------------------------------- GEMM
def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a [m, k] . w [n, k]^T on the float32 cores, ascending k."""
    _need_cuda(a, w)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or a.dtype != w.dtype:
        raise KernelError("gemm_nt_simt wants a [m, k] and w [n, k] of one dtype")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_nt_simt wants rows that are contiguous")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    fn = _fn("gemm_simt", "tvb_gemm_nt_simt",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_int, c_void_p])
    _check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, dtype_tag(a.dtype), dtype_tag(out.dtype), _stream()), "gemm_nt_simt")
    return out


# ------------------------------------------------------------------- sampling
def sample_rows(logits: torch.Tensor, packed: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of logits [rows, vocab].  ``packed`` is int32 [7, capacity >= rows],
    field-major: temperature and top_p as float32 bits, top_k, low and high word of the seed,
    low and high word of the draw counter; row r reads column r."""
    _need_cuda(logits, packed)
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample_rows wants rows that are contiguous")
    if packed.dtype != torch.int32 or packed.dim() != 2 or packed.shape[0] != 7 or \
            packed.shape[1] < rows or not packed.is_contiguous():
        raise KernelError("sample_rows: packed must be contiguous int32 [7, capacity >= rows]")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    fn = _fn("sampling", "tvb_sample_rows",
             [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), rows, vocab, packed.data_ptr(), packed.shape[1],
              out.data_ptr(), dtype_tag(logits.dtype), _pdl("sample"), _stream()), "sample_rows")
    return out


# ------------------------------------------------- tiled attention (bfloat16)
DECODE_MAX_PIECES = 8


def attention_decode_supports(head_dim: int, num_q: int, num_kv: int, splits: int) -> bool:
    """Head sizes 64, 128 and 256, whole groups of q heads, 1 to 8 pieces (answered here, so that
    asking compiles nothing; the libraries check the same)."""
    return (head_dim in DECODE_HEAD_DIMS and num_q > 0 and num_kv > 0 and num_q % num_kv == 0
            and 1 <= splits <= DECODE_MAX_PIECES)


def attention_decode(qkv: torch.Tensor, *, num_q: int, num_kv: int, head_dim: int,
                     positions: torch.Tensor, token_row: torch.Tensor, slots: torch.Tensor | None,
                     q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                     cos: torch.Tensor | None, sin: torch.Tensor | None, key_cache: torch.Tensor,
                     value_cache: torch.Tensor, block_tables: torch.Tensor, window: int | None,
                     scale: float, splits: int, max_context: int,
                     out: torch.Tensor | None = None, new_in_cache: bool = False,
                     far_groups: int = 1, far_from: int = 0,
                     library_of: torch.dtype | None = None) -> torch.Tensor:
    """One new token per request, from the raw packed projection to the attention output:
    q/k norm and rotation, cache write (unless ``slots`` is None) and attention in one launch.
    ``new_in_cache``: the new tokens' keys and values are in the cache already and q comes
    prepared (no norm weights, no tables, no slots): only the attention is left to do.
    Request i is row ``token_row[i]`` of ``block_tables`` (-1: padding) and stands at
    ``positions[i]``.  Every request's keys are cut into ``splits`` pieces, one per CTA of a cluster;
    ``max_context`` bounds ``positions + 1``."""
    _need_cuda(qkv, positions, token_row, slots, q_weight, k_weight, cos, sin, key_cache, value_cache,
               block_tables)
    requests = qkv.shape[0]
    if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous() or \
            qkv.shape[1] != (num_q + 2 * num_kv) * head_dim:
        raise KernelError("attention_decode wants contiguous bfloat16 [requests, (q + 2 kv) * head_dim]")
    if not attention_decode_supports(head_dim, num_q, num_kv, splits):
        raise KernelError(f"attention_decode does not take head_dim {head_dim}, {num_q}/{num_kv} heads, "
                          f"{splits} splits")
    if key_cache.dtype != torch.bfloat16 or key_cache.dim() != 4 or \
            (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            value_cache.shape != key_cache.shape or not key_cache.is_contiguous():
        raise KernelError("attention_decode: caches must be contiguous bfloat16 "
                          "[pages, num_kv, page_size, head_dim]")
    for t in (positions, token_row, block_tables) + ((slots,) if slots is not None else ()):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_decode: index tensors must be contiguous int32")
    if new_in_cache and not (slots is None and q_weight is None and k_weight is None and cos is None and sin is None):
        raise KernelError("attention_decode: with new_in_cache nothing is normalised, rotated or stored")
    # without norm weights either library of the head size does: ``library_of`` names the type of
    # the one the caller uses elsewhere, so that no second one is compiled
    weight_tag = BF16 if library_of is None else dtype_tag(library_of)
    if q_weight is not None:
        if k_weight is None or q_weight.dtype != k_weight.dtype or q_weight.shape != (head_dim,):
            raise KernelError("attention_decode: norm weights come together, [head_dim], one dtype")
        weight_tag = dtype_tag(q_weight.dtype)
    table_positions = cos.shape[0] if cos is not None else 0
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2):
        raise KernelError("attention_decode: tables must be float32 [positions, head_dim / 2]")
    if out is None:
        out = torch.empty((requests, num_q * head_dim), dtype=qkv.dtype, device=qkv.device)
    pdl = _pdl("attention")
    if not pdl and _pdl("attention_few") and requests <= PDL_ATTENTION_ROWS:
        # only where the launch runs as CTAs of eight warps, all on the GPU at once
        pdl = int(attention_decode_fits_wide(
            requests * far_groups, num_q=num_q, num_kv=num_kv, head_dim=head_dim, page_size=key_cache.shape[2],
            splits=splits, max_context=max_context, weight_dtype=BF16_OR_F32[weight_tag]))
    if far_groups > 1:
        # a request of far_from keys or more is cut over far_groups clusters per kv head, which
        # leave their pieces in global memory (head size 128; all clusters on the GPU at once)
        pieces, arrived = _far_scratch_of(qkv.device, requests, num_q, num_kv, head_dim, far_groups, weight_tag)
        fn = _fn_of(_decode_library(head_dim, weight_tag), "tvb_attention_decode_far",
                 [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                  c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
        _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), eps, _ptr(cos), _ptr(sin), table_positions,
                  positions.data_ptr(), token_row.data_ptr(), _ptr(slots), key_cache.data_ptr(),
                  value_cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
                  key_cache.shape[2], out.data_ptr(), requests, num_q, num_kv, head_dim, window or 0, scale,
                  splits, 2 if new_in_cache else (1 if slots is not None else 0), max_context, weight_tag,
                  pdl, far_groups, max(1, far_from), pieces.data_ptr(), arrived.data_ptr(),
                  _stream()),
               "attention_decode (far)")
        return out
    fn = _fn_of(_decode_library(head_dim, weight_tag), "tvb_attention_decode",
             [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
              c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), eps, _ptr(cos), _ptr(sin), table_positions,
              positions.data_ptr(), token_row.data_ptr(), _ptr(slots), key_cache.data_ptr(),
              value_cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
              key_cache.shape[2], out.data_ptr(), requests, num_q, num_kv, head_dim, window or 0, scale,
              splits, 2 if new_in_cache else (1 if slots is not None else 0), max_context, weight_tag,
              pdl,
              _stream()),
           "attention_decode")
    return out


_fits_wide: dict[tuple, bool] = {}
_far_scratch: dict[int, list] = {}


def _far_scratch_of(device: torch.device, requests: int, num_q: int, num_kv: int, head_dim: int,
                    groups: int, weight_tag: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Pieces and counters of the decode attention that cuts a request over several clusters, per
    device; they grow with the largest launch and the earlier ones are kept, since CUDA graphs keep
    their addresses.  Launches that use them must follow one another (those of one stream do)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    floats = _fn_of(_decode_library(head_dim, weight_tag), "tvb_attention_decode_far_floats",
                    [c_int, c_int, c_int, c_int, c_int], c_longlong)(requests, num_q, num_kv, head_dim, groups)
    if floats <= 0:
        raise KernelError("attention_decode (far): the kernel does not take these heads")
    held = _far_scratch.setdefault(index, [])
    if not held or held[-1][0].numel() < floats or held[-1][1].numel() < requests * num_q:
        held.append((torch.empty(floats, dtype=torch.float32, device=device),
                     torch.zeros(max(requests * num_q, 1024), dtype=torch.int32, device=device)))
    return held[-1]


def attention_decode_fits_wide(rows: int, *, num_q: int, num_kv: int, head_dim: int, page_size: int,
                               splits: int, max_context: int, weight_dtype: torch.dtype | None = None) -> bool:
    """Whether ``rows`` rows cut into ``splits`` pieces run in the fused decode kernel's form for
    small grids (CTAs of eight warps, one an SM) with all their clusters on the GPU at once.  Asks
    the runtime how many clusters of that shape fit; launches nothing.  Remembered per shape."""
    tag = BF16 if weight_dtype is None else dtype_tag(weight_dtype)
    key = (rows, num_q, num_kv, head_dim, page_size, splits, max_context, tag)
    known = _fits_wide.get(key)
    if known is None:
        if head_dim not in DECODE_HEAD_DIMS:
            _fits_wide[key] = False
            return False
        fn = _fn_of(_decode_library(head_dim, tag), "tvb_attention_decode_fits_wide",
                    [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int])
        known = _fits_wide[key] = bool(fn(rows, num_q, num_kv, head_dim, page_size, splits, max_context, tag))
    return known


def attention_prefill_supports(head_dim: int, num_q: int, num_kv: int) -> bool:
    fn = _fn("attention_prefill", "tvb_attention_prefill_supports", [c_int, c_int, c_int])
    return bool(fn(head_dim, num_q, num_kv))


_prefill_tile: int | None = None


def attention_prefill_tile_tokens() -> int:
    global _prefill_tile
    if _prefill_tile is None:
        _prefill_tile = _fn("attention_prefill", "tvb_attention_prefill_tile_tokens", [])()
    return _prefill_tile


def attention_prefill(q: torch.Tensor, q_token_stride: int, key_cache: torch.Tensor,
                      value_cache: torch.Tensor, block_tables: torch.Tensor, positions: torch.Tensor,
                      tile_row: torch.Tensor, tile_first: torch.Tensor, tile_count: torch.Tensor, *,
                      num_q: int, num_kv: int, head_dim: int, window: int | None, scale: float,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Paged causal attention on the tensor cores for tiles of up to 64 consecutive query
    tokens of one request (bfloat16).  Tile i holds ``tile_count[i]`` tokens from flat index
    ``tile_first[i]`` on of request row ``tile_row[i]``."""
    _need_cuda(q, key_cache, value_cache, block_tables, positions, tile_row, tile_first, tile_count)
    if q.dtype != torch.bfloat16 or key_cache.dtype != torch.bfloat16:
        raise KernelError("attention_prefill is a bfloat16 kernel")
    if not attention_prefill_supports(head_dim, num_q, num_kv):
        raise KernelError(f"attention_prefill does not take head_dim {head_dim}, {num_q}/{num_kv} heads")
    if key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            value_cache.shape != key_cache.shape or not key_cache.is_contiguous() or \
            not value_cache.is_contiguous():
        raise KernelError("attention_prefill: caches must be contiguous [pages, num_kv, page_size, head_dim]")
    for t in (block_tables, positions, tile_row, tile_first, tile_count):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_prefill: index tensors must be contiguous int32")
    tokens, tiles = positions.shape[0], tile_row.shape[0]
    if out is None:
        out = torch.empty((tokens, num_q * head_dim), dtype=q.dtype, device=q.device)
    fn = _fn("attention_prefill", "tvb_attention_prefill",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(q.data_ptr(), q_token_stride, key_cache.data_ptr(), value_cache.data_ptr(),
              block_tables.data_ptr(), block_tables.shape[1], positions.data_ptr(), tile_row.data_ptr(),
              tile_first.data_ptr(), tile_count.data_ptr(), out.data_ptr(), tiles, num_q, num_kv,
              head_dim, key_cache.shape[2], window or 0, scale, _stream()), "attention_prefill")
    return out


# ------------------------------------------- tcgen05 prefill attention (head size 128)
_prefill_tc_tile: int | None = None
_attention_tc_unchecked = False


def attention_prefill_tc_tile_tokens() -> int:
    global _prefill_tc_tile
    if _prefill_tc_tile is None:
        _prefill_tc_tile = _fn("attention_prefill_tc", "tvb_attention_prefill_tc_tile_tokens", [])()
    return _prefill_tc_tile


def attention_prefill_tc_supports(head_dim: int, num_q: int, num_kv: int, page_size: int) -> bool:
    """Head size 128, pages of 8 to 128 tokens (a power of two), whole groups of q heads."""
    return (head_dim == 128 and num_q > 0 and num_kv > 0 and num_q % num_kv == 0
            and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0)


def attention_prefill_tc(q: torch.Tensor, q_token_stride: int, key_cache: torch.Tensor,
                         value_cache: torch.Tensor, block_tables: torch.Tensor, positions: torch.Tensor,
                         tile_row: torch.Tensor, tile_first: torch.Tensor, tile_count: torch.Tensor, *,
                         num_q: int, num_kv: int, head_dim: int, window: int | None, scale: float,
                         out: torch.Tensor | None = None) -> torch.Tensor:
    """Paged causal attention on the tcgen05 tensor cores for tiles of up to 128 consecutive
    query tokens of one request (bfloat16, head size 128).  Tile i holds ``tile_count[i]`` tokens
    from flat index ``tile_first[i]`` on of request row ``tile_row[i]``; the tiles with the longest
    context come first.  The kernel reads whole pages: cache slots past a request's last key must
    hold finite values (they are multiplied by zero)."""
    _need_cuda(q, key_cache, value_cache, block_tables, positions, tile_row, tile_first, tile_count)
    if q.dtype != torch.bfloat16 or key_cache.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc is a bfloat16 kernel")
    if key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            value_cache.shape != key_cache.shape or not key_cache.is_contiguous() or \
            not value_cache.is_contiguous():
        raise KernelError("attention_prefill_tc: caches must be contiguous [pages, num_kv, page_size, head_dim]")
    if not attention_prefill_tc_supports(head_dim, num_q, num_kv, key_cache.shape[2]):
        raise KernelError(f"attention_prefill_tc does not take head_dim {head_dim}, {num_q}/{num_kv} heads, "
                          f"pages of {key_cache.shape[2]}")
    if q.dim() != 2 or q.stride(1) != 1 or q.stride(0) != q_token_stride or q_token_stride % 8 \
            or q.shape[1] < num_q * head_dim:
        raise KernelError("attention_prefill_tc: q must be [tokens, >= num_q * head_dim] with 16-byte aligned rows")
    for t in (block_tables, positions, tile_row, tile_first, tile_count):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_prefill_tc: index tensors must be contiguous int32")
    tokens, tiles = positions.shape[0], tile_row.shape[0]
    if out is None:
        out = torch.empty((tokens, num_q * head_dim), dtype=q.dtype, device=q.device)
    fn = _fn("attention_prefill_tc", "tvb_attention_prefill_tc",
             [c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p,
              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
              c_int, c_void_p])
    global _attention_tc_unchecked
    _check(fn(q.data_ptr(), q_token_stride, tokens, key_cache.data_ptr(), value_cache.data_ptr(),
              key_cache.shape[0], block_tables.data_ptr(), block_tables.shape[1], positions.data_ptr(),
              tile_row.data_ptr(), tile_first.data_ptr(), tile_count.data_ptr(), tiles, out.data_ptr(),
              num_q, num_kv, head_dim, key_cache.shape[2], window or 0, scale, _pdl("prefill"), _stream()),
           "attention_prefill_tc")
    _attention_tc_unchecked = True
    _guarded_counts[1] += 1
    return out


def attention_prefill_tc_status() -> int:
    """0, or which bounded wait of an attention_prefill_tc launch gave up since the last call.
    Synchronises the device; reading clears the record."""
    global _attention_tc_unchecked
    _attention_tc_unchecked = False
    return _fn("attention_prefill_tc", "tvb_attention_prefill_tc_status", [])()


# ------------------------------------------------ weight-streaming small-M GEMM
SMALL_M_MAX_ROWS = 32
PREFETCH_MAX_BYTES = 32 << 20
GEMM_BF16, GEMM_F32, GEMM_SILU = 0, 1, 2


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16, *,
                 out: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
                 residual: torch.Tensor | None = None, eps: float = 0.0, want_residual: bool = True,
                 row_squares: torch.Tensor | None = None, add_stream: torch.Tensor | None = None,
                 prefetch: torch.Tensor | None = None):
    """x [m <= 32, k] . w [n, k]^T, bfloat16 operands.  mode GEMM_BF16 / GEMM_F32: result
    [m, n] in that dtype; GEMM_SILU: w is [gate | up] with 2 n rows and the result is
    silu(x . gate^T) * (x . up^T), bfloat16 [m, n].

    With ``norm_weight`` the product is taken of RMSNorm(x + residual) * norm_weight instead
    of x (``residual`` may be None), and (result, rounded sum x + residual) is returned; the
    sum is None without a residual or with ``want_residual=False``.

    ``add_stream`` (GEMM_BF16; contiguous [m, n]): the result is round(round(product) + add_stream),
    the new residual stream, and (result, squares) is returned: squares [ceil(n / 16), m rounded up
    to 8] float32 holds the sum of squares of the result's rows over each tile of 16 columns.
    ``row_squares`` (with ``norm_weight``, without ``residual``): such sums for the rows of x, which
    is the stream itself; the result is (round(x * norm_weight) . w^T) * inverse RMS of the row, and
    only the result is returned.

    ``prefetch``: a tensor (the weight of the product after this one) whose first
    ``PREFETCH_MAX_BYTES`` the grid asks into L2 while it works."""
    _need_cuda(x, w, norm_weight, residual)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        raise KernelError("gemm_small_m wants bfloat16 matrices")
    m, k = x.shape
    rows = w.shape[0]
    if w.shape[1] != k or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_small_m: x [m, k] and w [n, k] with contiguous rows")
    if m < 1 or m > SMALL_M_MAX_ROWS or k % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError(f"gemm_small_m takes up to {SMALL_M_MAX_ROWS} rows (and one at least), k and row strides "
                          f"multiples of 8 (m {m}, k {k})")
    if mode == GEMM_SILU and rows % 2:
        raise KernelError("gemm_small_m: a [gate | up] weight has an even number of rows")
    n = rows // 2 if mode == GEMM_SILU else rows
    residual_out = None
    weight_tag = BF16
    padded_rows = -(-m // 8) * 8
    squares_out = None
    if add_stream is not None:
        if (mode != GEMM_BF16 or add_stream.shape != (m, n) or add_stream.dtype != torch.bfloat16
                or not add_stream.is_contiguous() or out is not None):
            raise KernelError("gemm_small_m: add_stream is a contiguous bfloat16 [m, n] and the result is new")
        squares_out = torch.empty((-(-n // 16), padded_rows), dtype=torch.float32, device=x.device)
    if row_squares is not None:
        if (norm_weight is None or residual is not None or norm_weight.shape != (k,) or not x.is_contiguous()
                or row_squares.dtype != torch.float32 or row_squares.dim() != 2
                or row_squares.shape[1] != padded_rows or not row_squares.is_contiguous()
                or norm_weight.data_ptr() % 16):
            raise KernelError("gemm_small_m: row_squares [tiles, m rounded up to 8] float32 goes with a norm "
                              "weight [k], contiguous x and no residual")
        weight_tag = dtype_tag(norm_weight.dtype)
    elif norm_weight is not None:
        if norm_weight.shape != (k,) or not x.is_contiguous() or not gemm_small_m_takes_norm(m, k):
            raise KernelError("gemm_small_m: the fused norm wants contiguous x, a weight [k] and "
                              "rows that fit into shared memory")
        if residual is not None:
            if residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_contiguous():
                raise KernelError("gemm_small_m: residual must match x")
            if want_residual:
                residual_out = torch.empty_like(x)
        weight_tag = dtype_tag(norm_weight.dtype)
    elif residual is not None:
        raise KernelError("gemm_small_m: a residual needs a norm weight")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32 if mode == GEMM_F32 else torch.bfloat16,
                          device=x.device)
    fn = _fn_of(f"gemm_small_m_nt{(m + 7) // 8}", "tvb_gemm_small_m",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_longlong, c_int, c_void_p])
    next_bytes = 0 if prefetch is None else min(prefetch.numel() * prefetch.element_size(),
                                                PREFETCH_MAX_BYTES)
    _check(fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, mode, _ptr(residual), _ptr(norm_weight), _ptr(residual_out), eps, weight_tag,
              _ptr(row_squares), 0 if row_squares is None else row_squares.shape[0], _ptr(add_stream),
              _ptr(squares_out), _ptr(prefetch), next_bytes, _pdl("gemm"), _stream()), "gemm_small_m")
    if add_stream is not None:
        return out, squares_out
    if norm_weight is not None and row_squares is None:
        return out, residual_out
    return out


def gemm_small_m_takes_norm(m: int, k: int) -> bool:
    """Whether the normalised rows [m rounded up to 8, k] fit into the kernel's shared memory."""
    return m <= SMALL_M_MAX_ROWS and k % 8 == 0 and (-(-m // 8) * 8) * (k + 32) * 2 <= 160 * 1024


# ------------------------------------------- tcgen05 matrix product (many rows)
def gemm_tc_takes(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16) -> bool:
    """Whether :func:`gemm_tc` takes this product: bfloat16, rows contiguous and 16-byte aligned,
    k and n multiples of 8."""
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2
            or x.shape[1] != w.shape[1] or x.stride(1) != 1 or w.stride(1) != 1):
        return False
    rows = w.shape[0]
    if mode == GEMM_SILU and rows % 2:
        return False
    n = rows // 2 if mode == GEMM_SILU else rows
    return (mode in (GEMM_BF16, GEMM_SILU) and x.shape[1] % 8 == 0 and n % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16, *, out: torch.Tensor | None = None,
            tile_n: int = 0) -> torch.Tensor:
    """x [m, k] . w [n, k]^T in bfloat16 on the tcgen05 tensor cores (float32 accumulation in
    tensor memory).  GEMM_BF16: [m, n]; GEMM_SILU: w is [gate | up] with 2 n rows, the result is
    silu(x . gate^T) * (x . up^T) [m, n].  ``tile_n`` 128 or 256 forces the width of a tile."""
    _need_cuda(x, w)
    if not gemm_tc_takes(x, w, mode):
        raise KernelError("gemm_tc wants bfloat16 x [m, k] and w [n, k] with contiguous, 16-byte "
                          "aligned rows, k and n multiples of 8")
    m, k = x.shape
    n = w.shape[0] // 2 if mode == GEMM_SILU else w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    elif (out.dtype != torch.bfloat16 or out.shape != (m, n) or out.stride(1) != 1 or out.stride(0) % 8
          or out.data_ptr() % 16):
        raise KernelError("gemm_tc: out must be bfloat16 [m, n] with 16-byte aligned rows")
    fn = _fn("gemm_tc", "tvb_gemm_tc",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_int, c_int, c_void_p])
    global _gemm_tc_unchecked
    _check(fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, mode, tile_n, _pdl("gemm"), _stream()), "gemm_tc")
    _gemm_tc_unchecked = True
    _guarded_counts[0] += 1
    return out


# ----------------------------- tcgen05 matrix product (few rows, a large weight)
STREAM_MAX_ROWS = 128
_stream_scratch: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
_gemm_stream_used = False


def _stream_scratch_of(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Workspace (partial sums of tiles that two CTAs share) and counters of the stream-k kernel,
    one pair per device, sized for the largest launch and never freed: CUDA graphs keep their
    addresses.  Launches that use them must follow one another (those of one stream do)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    found = _stream_scratch.get(index)
    if found is None:
        sms = torch.cuda.get_device_properties(index).multi_processor_count
        workspace = torch.empty(sms * 2 * 2 * STREAM_MAX_ROWS * 128, dtype=torch.float32, device=device)
        counters = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        found = _stream_scratch[index] = (workspace, counters)
    return found


def gemm_stream_takes(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16) -> bool:
    """Whether :func:`gemm_stream` takes this product: bfloat16, up to 128 rows of x, rows contiguous
    and 16-byte aligned, k a multiple of 8."""
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2
            or x.shape[1] != w.shape[1] or x.stride(1) != 1 or w.stride(1) != 1):
        return False
    rows = w.shape[0]
    if mode == GEMM_SILU and rows % 2:
        return False
    n = rows // 2 if mode == GEMM_SILU else rows
    return (mode in (GEMM_BF16, GEMM_F32, GEMM_SILU) and 0 < x.shape[0] <= STREAM_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and n * 4 <= (1 << 16) * 128)


def gemm_stream(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16, *, out: torch.Tensor | None = None,
                add_stream: torch.Tensor | None = None) -> torch.Tensor:
    """x [m <= 128, k] . w [n, k]^T for a large bfloat16 weight, streamed once through the tcgen05
    tensor cores with the work cut evenly over the SMs.  GEMM_BF16: bfloat16 [m, n], with
    ``add_stream`` (contiguous bfloat16 [m, n]) round(round(product) + add_stream); GEMM_F32:
    float32 [m, n]; GEMM_SILU: w is [gate | up] with 2 n rows, the result is
    silu(x . gate^T) * (x . up^T)."""
    _need_cuda(x, w, add_stream)
    if not gemm_stream_takes(x, w, mode):
        raise KernelError("gemm_stream wants bfloat16 x [m <= 128, k] and w [n, k] with contiguous, 16-byte "
                          "aligned rows and k a multiple of 8")
    m, k = x.shape
    n = w.shape[0] // 2 if mode == GEMM_SILU else w.shape[0]
    out_dtype = torch.float32 if mode == GEMM_F32 else torch.bfloat16
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    elif out.dtype != out_dtype or out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError(f"gemm_stream: out must be {out_dtype} [m, n] with contiguous rows")
    if add_stream is not None and (mode != GEMM_BF16 or add_stream.shape != (m, n)
                                   or add_stream.dtype != torch.bfloat16 or not add_stream.is_contiguous()):
        raise KernelError("gemm_stream: add_stream is a contiguous bfloat16 [m, n] of a bfloat16 result")
    workspace, counters = _stream_scratch_of(x.device)
    fn = _fn("gemm_stream", "tvb_gemm_stream",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    global _gemm_tc_unchecked, _gemm_stream_used
    _check(fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, mode, _ptr(add_stream), workspace.data_ptr(), counters.data_ptr(), _pdl("gemm"),
              _stream()), "gemm_stream")
    _gemm_tc_unchecked = _gemm_stream_used = True
    _guarded_counts[0] += 1
    return out


def gemm_stream_status() -> int:
    """0, or which bounded wait of a gemm_stream launch gave up since the last call.  Synchronises
    the device; reading clears the record."""
    return _fn("gemm_stream", "tvb_gemm_stream_status", [])()


_gemm_tc_unchecked = False


def gemm_tc_status() -> int:
    """0, or which bounded wait of a gemm_tc launch gave up since the last call (the results of
    that launch are not valid).  Synchronises the device; reading clears the record."""
    global _gemm_tc_unchecked
    _gemm_tc_unchecked = False
    return _fn("gemm_tc", "tvb_gemm_tc_status", [])()


def wait_probe(code: int = 77) -> tuple[int, int]:
    """Run the one-CTA kernel that waits on a barrier nothing arrives on: (status code the bounded
    wait recorded, millions of SM cycles it waited).  Takes about a second; the context stays
    usable.  Shows that a wait of the tcgen05 kernels that is never satisfied ends by itself."""
    waited = ctypes.c_int(0)
    fn = _fn("wait_probe", "tvb_wait_probe", [c_int, ctypes.POINTER(ctypes.c_int), c_void_p])
    status = fn(code, ctypes.byref(waited), _stream())
    if status < 0:
        raise KernelError(f"wait_probe failed ({status})")
    return status, waited.value


_guarded_counts = [0, 0]


def guarded_launch_counts() -> tuple[int, int]:
    """How often (gemm_tc or gemm_stream, attention_prefill_tc), the kernels with bounded waits, were launched
    through this module so far.  A caller that records a step into a CUDA graph compares the
    counts around one pass of the step and hands what it finds to :func:`note_guarded_launches`
    at every replay: a replay launches the kernels without passing through this module."""
    return _guarded_counts[0], _guarded_counts[1]


def note_guarded_launches(gemm: bool, attention: bool) -> None:
    """Kernels with bounded waits ran without this module seeing it (a graph replay): their status
    words are read at the next :func:`check_finished_launches`."""
    global _gemm_tc_unchecked, _attention_tc_unchecked
    _gemm_tc_unchecked = _gemm_tc_unchecked or bool(gemm)
    _attention_tc_unchecked = _attention_tc_unchecked or bool(attention)


def check_finished_launches() -> None:
    """Call after a step's results have reached the host: raises if a kernel with bounded waits
    gave up in a launch since the last call.  Costs nothing when no such kernel was launched."""
    if _gemm_tc_unchecked:
        status = gemm_tc_status()
        if status:
            raise KernelError(f"gemm_tc: a wait inside the kernel ran out (code {status}); "
                              "the results of this step are not valid")
        if _gemm_stream_used:
            status = gemm_stream_status()
            if status:
                raise KernelError(f"gemm_stream: a wait inside the kernel ran out (code {status}); "
                                  "the results of this step are not valid")
    if _attention_tc_unchecked:
        status = attention_prefill_tc_status()
        if status:
            raise KernelError(f"attention_prefill_tc: a wait inside the kernel ran out (code {status}); "
                              "the results of this step are not valid")
