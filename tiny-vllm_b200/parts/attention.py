"""Grouped-query attention over the paged cache, with per-head q/k RMSNorm.

qkv = x . Wqkv^T packed as [q | k | v] (tinyvllm/models/qwen3.py:230-240,
:273-280); q and k are normalised per head and rotated, k and v go to their
cache pages (:284-299; tinyvllm/kernels/kv_store.cu:26-90); every query attends
the keys of its request up to its own position, at most ``window`` of them
(tinyvllm/runtime/attention.py:34-55; tinyvllm/kernels/paged_decode.cu:85-466);
then the output projection (:303).  All sizes, the scale, the eps and the window
are parameters; the position encoding is a part of its own.
"""

from __future__ import annotations

from ..ops import attention as attention_ops
from ..ops import kernels, linear, linear_into_stream, linear_norm
from .base import BuildContext, KVNeed, ParamSpec, Part
from .registry import register_part


class GQAAttention(Part):
    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, qk_norm_eps: float | None, window: int | None,
                 position=None, names: dict | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("query heads must be a multiple of key-value heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"the attention kernels take head sizes in steps of 16 up to 256, not {head_dim}")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.prefix = ctx.prefix
        n = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.position = ctx.build("position", position, ctx) if position is not None else None
        self.qkv_weight = self.o_weight = self.q_norm_weight = self.k_norm_weight = None

    # ------------------------------------------------------------ declaration
    def param_specs(self):
        q_rows, kv_rows = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = [
            ParamSpec.packed("qkv_weight", [(self.names["q"], q_rows), (self.names["k"], kv_rows),
                                            (self.names["v"], kv_rows)], self.hidden_size),
            ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, q_rows)),
        ]
        if self.qk_norm_eps is not None:
            specs += [
                ParamSpec.single("q_norm_weight", self.names["q_norm"], (self.head_dim,),
                                 role="vector", init="around_one"),
                ParamSpec.single("k_norm_weight", self.names["k_norm"], (self.head_dim,),
                                 role="vector", init="around_one"),
            ]
        return specs

    def children(self):
        return [self.position] if self.position is not None else []

    def streamed_weights(self):
        return [self.qkv_weight, self.o_weight]

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        """Whether this mixer's prefill may run on the tcgen05 tile kernel; the step cuts its
        tile lists for that kernel only if every mixer of the model says so."""
        return kernels.attention_prefill_tc_supports(self.head_dim, self.num_heads, self.num_kv_heads,
                                                     page_size)

    def scratch_floats(self, rows: int, chunks: int) -> int:
        """float32 scratch the row kernel asks for when it spreads ``chunks`` key chunks of
        ``rows`` single tokens over the grid."""
        return kernels.attention_rows_scratch_floats(rows, self.num_heads, self.head_dim, chunks)

    # ---------------------------------------------------------------- running
    def forward(self, x, ctx, run: int):
        qkv = linear(x, self.qkv_weight)
        attended = attention_ops.mixer_attention(ctx, self, qkv, run)
        return linear(attended, self.o_weight)

    def forward_normed(self, hidden, residual, norm, ctx, run: int):
        """forward(norm(hidden + residual)) and the new residual stream; the output is None when
        the output projection has added it to the stream itself."""
        qkv, residual = linear_norm(hidden, residual, norm, self.qkv_weight)
        attended = attention_ops.mixer_attention(ctx, self, qkv, run)
        return linear_into_stream(attended, self.o_weight, residual)


register_part("mixer", "gqa_attention", GQAAttention)
