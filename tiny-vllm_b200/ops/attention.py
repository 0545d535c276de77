"""Attention over the paged cache: which kernel runs a step.

Every kernel computes the same thing: the query at position p attends the keys
of its request from max(0, p - window + 1) to p through the block table.  The
row kernel (one warp per token and head) takes every size and dtype; tiled
kernels take over for the shapes they are written for.
"""

from __future__ import annotations

from . import kernels

# rows (tokens * heads) up to which the chunks of a row are spread over the grid
SPLIT_MAX_TOKENS = 256


def choose_split(tokens: int, max_position: int) -> int:
    """Number of key chunks to spread over the grid, or 0 to walk them per row.

    Both ways give a row the same arithmetic, so the choice only trades
    parallelism against scratch memory: few tokens with long contexts split."""
    chunk = kernels.attention_chunk_keys()
    if tokens <= SPLIT_MAX_TOKENS and max_position + 1 > chunk:
        return -(-(max_position + 1) // chunk)
    return 0


def paged_attention(ctx, mixer, qkv, keys, values, group: int):
    """Attention output [tokens, heads * head_dim] for the step ``ctx``; the
    query heads are read in place from the packed projection ``qkv``."""
    scratch = None
    if ctx.split_chunks > 0:
        scratch = ctx.workspace(kernels.attention_rows_scratch_floats(
            ctx.num_tokens, mixer.num_heads, mixer.head_dim, ctx.split_chunks))
    return kernels.attention_rows(
        qkv, qkv.shape[1], keys, values, ctx.block_tables[group], ctx.token_row, ctx.positions,
        num_q=mixer.num_heads, num_kv=mixer.num_kv_heads, head_dim=mixer.head_dim,
        window=mixer.window, scale=mixer.scale, scratch=scratch, max_chunks=ctx.split_chunks)
