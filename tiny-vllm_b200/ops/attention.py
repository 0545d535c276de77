"""Attention over the paged cache: which kernels run a mixer's step.

Every path computes the same thing: q and k are normalised per head and rotated, k and v
go to their cache pages, and the query at position p attends the keys of its request from
max(0, p - window + 1) to p through the block table.

* bfloat16, every entry one token, head size 64/128/256: one fused launch
  (``attention_decode``): norm, rotation, cache write and attention split over a cluster.
* bfloat16 prompt portions, head size 128: ``qk_norm_rope_store``, then tiles of up to 128
  tokens on the tcgen05 kernel (``attention_prefill_tc``: S, P and O in tensor memory); the
  decoded tokens of the same step and the rests of portions shorter than 32 tokens are
  attended token by token by ``attention_decode`` (their keys are in the cache by then).
* bfloat16 prompt portions, head size 64 (or pages the tcgen05 kernel does not take): tiles of
  64 tokens on the mma.sync kernel (``attention_prefill``).
* everything else (float32, other head sizes): ``qk_norm_rope_store`` then the row kernel,
  one warp per token and head.
"""

from __future__ import annotations

import torch

from . import kernels

# tokens up to which the row kernel spreads the chunks of a row over the grid
SPLIT_MAX_TOKENS = 256
DECODE_MAX_SPLITS = 8
DECODE_SPLIT_GRAIN = 64


def choose_split(tokens: int, max_position: int) -> int:
    """Number of key chunks the row kernel spreads over the grid, or 0 to walk them per row.

    Both ways give a row the same arithmetic, so the choice only trades parallelism
    against scratch memory: few tokens with long contexts split."""
    chunk = kernels.attention_chunk_keys()
    if tokens <= SPLIT_MAX_TOKENS and max_position + 1 > chunk:
        return -(-(max_position + 1) // chunk)
    return 0


def decode_splits(max_model_len: int, rows: int = 1) -> int:
    """Cluster size of the fused decode kernel: into how many pieces a request's keys are cut.
    The size of a piece follows from the request's own position inside the kernel.  Few requests
    need many pieces to fill the GPU; with many requests the pieces' fixed cost (set-up, merge)
    outweighs that, so their number falls with the rows of the step: about 32 pieces a kv head
    over all rows (32 / rows, rounded); beyond 48 rows two pieces, with which the grid runs as CTAs
    of three warps in two waves (measured at 16 q / 8 kv heads, head size 128, context 2,100, us a
    layer: 8 rows 4 pieces 18.7, 6 pieces 20.0; 12 rows 2 pieces 27.0, 3 pieces 25.7; 16 rows
    2 pieces 30.9, 4 pieces 31.9; 20 rows 1 piece 44.1, 2 pieces 40.3, 4 pieces 48.8; 24 rows
    1 piece 44.4, 2 pieces 43.3, 3 pieces 53.8; 32 rows 1 piece 53.1, 2 pieces 56.0; 48 rows
    1 piece 78.7, 2 pieces 88.7; 64 rows 2 pieces 95.9, 1 piece 104.4, 3 pieces 102.5).
    Between 37 and 45 rows one piece a request gives a few SMs a third CTA with a whole context to
    read, which the others wait for; three pieces even that out (36 rows 1 piece 59.8, 3 pieces
    64.1; 38 rows 71.7 and 65.5; 40 rows 74.0 and 68.7; 44 rows 75.7 and 73.4; 46 rows 77.6 and
    85.9).
    A request's result differs between piece counts by rounding only (the order in which partial
    sums are merged)."""
    by_length = max(1, min(DECODE_MAX_SPLITS, -(-max_model_len // DECODE_SPLIT_GRAIN)))
    rows = max(rows, 1)
    by_rows = 2 if rows > 48 else 3 if 37 <= rows <= 45 else max(1, min(DECODE_MAX_SPLITS, (64 + rows) // (2 * rows)))
    return max(1, min(by_length, by_rows))


FEW_ROWS = 3                 # rows up to which the pieces are fitted to the kernel's form for small grids
FEWEST_FITTED_SPLITS = 4


def fitted_splits(splits: int, rows: int, mixer, page_size: int, max_context: int) -> int:
    """With two or three rows the fused decode kernel's form for small grids (CTAs of eight warps,
    which keep twice the bytes in flight) still has room, but only if every cluster is on the GPU
    at once, and clusters of 8 CTAs fit 14 to 16 times: the largest number of pieces with which
    they all fit, if that leaves 4 or more (measured at 16 q / 8 kv heads, head size 128, us a
    layer at contexts of 2,100 / 8,190: 2 rows 8 pieces, which do not fit, 12.9 / 29.6, 6 pieces
    10.8 / 20.9; 3 rows 8 pieces 13.4 / 31.0, 5 pieces 11.3 / 23.7; from 4 rows on the smaller CTAs
    with more pieces are as fast)."""
    if rows > FEW_ROWS or splits <= FEWEST_FITTED_SPLITS:
        return splits
    weight = mixer.q_norm_weight
    for candidate in range(splits, FEWEST_FITTED_SPLITS - 1, -1):
        if kernels.attention_decode_fits_wide(
                rows, num_q=mixer.num_heads, num_kv=mixer.num_kv_heads, head_dim=mixer.head_dim,
                page_size=page_size, splits=candidate, max_context=max_context,
                weight_dtype=None if weight is None else weight.dtype):
            return candidate
    return splits


FAR_FROM_KEYS = 12288        # keys from which a lone request is cut over several clusters a kv head
FAR_PLANS = ((4, 4), (6, 2))  # (pieces a cluster, clusters a kv head), in the order of preference


def far_plan(rows: int, mixer, page_size: int, max_context: int):
    """(pieces a cluster, clusters a kv head) for a lone request with a long context (the step says
    so: ``StepContext.decode_far``), or None.  Clusters of 8 CTAs give one request of 8 kv heads
    64 CTAs for 148 SMs; cut 16 times, in 4 clusters of 4 CTAs per kv head whose first CTAs hand
    their pieces to the last one through global memory, it has 128 (measured at 16 q / 8 kv
    heads, us a layer: context 32,700 34.8 against 44.8; 16,000 22.1 against 25.7; 12,300 19.6
    against 21.6; 8,190 16.7 against 17.0; 2,100 10.9 against 8.9: the hand-over costs about 3 us,
    so shorter requests keep one cluster of 8)."""
    if rows != 1 or mixer.head_dim != 128:
        return None
    weight = mixer.q_norm_weight
    for pieces, groups in FAR_PLANS:
        if kernels.attention_decode_fits_wide(
                rows * groups, num_q=mixer.num_heads, num_kv=mixer.num_kv_heads, head_dim=mixer.head_dim,
                page_size=page_size, splits=pieces, max_context=max_context,
                weight_dtype=None if weight is None else weight.dtype):
            return pieces, groups
    return None


# tiles with fewer tokens than this go to the 64-row kernel: a 128-row tensor-memory tile is mostly
# empty for them
TC_MIN_TILE_TOKENS = 32


def prefill_tiles(counts, starts=None, *, tensor_memory: bool = False, singles_apart: bool = False):
    """Cut every entry of a step into tiles of consecutive tokens.

    Returns two triples of lists (row, first flat token, count) and a list of runs: tiles of up to
    128 tokens for the tcgen05 kernel, the longest context first; tiles of up to 64 tokens for the
    mma.sync kernel; and, with ``singles_apart``, (first flat token, count) of every run of
    consecutive tokens that are attended one by one: single-token entries (decoded tokens beside
    prompt portions) and, with ``tensor_memory``, the rests of entries too short for a tile.  Without
    ``tensor_memory`` nothing is in the first set; with it only the short rests of entries are in
    the second.  ``starts``: tokens each entry has in the cache before the step."""
    small = kernels.attention_prefill_tile_tokens()
    large = kernels.attention_prefill_tc_tile_tokens() if tensor_memory else 0
    starts = starts if starts is not None else [0] * len(counts)
    big, ends = ([], [], []), []
    rest = ([], [], [])
    runs: list[list[int]] = []
    cursor = 0
    for row, count in enumerate(counts):
        if singles_apart and count == 1:
            if runs and runs[-1][0] + runs[-1][1] == cursor:
                runs[-1][1] += 1
            else:
                runs.append([cursor, 1])
            cursor += 1
            continue
        done = 0
        if tensor_memory:
            while count - done >= TC_MIN_TILE_TOKENS:
                size = min(large, count - done)
                big[0].append(row), big[1].append(cursor + done), big[2].append(size)
                ends.append(starts[row] + done + size)
                done += size
            if singles_apart and done < count:
                # the short rest of an entry: token by token like decoded tokens (a 64-row tile for a
                # few tokens walks a long context alone: 75 us at 2,048 keys, whatever their number)
                if runs and runs[-1][0] + runs[-1][1] == cursor + done:
                    runs[-1][1] += count - done
                else:
                    runs.append([cursor + done, count - done])
                done = count
        for start in range(done, count, small):
            rest[0].append(row), rest[1].append(cursor + start), rest[2].append(min(small, count - start))
        cursor += count
    order = sorted(range(len(ends)), key=lambda i: -ends[i])
    big = tuple([column[i] for i in order] for column in big)
    return big, rest, tuple((first, count) for first, count in runs)


def mixer_attention(ctx, mixer, qkv: torch.Tensor, run: int) -> torch.Tensor:
    """From the packed projection ``qkv`` [tokens, (q + 2 kv) * head_dim] of a step to the
    attention output [tokens, q * head_dim]; writes the step's keys and values."""
    keys, values = ctx.storage.kv_of(run)
    group = ctx.storage.group_of(run)
    writes = ctx.writes_cache(run)
    position = mixer.position
    cos = sin = None
    if position is not None:
        if getattr(position, "pairing", None) != "half_split":
            raise kernels.KernelError(
                f"the attention kernels rotate q and k from tables with the half-split pairing; the position "
                f"part {type(position).__name__} declares pairing {getattr(position, 'pairing', None)!r} (a part "
                "with another pairing needs a kernel of its own, or a mixer that applies it before attention)")
        cos, sin = position.cos, position.sin
    heads = dict(num_q=mixer.num_heads, num_kv=mixer.num_kv_heads, head_dim=mixer.head_dim)
    tiled = qkv.dtype == torch.bfloat16
    if (tiled and ctx.decode_only and writes and ctx.decode_splits > 0
            and kernels.attention_decode_supports(mixer.head_dim, mixer.num_heads, mixer.num_kv_heads,
                                                  ctx.decode_splits)):
        far = None
        if ctx.decode_far and ctx.decode_splits > 1:
            far = far_plan(qkv.shape[0], mixer, keys.shape[2], ctx.max_context)
        if far is not None:
            splits, far_groups = far
            far_from = 1                    # the step is one of a long request: always
        else:
            splits = fitted_splits(ctx.decode_splits, qkv.shape[0], mixer, keys.shape[2], ctx.max_context)
            far_groups, far_from = 1, 0
        return kernels.attention_decode(
            qkv, **heads, positions=ctx.positions, token_row=ctx.token_row, slots=ctx.slots[group],
            q_weight=mixer.q_norm_weight, k_weight=mixer.k_norm_weight, eps=mixer.qk_norm_eps or 0.0,
            cos=cos, sin=sin, key_cache=keys, value_cache=values, block_tables=ctx.block_tables[group],
            window=mixer.window, scale=mixer.scale, splits=splits, max_context=ctx.max_context,
            far_groups=far_groups, far_from=far_from)
    kernels.qk_norm_rope_store(
        qkv, **heads, positions=ctx.positions, q_weight=mixer.q_norm_weight,
        k_weight=mixer.k_norm_weight, eps=mixer.qk_norm_eps or 0.0, cos=cos, sin=sin,
        slots=ctx.slots[group] if writes else None, key_cache=keys, value_cache=values)
    if (tiled and ctx.tile_row is not None
            and kernels.attention_prefill_supports(mixer.head_dim, mixer.num_heads, mixer.num_kv_heads)):
        out = torch.empty((qkv.shape[0], mixer.num_heads * mixer.head_dim), dtype=qkv.dtype, device=qkv.device)
        if ctx.tile_tc_row is not None and ctx.tile_tc_row.shape[0] > 0:
            # the step's tile lists were cut for the tcgen05 kernel: every mixer of the model takes it
            kernels.attention_prefill_tc(
                qkv, qkv.shape[1], keys, values, ctx.block_tables[group], ctx.positions, ctx.tile_tc_row,
                ctx.tile_tc_first, ctx.tile_tc_count, **heads, window=mixer.window, scale=mixer.scale, out=out)
        if ctx.tile_row.shape[0] > 0:
            kernels.attention_prefill(
                qkv, qkv.shape[1], keys, values, ctx.block_tables[group], ctx.positions, ctx.tile_row,
                ctx.tile_first, ctx.tile_count, **heads, window=mixer.window, scale=mixer.scale, out=out)
        for first, count in ctx.single_runs:
            # Decoded tokens beside the portions.  Their q is normalised and rotated and their k, v are
            # in the cache already, so the fused decode kernel runs without its norm, rotation and
            # cache write: context split over a cluster, keys streamed once per group of q heads.
            part = slice(first, first + count)
            splits = fitted_splits(decode_splits(ctx.max_context, count), count, mixer, keys.shape[2], ctx.max_context)
            if kernels.attention_decode_supports(mixer.head_dim, mixer.num_heads, mixer.num_kv_heads, splits):
                kernels.attention_decode(
                    qkv[part], **heads, positions=ctx.positions[part], token_row=ctx.token_row[part],
                    slots=None, q_weight=None, k_weight=None, eps=0.0, cos=None, sin=None, key_cache=keys,
                    value_cache=values, block_tables=ctx.block_tables[group], window=mixer.window,
                    scale=mixer.scale, splits=splits, max_context=ctx.max_context, out=out[part],
                    new_in_cache=True,
                    library_of=None if mixer.q_norm_weight is None else mixer.q_norm_weight.dtype)
                continue
            # chunks for the longest context a request may reach, not for this step's: the count is
            # then the same for every step with these entry sizes, which a recorded step relies on
            # (the merge walks only the chunks a row's own position reaches)
            chunks = choose_split(count, max(ctx.max_context - 1, ctx.max_position))
            scratch = None
            if chunks > 0:
                scratch = ctx.workspace(kernels.attention_rows_scratch_floats(
                    count, mixer.num_heads, mixer.head_dim, chunks))
            kernels.attention_rows(
                qkv[part], qkv.shape[1], keys, values, ctx.block_tables[group], ctx.token_row[part],
                ctx.positions[part], **heads, window=mixer.window, scale=mixer.scale, out=out[part],
                scratch=scratch, max_chunks=chunks)
        return out
    scratch = None
    if ctx.split_chunks > 0:
        scratch = ctx.workspace(kernels.attention_rows_scratch_floats(
            ctx.num_tokens, mixer.num_heads, mixer.head_dim, ctx.split_chunks))
    return kernels.attention_rows(
        qkv, qkv.shape[1], keys, values, ctx.block_tables[group], ctx.token_row, ctx.positions,
        **heads, window=mixer.window, scale=mixer.scale, scratch=scratch, max_chunks=ctx.split_chunks)
