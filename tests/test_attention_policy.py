"""The host-side choices of the attention launches: pieces per request, tiles of a step.  No GPU."""

from tinyvllm_b200.ops.attention import DECODE_MAX_SPLITS, decode_splits, prefill_tiles


def test_pieces_fall_with_the_rows_of_the_step():
    long = 4096
    assert [decode_splits(long, rows) for rows in (1, 2, 3, 4)] == [8, 8, 8, 8]
    assert [decode_splits(long, rows) for rows in (5, 6, 8, 10, 12, 16, 20)] == [6, 5, 4, 3, 3, 2, 2]
    assert [decode_splits(long, rows) for rows in (22, 24, 32, 36)] == [1, 1, 1, 1]
    assert [decode_splits(long, rows) for rows in (37, 40, 45)] == [3, 3, 3]          # evens out a third CTA on few SMs
    assert [decode_splits(long, rows) for rows in (46, 48)] == [1, 1]
    assert [decode_splits(long, rows) for rows in (49, 64, 256)] == [2, 2, 2]
    assert all(1 <= decode_splits(long, rows) <= DECODE_MAX_SPLITS for rows in range(0, 300))


def test_pieces_are_bounded_by_the_context_limit():
    # a piece is not worth less than 64 keys of the longest request the engine admits
    assert decode_splits(64, 1) == 1
    assert decode_splits(128, 1) == 2
    assert decode_splits(300, 1) == 5
    assert decode_splits(300, 8) == 4
    assert decode_splits(1, 1) == 1


def test_tiles_cover_every_token_once(monkeypatch):
    from tinyvllm_b200.ops import kernels

    # the tile sizes of the two kernels, without compiling them
    monkeypatch.setattr(kernels, "attention_prefill_tile_tokens", lambda: 64)
    monkeypatch.setattr(kernels, "attention_prefill_tc_tile_tokens", lambda: 128)
    counts, starts = [300, 1, 70, 3, 64, 777], [0, 40, 0, 512, 0, 223]
    big, rest, runs = prefill_tiles(counts, starts, tensor_memory=True, singles_apart=True)
    covered = []
    for rows, firsts, sizes in (big, rest):
        assert len(rows) == len(firsts) == len(sizes)
        for first, size in zip(firsts, sizes):
            covered.extend(range(first, first + size))
    for first, count in runs:
        covered.extend(range(first, first + count))
    assert sorted(covered) == list(range(sum(counts)))
    assert all(size <= 128 for size in big[2]) and all(size <= 64 for size in rest[2])
    # the tiles of the tensor-memory kernel come with the longest context first
    ends = []
    offsets = [sum(counts[:i]) for i in range(len(counts))]
    for row, first, size in zip(*big):
        ends.append(starts[row] + (first - offsets[row]) + size)
    assert ends == sorted(ends, reverse=True)
