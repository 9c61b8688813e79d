"""The tile list of the grouped fp8 GEMM (csrc/grouped_gemm_fp8.cu) restated on the CPU: a prefix sum of
ceil(rows_e / 128) * (N / BN) over the experts and a binary search for "the last expert whose prefix is <= q".
Checked for ragged and empty experts: every output tile of every non-empty expert is visited exactly once, row
tiles start inside their expert, and the CTAs' shares (tiles b, b + grid, ...) differ by at most one tile."""

import random

import pytest

BM = 128


def tile_prefix(offsets, T, tiles_n):
    acc, prefix = 0, []
    for e in range(len(offsets) - 1):
        prefix.append(acc)
        rows = max(0, min(offsets[e + 1], T) - max(offsets[e], 0))
        acc += -(-rows // BM) * tiles_n
    return prefix + [acc]


def locate(q, prefix, offsets, T):
    lo, hi = 0, len(prefix) - 2
    while lo < hi:
        mid = (lo + hi + 1) >> 1
        if prefix[mid] <= q:
            lo = mid
        else:
            hi = mid - 1
    e = lo
    first, row_end = max(offsets[e], 0), min(offsets[e + 1], T)
    mt = -(-(row_end - first) // BM)
    local = q - prefix[e]
    return e, first + (local % mt) * BM, row_end, local // mt


@pytest.mark.parametrize("seed", range(20))
def test_every_tile_is_visited_once(seed):
    rng = random.Random(seed)
    E, tiles_n = rng.randrange(1, 40), rng.choice((1, 2, 7, 16))
    sizes = [rng.choice((0, 0, 1, 5, 127, 128, 129, 300, 1000)) for _ in range(E)]
    offsets = [0]
    for s in sizes:
        offsets.append(offsets[-1] + s)
    T = offsets[-1]
    prefix = tile_prefix(offsets, T, tiles_n)
    seen = set()
    for q in range(prefix[-1]):
        e, a_row, row_end, tile_n = locate(q, prefix, offsets, T)
        assert sizes[e] > 0 and offsets[e] <= a_row < row_end == offsets[e + 1] and 0 <= tile_n < tiles_n
        assert (a_row - offsets[e]) % BM == 0
        seen.add((e, a_row, tile_n))
    want = {(e, offsets[e] + BM * i, n) for e in range(E) for i in range(-(-sizes[e] // BM)) for n in range(tiles_n)}
    assert seen == want and len(seen) == prefix[-1]
    grid = 148
    shares = [len(range(b, prefix[-1], grid)) for b in range(grid)]
    assert max(shares) - min(shares) <= 1
