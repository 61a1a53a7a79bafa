"""Bucket cutting of the host-streamed step (host logic, no GPU): every block of every tensor lands in
exactly one bucket, in order, and a tensor appears at most once per bucket (the step's block ranges are
keyed by tensor)."""
import math

import pytest

from gefen_b200.host_stream import cut_buckets

SHAPES = [(64, 512), (2048,), (96, 768), (600, 2048), (33, 24), (128, 1024), (7,), (256, 256)]
PERIODS = [512, 1, 768, 2048, 24, 1024, 1, 256]


@pytest.mark.parametrize("n_buckets", [1, 2, 3, 4, 8, 16, 64, 1000])
def test_cut_buckets_cover_every_block_once(n_buckets):
    numels = [math.prod(s) for s in SHAPES]
    buckets = cut_buckets(numels, [2] * len(numels), PERIODS, n_buckets)
    assert 1 <= len(buckets) <= n_buckets
    runs = {}
    for bucket in buckets:
        seen = set()
        for i, b0, b1, whole in bucket:
            assert i not in seen
            seen.add(i)
            assert b0 < b1
            runs.setdefault(i, []).append((b0, b1, whole))
    for i, (numel, period) in enumerate(zip(numels, PERIODS)):
        blocks = numel // period if period > 1 else 1
        r = runs[i]
        assert r[0][0] == 0 and r[-1][1] == blocks
        for a, b in zip(r, r[1:]):
            assert a[1] == b[0]
        assert all(whole == (len(r) == 1) for _, _, whole in r)
        if period == 1:
            assert len(r) == 1


def test_cut_buckets_balances_bytes():
    numels = [math.prod(s) for s in SHAPES]
    buckets = cut_buckets(numels, [2] * len(numels), PERIODS, 8)
    sizes = [sum((b1 - b0) * (PERIODS[i] if PERIODS[i] > 1 else numels[i]) * 2 for i, b0, b1, _ in b) for b in buckets]
    assert len(buckets) == 8
    assert max(sizes) <= 1.1 * (sum(sizes) / 8)


@pytest.mark.parametrize("world,n_buckets", [(2, 8), (3, 4), (2, 1)])
def test_push_plan_covers_every_owned_piece_once(world, n_buckets):
    """Buckets of the pushed reduce-scatter of ZeRO-1 (host logic): for every rank the bucket ranges lie inside
    its segment, do not overlap, ascend, and together contain every element of every piece it owns; the block
    runs of the cuts cover every block exactly once."""
    from gefen_b200.zero1 import FlatLayout, push_plan

    shapes = [(96, 512), (64, 2048), (2048,), (40, 768), (33, 24), (7,), (128, 1024), (300, 2048)]
    periods = {0: 512, 1: 2048, 2: 1, 3: 768, 4: 24, 5: 1, 6: 1024, 7: 2048}
    layout = FlatLayout(shapes, world)
    for q in range(world):
        pieces, used, cuts, ranges = push_plan(layout, periods, q, n_buckets, 2)
        assert len(ranges) == n_buckets
        filled = [r for r in ranges if r[1] > r[0]]
        assert all(0 <= lo < hi <= layout.segment for lo, hi in filled)
        assert all(a[1] <= b[0] for a, b in zip(filled, filled[1:]))
        for pc in pieces:   # every element of the piece lies in some bucket's range
            lo, hi = pc.offset - q * layout.segment, pc.offset + pc.numel - q * layout.segment
            covered = sorted((max(lo, a), min(hi, b)) for a, b in filled if a < hi and b > lo)
            assert covered and covered[0][0] == lo and covered[-1][1] == hi
            assert all(x[1] == y[0] for x, y in zip(covered, covered[1:]))
        runs = {}
        for bucket in cuts:
            for i, b0, b1, whole in bucket:
                runs.setdefault(i, []).append((b0, b1))
        for i, pc in enumerate(pieces):
            blocks = pc.numel // used[i] if used[i] > 1 else 1
            r = runs[i]
            assert r[0][0] == 0 and r[-1][1] == blocks and all(a[1] == b[0] for a, b in zip(r, r[1:]))


def test_cut_buckets_follows_weights():
    numels = [math.prod(s) for s in SHAPES]
    weights = [0.125, 0.25, 0.5, 1, 1, 1, 1, 1, 1, 1, 0.5, 0.25, 0.125]
    buckets = cut_buckets(numels, [2] * len(numels), PERIODS, len(weights), weights)
    sizes = [sum((b1 - b0) * (PERIODS[i] if PERIODS[i] > 1 else numels[i]) * 2 for i, b0, b1, _ in b) for b in buckets]
    assert len(buckets) == len(weights)
    total = sum(sizes)
    for size, w in zip(sizes[:-1], weights[:-1]):   # a bucket closes with the block that fills it: up to one block over
        assert 0 <= size - total * w / sum(weights) <= 4096 + 8
    assert 0 < sizes[-1] <= total * weights[-1] / sum(weights)   # the last one takes what is left
