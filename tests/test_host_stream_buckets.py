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
