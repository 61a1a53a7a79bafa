"""GPU parity of the calibration pipeline: exact histogram (bit-exact integers), period scores and
decisions, exact-DP codebook (bit-exact floats), Lloyd-Max kernels."""
import pytest
import torch

from tests.util import make_grad, reference_like_codebook

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("nb,period", [(512, 768), (64, 2048), (1000, 12), (5000, 1), (3, 20000), (1, 4096)])
def test_histogram_bit_exact(oracle, cuda_device, dtype, nb, period):
    from gefen_b200.kernels.exact_histogram_fused import gefen_exact_histogram_cuda

    g = make_grad((nb, period), 5, 2, 0, dtype).reshape(-1)
    g[:period].zero_()  # an all-zero block: every element lands in the middle bin
    g[period // 2] = g.abs().max() * 3  # a +absmax element: clamped into the last bin
    want = torch.zeros(4096, dtype=torch.int64)
    oracle.gefen_exact_histogram(g, period, want)
    got = torch.zeros(4096, dtype=torch.int64, device=cuda_device)
    gefen_exact_histogram_cuda(g.to(cuda_device), period, got)
    gefen_exact_histogram_cuda(g.to(cuda_device), period, got)  # counts are added to
    assert int(got.sum()) == 2 * g.numel()
    assert torch.equal(got.cpu(), 2 * want)


def test_histogram_small_bin_count(oracle, cuda_device):
    from gefen_b200.kernels.exact_histogram_fused import gefen_exact_histogram_cuda

    g = make_grad((64, 256), 5, 2, 0).reshape(-1)
    want = torch.zeros(100, dtype=torch.int64)
    oracle.gefen_exact_histogram(g, 256, want)
    got = torch.zeros(100, dtype=torch.int64, device=cuda_device)
    gefen_exact_histogram_cuda(g.to(cuda_device), 256, got)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(768, 768), (64, 2304), (2048, 512), (1000,), (37, 12), (7,), (96, 1536)])
def test_period_scores_and_decision(oracle, cuda_device, dtype, shape):
    from gefen_b200 import partitioning
    from gefen_b200.kernels.period_variance import average_adjacent_log_block_mean_difference_cuda_kernel

    g = make_grad(shape, 7, 4, 0, dtype)
    flat = g.reshape(-1).contiguous()
    n = flat.numel()
    dflat = flat.to(cuda_device)
    cands = oracle.candidate_periods(n)
    assert cands == partitioning.candidate_periods(n)
    for p in cands:
        want = oracle.average_adjacent_log_block_mean_difference(flat, p, False, 1e-12)
        got = average_adjacent_log_block_mean_difference_cuda_kernel(dflat, p, input_is_squared=False, epsilon=1e-12)
        assert got == pytest.approx(want, rel=1e-11, abs=1e-13)
    want_period = oracle.find_period(g, cuda_kernel_semantics=True)
    got_period = partitioning.find_period_by_block_variance(dflat, print_results=False, backend="cuda_kernel",
                                                            input_is_squared=False)
    assert got_period == want_period


def test_period_score_rejects_nonpositive_log_input(cuda_device):
    from gefen_b200.kernels.period_variance import average_adjacent_log_block_mean_difference_cuda_kernel

    values = -torch.ones(64, device=cuda_device)
    with pytest.raises(RuntimeError):
        average_adjacent_log_block_mean_difference_cuda_kernel(values, 8, input_is_squared=True, epsilon=1e-12)
    with pytest.raises(ValueError):
        average_adjacent_log_block_mean_difference_cuda_kernel(values, 64, input_is_squared=True, epsilon=1e-12)


def test_unused_scores_match(oracle, cuda_device):
    from gefen_b200.kernels.period_variance import (
        average_within_block_coefficient_of_variation_cuda_kernel,
        average_within_block_variance_cuda_kernel,
    )

    g = make_grad((128, 512), 3, 3, 0).reshape(-1).contiguous()
    for period in (64, 512, 2048):
        stats = oracle.block_moments(g, period, False, False)
        want = float((stats[0] / (g.numel() // period)).sqrt())
        got = average_within_block_variance_cuda_kernel(g.to(cuda_device), period, input_is_squared=False)
        assert got == pytest.approx(want, rel=1e-4)
        stats = oracle.block_moments(g, period, False, True)
        want = float(stats[0] / stats[1])
        got = average_within_block_coefficient_of_variation_cuda_kernel(g.to(cuda_device), period, input_is_squared=False)
        assert got == pytest.approx(want, rel=1e-4)
    # the opaque custom operator of the variance score (reference: kernels/period_variance.py:49-72)
    opaque = torch.ops.gefen_b200.average_within_block_variance_cuda(g.to(cuda_device), 512, False)
    assert float(opaque) == average_within_block_variance_cuda_kernel(g.to(cuda_device), 512, input_is_squared=False)


@pytest.mark.parametrize("k,force,active", [(256, True, 4096), (256, True, 700), (16, True, 300), (32, False, 1000),
                                            (256, True, 100)])
def test_exact_dp_bit_exact(oracle, cuda_device, k, force, active):
    from gefen_b200 import quantization

    gen = torch.Generator().manual_seed(active + k)
    bins = 4096
    counts = torch.zeros(bins)
    idx = torch.randperm(bins, generator=gen)[:active]
    centre_weight = torch.exp(-((idx.float() - 2048) / 600.0) ** 2)
    counts[idx] = torch.floor(centre_weight * 1e6 * torch.rand(active, generator=gen)) + 1
    edges = torch.linspace(-1, 1, bins + 1)
    centers = 0.5 * (edges[:-1] + edges[1:])
    mask = counts > 0
    want = oracle.exact_dp(centers[mask], counts[mask], k, force)
    got = quantization.exact_dp({"active_centers": centers[mask], "active_counts": counts[mask]}, k, force,
                                device=cuda_device)
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lloyd_kernels(oracle, cuda_device, dtype):
    from gefen_b200.kernels.lloyd_max_fused import gefen_lloyd_accumulate_cuda, gefen_lloyd_mse_cuda, lloyd_max_fit

    cb = reference_like_codebook()
    g = make_grad((200, 1024), 11, 0, 0, dtype).reshape(-1).contiguous()
    want_sums = torch.zeros(256, dtype=torch.float64)
    want_counts = torch.zeros(256, dtype=torch.int64)
    oracle.gefen_lloyd_accumulate(g, cb, 1024, want_sums, want_counts)
    sums = torch.zeros(256, device=cuda_device)
    counts = torch.zeros(256, dtype=torch.int64, device=cuda_device)
    gefen_lloyd_accumulate_cuda(g.to(cuda_device), cb.to(cuda_device), 1024, sums, counts)
    assert torch.equal(counts.cpu(), want_counts)
    assert torch.allclose(sums.cpu().double(), want_sums, rtol=1e-4, atol=1e-3)

    new_cb = (cb * 0.99).contiguous()
    want = oracle.gefen_lloyd_mse(g, cb, new_cb, 1024)
    a = torch.zeros(1, device=cuda_device)
    b = torch.zeros(1, device=cuda_device)
    gefen_lloyd_mse_cuda(g.to(cuda_device), cb.to(cuda_device), new_cb.to(cuda_device), 1024, a, b)
    assert float(a) == pytest.approx(float(want[0]), rel=1e-4)
    assert float(b) == pytest.approx(float(want[1]), rel=1e-4)

    fitted = lloyd_max_fit([(g.to(cuda_device), 1024)], cb.to(cuda_device), iterations=3)
    assert fitted.numel() == 256 and float(fitted[0]) == -1.0 and float(fitted[-1]) == 1.0
    assert bool((fitted[1:] >= fitted[:-1]).all())
