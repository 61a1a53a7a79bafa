"""GPU: this library's kernels and the CPU oracle against the REFERENCE'S OWN CUDA kernels, built
unmodified from the reference sources into oracle/_ref (oracle/build_ref.py). Skipped when that
build is not present. Everything that does not depend on a summation order must be bit-identical."""
import pytest
import torch

from tests.util import make_grad, make_param, reference_like_codebook

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_ext(cuda_device):
    from oracle import build_ref

    module = build_ref.load_module()
    if module is None:
        pytest.skip("oracle/_ref has not been built")
    return module


def _state(nb, period, dtype, seed):
    g = make_grad((nb, period), seed, 0, 0, dtype)
    p = make_param((nb, period), seed, 0, dtype)
    gen = torch.Generator().manual_seed(seed + 5)
    codes = torch.randint(0, 256, (nb, period), dtype=torch.uint8, generator=gen)
    mag = (torch.rand(nb, 1, generator=gen) * 2e-3).to(dtype)
    v = (torch.rand(nb, 1, generator=gen) * 1e-6 + 1e-9).to(dtype)
    return p, g, codes, mag, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("nb,period", [(128, 2048), (64, 512), (40, 1152), (100, 24), (6, 4096)])
def test_step_is_bit_identical_to_the_reference_kernels(ref_ext, oracle, cuda_device, dtype, nb, period):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    cb = reference_like_codebook()
    dcb = cb.to(cuda_device)
    p, g, codes, mag, v = _state(nb, period, dtype, seed=nb + period)
    args = (0.9, 3e-4, 1 - 0.9 ** 3, 1 - 0.999 ** 3, 1e-8)
    rp, rg, rc, rm, rv = (t.clone().to(cuda_device) for t in (p, g, codes, mag, v))
    mp, mg, mc, mm, mv = (t.clone().to(cuda_device) for t in (p, g, codes, mag, v))
    for _ in range(3):
        ref_ext.automatic_gefen_fused_update_from_vmean_cuda(rp, rg, rc, rm, rv, dcb, False, *args)
        automatic_gefen_fused_update_from_vmean_cuda(mp, mg, mc, mm, mv, dcb, False, *args)
        oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, *args)
        torch.cuda.synchronize()
        assert torch.equal(mc, rc) and torch.equal(mm, rm) and torch.equal(mp, rp)
        assert torch.equal(codes, rc.cpu()) and torch.equal(mag, rm.cpu()) and torch.equal(p, rp.cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_period1_and_muon_against_the_reference_kernels(ref_ext, cuda_device, dtype):
    from gefen_b200.kernels.automatic_gefen_fused import (
        automatic_gefen_muon_momentum_cuda,
        automatic_gefen_period1_update_cuda,
    )

    dcb = reference_like_codebook().to(cuda_device)
    n, d = 4096, 256
    g = make_grad((n,), 1, 3, 0, dtype).to(cuda_device)
    p = make_param((n,), 1, 3, dtype).to(cuda_device)
    codes = torch.randint(0, 256, (n, 1), dtype=torch.uint8, device=cuda_device)
    mag = (torch.rand(n // d, 1, device=cuda_device) * 2e-3).to(dtype)
    v = (torch.rand(n, 1, device=cuda_device) * 1e-6).to(dtype)
    a = [t.clone() for t in (p, g, codes, mag, v)]
    b = [t.clone() for t in (p, g, codes, mag, v)]
    args = (d, 0.9, 0.999, 1e-3, 0.19, 0.002, 1e-8)
    ref_ext.automatic_gefen_period1_update_cuda(a[0], a[1], a[2], a[3], a[4], dcb, *args)
    automatic_gefen_period1_update_cuda(b[0], b[1], b[2], b[3], b[4], dcb, *args)
    for x, y in zip(a, b):
        assert torch.equal(x, y)

    nb, period = 48, 1536
    _, g2, c2, m2, _ = _state(nb, period, dtype, seed=9)
    ra = [t.clone().to(cuda_device) for t in (g2, c2, m2)]
    rb = [t.clone().to(cuda_device) for t in (g2, c2, m2)]
    out_a, out_b = torch.empty_like(ra[0]), torch.empty_like(rb[0])
    ref_ext.automatic_gefen_muon_momentum_cuda(ra[0], ra[1], ra[2], dcb, out_a, False, 0.95)
    automatic_gefen_muon_momentum_cuda(rb[0], rb[1], rb[2], dcb, out_b, False, 0.95)
    assert torch.equal(ra[1], rb[1]) and torch.equal(ra[2], rb[2]) and torch.equal(out_a, out_b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_calibration_kernels_against_the_reference_kernels(ref_ext, oracle, cuda_device, dtype):
    from gefen_b200.kernels.automatic_vmean import automatic_vmean_update_cuda
    from gefen_b200.kernels.exact_histogram_fused import gefen_exact_histogram_cuda
    from gefen_b200.kernels.period_variance import average_adjacent_log_block_mean_difference_cuda_kernel

    g = make_grad((256, 768), 3, 1, 0, dtype)
    dg = g.to(cuda_device)
    flat = dg.reshape(-1)
    for period in (768, 96, 4, 1536):
        want = torch.zeros(4096, dtype=torch.int64, device=cuda_device)
        got = torch.zeros_like(want)
        ref_ext.gefen_exact_histogram_cuda(flat, period, want)
        gefen_exact_histogram_cuda(flat, period, got)
        assert torch.equal(got, want)                       # integers: bit-exact
        ref_score = float(ref_ext.average_adjacent_log_block_mean_difference_cuda(flat, period, False, 1e-12).item())
        my_score = average_adjacent_log_block_mean_difference_cuda_kernel(flat, period, input_is_squared=False, epsilon=1e-12)
        assert my_score == pytest.approx(ref_score, rel=1e-11)   # fp64 sums in a different order
    v_ref = (torch.rand(256, 1, device=cuda_device) * 1e-6).to(dtype)
    v_mine = v_ref.clone()
    v_cpu = v_ref.cpu().clone()
    ref_ext.automatic_vmean_update_cuda(v_ref, dg, 0.999)
    automatic_vmean_update_cuda(v_mine, dg, 0.999)
    oracle.automatic_vmean_update(v_cpu, g, 0.999)
    assert torch.equal(v_cpu, v_ref.cpu())                  # the oracle restates the kernel's summation order
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert torch.allclose(v_mine.float(), v_ref.float(), rtol=tol, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nb,period", [(64, 512), (33, 24), (5, 4096), (17, 130), (33, 25), (8, 9), (5, 4097), (1, 7)])
def test_packed_4bit_codes_against_the_reference_kernels(ref_ext, oracle, cuda_device, dtype, nb, period):
    """packed_indices=True: two 4-bit codes per byte, a 16-entry codebook (reference:
    automatic_gefen_fused_kernel.cu:14-57). Bit-identical codes, magnitudes and parameters for the
    AdamW step and for GefenMuon's momentum. Odd periods, where neighbouring blocks share a byte (the reference
    updates nibbles with atomicCAS), included."""
    from gefen_b200.kernels.automatic_gefen_fused import (
        automatic_gefen_fused_update_from_vmean_cuda,
        automatic_gefen_muon_momentum_cuda,
    )

    cb = torch.sort(torch.tanh(torch.linspace(-2.0, 2.0, 16))).values.float().contiguous()
    cb[0], cb[-1] = -1.0, 1.0
    dcb = cb.to(cuda_device)
    p, g, _, mag, v = _state(nb, period, dtype, seed=nb * 7 + period)
    gen = torch.Generator().manual_seed(nb + period)
    packed = torch.randint(0, 256, ((nb * period + 1) // 2,), dtype=torch.uint8, generator=gen)
    args = (0.9, 3e-4, 1 - 0.9 ** 3, 1 - 0.999 ** 3, 1e-8)
    rp, rg, rc, rm, rv = (t.clone().to(cuda_device) for t in (p, g, packed, mag, v))
    mp, mg, mc, mm, mv = (t.clone().to(cuda_device) for t in (p, g, packed, mag, v))
    op, oc, om = p.clone(), packed.clone(), mag.clone()
    for _ in range(3):
        ref_ext.automatic_gefen_fused_update_from_vmean_cuda(rp, rg, rc, rm, rv, dcb, True, *args)
        automatic_gefen_fused_update_from_vmean_cuda(mp, mg, mc, mm, mv, dcb, True, *args)
        oracle.automatic_gefen_fused_update_from_vmean(op, g, oc, om, v, cb, True, *args)
        torch.cuda.synchronize()
        assert torch.equal(mc, rc) and torch.equal(mm, rm) and torch.equal(mp, rp)
        assert torch.equal(oc, rc.cpu()) and torch.equal(om, rm.cpu()) and torch.equal(op, rp.cpu())
    out_r, out_m = torch.empty_like(rg), torch.empty_like(mg)
    ref_ext.automatic_gefen_muon_momentum_cuda(rg, rc, rm, dcb, out_r, True, 0.95)
    automatic_gefen_muon_momentum_cuda(mg, mc, mm, dcb, out_m, True, 0.95)
    torch.cuda.synchronize()
    assert torch.equal(mc, rc) and torch.equal(mm, rm) and torch.equal(out_m, out_r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,period", [(200, 1024), (64, 96), (3, 12000)])
def test_lloyd_kernels_against_the_reference_kernels(ref_ext, cuda_device, dtype, rows, period):
    """Lloyd-Max E-step and logging MSE (reference: lloyd_max_fused_kernel.cu:50-195): the per-entry
    counts are integers and must be identical; the per-entry sums and the two squared errors are fp32
    atomics in the reference (order-dependent there too): 1e-5 relative to the largest sum."""
    from gefen_b200.kernels.lloyd_max_fused import gefen_lloyd_accumulate_cuda, gefen_lloyd_mse_cuda

    cb = reference_like_codebook().to(cuda_device)
    new_cb = (cb * 0.99).contiguous()
    g = make_grad((rows, period), 11, 0, 0, dtype).to(cuda_device).reshape(-1).contiguous()
    want_sums = torch.zeros(256, device=cuda_device)
    want_counts = torch.zeros(256, dtype=torch.int64, device=cuda_device)
    got_sums, got_counts = torch.zeros_like(want_sums), torch.zeros_like(want_counts)
    ref_ext.gefen_lloyd_accumulate_cuda(g, cb, period, want_sums, want_counts)
    gefen_lloyd_accumulate_cuda(g, cb, period, got_sums, got_counts)
    assert torch.equal(got_counts, want_counts)
    assert int(got_counts.sum()) == g.numel()
    scale = float(want_sums.abs().max())
    assert float((got_sums - want_sums).abs().max()) <= 1e-5 * scale
    want = [torch.zeros(1, device=cuda_device) for _ in range(2)]
    got = [torch.zeros(1, device=cuda_device) for _ in range(2)]
    ref_ext.gefen_lloyd_mse_cuda(g, cb, new_cb, period, want[0], want[1])
    gefen_lloyd_mse_cuda(g, cb, new_cb, period, got[0], got[1])
    for a, b in zip(got, want):
        assert float(a) == pytest.approx(float(b), rel=1e-4)
