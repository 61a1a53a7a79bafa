"""GPU parity of the step kernels against the CPU oracle, through the reference-shaped wrappers
(which call the C ABI). Integer outputs (codes) and the stored magnitudes must be bit-exact; the
north-star tolerance (>= 99.99 % equal codes, |diff| <= 1 elsewhere) is asserted as well so that a
failure report says how far off a kernel is."""
import pytest
import torch

from tests.util import make_grad, make_param, reference_like_codebook, rel_l2

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]
# (num_blocks, period): fast path (multiples of 8 up to 2048, ragged last pass included), the generic
# warp path (odd / tiny periods) and the generic CTA path (period > 2048)
SHAPES = [(64, 512), (33, 768), (20, 1152), (16, 2048), (9, 1120), (7, 1664), (5, 8), (40, 24), (11, 12),
          (301, 1), (13, 37), (6, 4096), (3, 3000), (2, 10007),
          # long blocks and more blocks than one wave of warps
          (700, 512), (333, 2048), (5, 5000), (4, 6144), (3, 8192), (2, 7688), (50, 520), (9, 1536),
          # blocks shorter than 256 elements share a warp (32, 16, 8, 4, 2 blocks per pass), ragged last pass
          (37, 128), (101, 64), (1001, 16), (67, 8), (3, 256), (50, 40), (21, 104), (1, 8)]


def _state(nb, period, dtype, state_dtype, seed):
    g = make_grad((nb, period), seed, 0, 0, dtype)
    p = make_param((nb, period), seed, 0, dtype)
    gen = torch.Generator().manual_seed(seed + 5)
    codes = torch.randint(0, 256, (nb, period), dtype=torch.uint8, generator=gen)
    mag = (torch.rand(nb, 1, generator=gen) * 2e-3).to(state_dtype)
    v = (torch.rand(nb, 1, generator=gen) * 1e-6 + 1e-9).to(state_dtype)
    return p, g, codes, mag, v


def _assert_codes(got, want):
    got = got.cpu().int()
    want = want.int()
    diff = (got - want).abs()
    frac = float((diff == 0).float().mean())
    assert frac >= 0.9999, "only {:.6f} of the codes agree".format(frac)
    assert int(diff.max()) <= 1
    assert frac == 1.0, "codes are within tolerance but not bit-exact ({:.8f})".format(frac)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nb,period", SHAPES)
def test_fused_update_from_vmean(oracle, cuda_device, dtype, nb, period):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    cb = reference_like_codebook()
    p, g, codes, mag, v = _state(nb, period, dtype, dtype, seed=nb * 131 + period)
    args = dict(beta1=0.9, lr=3e-4, bias_correction_1=1 - 0.9 ** 3, bias_correction_2=1 - 0.999 ** 3, eps=1e-8)
    dp, dg, dc, dm, dv = (t.to(cuda_device) for t in (p, g, codes, mag, v))
    dcb = cb.to(cuda_device)
    for _ in range(3):  # three steps from the same starting state on both sides
        oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, **args)
        automatic_gefen_fused_update_from_vmean_cuda(dp, dg, dc, dm, dv, dcb, False, **args)
        _assert_codes(dc, codes)
        assert torch.equal(dm.cpu(), mag)
        assert torch.equal(dp.cpu(), p)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_update_zero_lr_and_zero_block(oracle, cuda_device, dtype):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    cb = reference_like_codebook()
    nb, period = 8, 512
    p, g, codes, mag, v = _state(nb, period, dtype, dtype, seed=3)
    g[2].zero_()
    mag[2] = 0  # all-zero block: absmax 0, normalised 0
    p0 = p.clone()
    dp, dg, dc, dm, dv = (t.to(cuda_device) for t in (p, g, codes, mag, v))
    args = dict(beta1=0.9, lr=0.0, bias_correction_1=0.1, bias_correction_2=0.001, eps=1e-8)
    oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, **args)
    automatic_gefen_fused_update_from_vmean_cuda(dp, dg, dc, dm, dv, cb.to(cuda_device), False, **args)
    assert torch.equal(dp.cpu(), p0) and torch.equal(p, p0)  # lr == 0 leaves p untouched
    _assert_codes(dc, codes)
    assert torch.equal(dm.cpu(), mag)
    assert float(dm[2]) == 0.0


def test_fused_update_fp64_and_mixed_state(oracle, cuda_device):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    cb = reference_like_codebook()
    for dtype, mag_dt, v_dt in [(torch.float64, torch.float32, torch.float32),
                                (torch.bfloat16, torch.float32, torch.float16),
                                (torch.float32, torch.bfloat16, torch.float32)]:
        nb, period = 12, 1024
        p, g, codes, mag, v = _state(nb, period, dtype, torch.float32, seed=17)
        mag, v = mag.to(mag_dt), v.to(v_dt)
        dp, dg, dc, dm, dv = (t.to(cuda_device) for t in (p, g, codes, mag, v))
        args = dict(beta1=0.9, lr=1e-3, bias_correction_1=0.19, bias_correction_2=0.002, eps=1e-8)
        oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, **args)
        automatic_gefen_fused_update_from_vmean_cuda(dp, dg, dc, dm, dv, cb.to(cuda_device), False, **args)
        _assert_codes(dc, codes)
        assert torch.equal(dm.cpu(), mag)
        assert torch.equal(dp.cpu(), p)


@pytest.mark.parametrize("dtype", DTYPES)
def test_precomputed_stepsize(oracle, cuda_device, dtype):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_cuda

    cb = reference_like_codebook()
    nb, period = 24, 768
    p, g, codes, mag, _ = _state(nb, period, dtype, dtype, seed=4)
    step = torch.rand(nb, 1) * 1e3
    dp, dg, dc, dm, ds = (t.to(cuda_device) for t in (p, g, codes, mag, step))
    oracle.automatic_gefen_fused_update(p, g, codes, mag, step, cb, False, 0.9, 1e-3)
    automatic_gefen_fused_update_cuda(dp, dg, dc, dm, ds, cb.to(cuda_device), False, 0.9, 1e-3)
    _assert_codes(dc, codes)
    assert torch.equal(dm.cpu(), mag)
    assert torch.equal(dp.cpu(), p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("numel,divisor", [(2048, 256), (768, 256), (770, 154), (1, 1), (8192, 256), (97, 97)])
def test_period1_update(oracle, cuda_device, dtype, numel, divisor):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_period1_update_cuda

    cb = reference_like_codebook()
    g = make_grad((numel,), 1, 3, 0, dtype)
    p = make_param((numel,), 1, 3, dtype)
    gen = torch.Generator().manual_seed(9)
    codes = torch.randint(0, 256, (numel, 1), dtype=torch.uint8, generator=gen)
    mag = (torch.rand(numel // divisor, 1, generator=gen) * 2e-3).to(dtype)
    v = (torch.rand(numel, 1, generator=gen) * 1e-6).to(dtype)
    dp, dg, dc, dm, dv = (t.to(cuda_device) for t in (p, g, codes, mag, v))
    args = (divisor, 0.9, 0.999, 1e-3, 1 - 0.9 ** 2, 1 - 0.999 ** 2, 1e-8)
    for _ in range(2):
        oracle.automatic_gefen_period1_update(p, g, codes, mag, v, cb, *args)
        automatic_gefen_period1_update_cuda(dp, dg, dc, dm, dv, cb.to(cuda_device), *args)
        _assert_codes(dc, codes)
        assert torch.equal(dm.cpu(), mag)
        assert torch.equal(dv.cpu(), v)
        assert torch.equal(dp.cpu(), p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nb,period", [(32, 1024), (10, 1536), (7, 2048), (19, 20), (3, 6144)])
def test_muon_momentum(oracle, cuda_device, dtype, nb, period):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_muon_momentum_cuda

    cb = reference_like_codebook()
    _, g, codes, mag, _ = _state(nb, period, dtype, dtype, seed=period)
    out = torch.empty_like(g)
    dg, dc, dm = (t.to(cuda_device) for t in (g, codes, mag))
    dout = torch.empty_like(dg)
    for _ in range(2):
        oracle.automatic_gefen_muon_momentum(g, codes, mag, cb, out, False, 0.95)
        automatic_gefen_muon_momentum_cuda(dg, dc, dm, cb.to(cuda_device), dout, False, 0.95)
        _assert_codes(dc, codes)
        assert torch.equal(dm.cpu(), mag)
        assert torch.equal(dout.cpu(), out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nb,period", [(64, 512), (9, 2048), (100, 12), (4, 5000)])
def test_vmean_update(oracle, cuda_device, dtype, nb, period):
    """The block sum of squares is accumulated in a different (but fixed) order than the reference's
    thread-strided tree, so fp32 results agree to rounding of the sum, not bit for bit."""
    from gefen_b200.kernels.automatic_vmean import automatic_vmean_update_cuda

    g = make_grad((nb, period), 2, 1, 0, dtype)
    v = (torch.rand(nb, 1) * 1e-6).to(dtype)
    dv, dg = v.to(cuda_device), g.to(cuda_device)
    oracle.automatic_vmean_update(v, g, 0.999)
    automatic_vmean_update_cuda(dv, dg, 0.999)
    tol = 2e-6 if dtype == torch.float32 else (8e-3 if dtype == torch.bfloat16 else 1e-3)
    assert torch.allclose(dv.cpu().float(), v.float(), rtol=tol, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("period", [128, 512, 2048, 3000])   # several blocks per warp, one block per warp, ragged
def test_nonfinite_gradients_follow_the_reference(oracle, cuda_device, dtype, period):
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    cb = reference_like_codebook()
    nb = 6
    p, g, codes, mag, v = _state(nb, period, dtype, dtype, seed=8)
    g[1, 5] = float("nan")
    g[3, 7] = float("inf")
    g[4, 0] = float("-inf")
    g[4, 9] = float("nan")
    g[5, period - 1] = float("nan")      # the last warp of the block holds it
    dp, dg, dc, dm, dv = (t.to(cuda_device) for t in (p, g, codes, mag, v))
    args = dict(beta1=0.9, lr=1e-3, bias_correction_1=0.1, bias_correction_2=0.001, eps=1e-8)
    oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, **args)
    automatic_gefen_fused_update_from_vmean_cuda(dp, dg, dc, dm, dv, cb.to(cuda_device), False, **args)
    _assert_codes(dc, codes)
    assert torch.equal(dm.cpu(), mag)
    assert torch.equal(torch.nan_to_num(dp.cpu(), nan=7.0), torch.nan_to_num(p, nan=7.0))


def test_degenerate_codebooks(oracle, cuda_device):
    """Duplicates (the padded path of the codebook fit), fewer than 256 entries, a largest entry below 1."""
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    books = [
        torch.tensor([-1.0, -0.5, -0.5, -0.5, 0.0, 0.0, 0.25, 0.2500001, 1.0]),
        torch.cat([torch.linspace(-1, 0.3, 40), torch.full((216,), 0.3)]),
        torch.tensor([0.3]),
        torch.linspace(-0.7, 0.6, 16),
    ]
    for cb in books:
        cb = cb.float().contiguous()
        nb, period = 10, 1024
        p, g, codes, mag, v = _state(nb, period, torch.float32, torch.float32, seed=21)
        codes.clamp_(max=cb.numel() - 1)
        dp, dg, dc, dm, dv = (t.to(cuda_device) for t in (p, g, codes, mag, v))
        args = dict(beta1=0.9, lr=1e-3, bias_correction_1=0.1, bias_correction_2=0.001, eps=1e-8)
        oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, **args)
        automatic_gefen_fused_update_from_vmean_cuda(dp, dg, dc, dm, dv, cb.to(cuda_device), False, **args)
        _assert_codes(dc, codes)
        assert torch.equal(dp.cpu(), p)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_multi_tensor_step_matches_per_tensor_sequence(oracle, cuda_device, dtype):
    """One multi-tensor launch (fused second moment + weight decay + step) over tensors of every
    kernel class against the oracle's per-tensor sequence vmean -> weight decay -> step."""
    import numpy as np

    from gefen_b200 import _lib

    lib = _lib.load()
    cb = reference_like_codebook()
    dcb = cb.to(cuda_device)
    ws = _lib.codebook_workspace(dcb)
    shapes = [(64, 1), (16, 12), (96, 64), (1, 1), (64, 192), (40, 36), (32, 512), (8, 2048), (3, 4096), (2, 10000)]
    lr, wd, beta1, beta2, eps = 1e-3, 0.1, 0.9, 0.999, 1e-8
    bc1, bc2 = 1 - beta1 ** 2, 1 - beta2 ** 2
    host, dev = [], []
    for i, (nb, period) in enumerate(shapes):
        p, g, codes, mag, v = _state(nb, period, dtype, dtype, seed=50 + i)
        period1 = period == 1
        if period1:  # per-element vmean, one magnitude for the whole tensor
            mag = mag[:1].clone()
        host.append((p, g, codes, mag, v, period1))
        dev.append(tuple(t.clone().to(cuda_device) for t in (p, g, codes, mag, v)))
    rows = np.zeros(len(shapes), dtype=_lib.STEP_TENSOR_DTYPE)
    for r, ((nb, period), (dp, dg, dc, dm, dv)) in enumerate(zip(shapes, dev)):
        period1 = period == 1
        block = nb if period1 else period
        rows[r]["p"], rows[r]["g"], rows[r]["codes"] = dp.data_ptr(), dg.data_ptr(), dc.data_ptr()
        rows[r]["mag"], rows[r]["v"] = dm.data_ptr(), dv.data_ptr()
        rows[r]["num_blocks"] = 1 if period1 else nb
        rows[r]["period"] = block
        rows[r]["flags"] = (_lib.STEP_PERIOD1 if period1 else _lib.STEP_FUSE_VMEAN) | _lib.STEP_WEIGHT_DECAY
        rows[r]["mag_dtype"] = rows[r]["v_dtype"] = _lib.dtype_tag(dtype)
    for k, val in dict(beta1=beta1, beta2=beta2, lr=lr, bc1=bc1, bc2=bc2, eps=eps, wd_mul=1 - lr * wd).items():
        rows[k] = val
    tag = _lib.dtype_tag(dtype)
    classes = [lib.gefen_b200_step_tensor_class(rows[r:r + 1].ctypes.data, tag) for r in range(len(shapes))]
    assert set(classes) >= {1, 0, -1} and set(classes) <= {2, 1, 0, -1}
    order = sorted(range(len(shapes)), key=lambda r: classes[r])
    rows = np.ascontiguousarray(rows[order])
    table = torch.empty(rows.nbytes, dtype=torch.uint8, device=cuda_device)
    _lib.check(lib.gefen_b200_multi_tensor_step(rows.ctypes.data, _lib.ptr(table), len(shapes), tag, _lib.ptr(ws),
                                                _lib.current_stream(cuda_device)))
    torch.cuda.synchronize()
    for (nb, period), (p, g, codes, mag, v, period1), (dp, dg, dc, dm, dv) in zip(shapes, host, dev):
        oracle.weight_decay(p, lr, wd)
        if period1:
            oracle.automatic_gefen_period1_update(p, g.reshape(-1), codes, mag, v, cb, nb, beta1, beta2, lr, bc1, bc2, eps)
        else:
            oracle.automatic_vmean_update(v, g, beta2)
            oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, beta1, lr, bc1, bc2, eps)
        _assert_codes(dc, codes)
        assert torch.equal(dm.cpu(), mag)
        if period1:
            assert torch.equal(dv.cpu(), v) and torch.equal(dp.cpu(), p)
        else:  # the block sum of squares is formed in a different order: rounding-level differences
            tol = 2e-6 if dtype == torch.float32 else 8e-3
            assert torch.allclose(dv.cpu().float(), v.float(), rtol=tol, atol=0)
            assert rel_l2(dp.cpu(), p) <= (1e-6 if dtype == torch.float32 else 2e-3)
