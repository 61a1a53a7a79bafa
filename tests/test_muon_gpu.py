"""GPU: GefenMuon against the oracle's restatement of the reference loop. The quantised momentum is
integer work (codes bit-exact); Newton-Schulz is bf16 matrix products whose accumulation order is not
pinned by the reference (cuBLAS on its GPU path, oneDNN on its CPU path), so parameters are compared
with the bf16 tolerance."""
import pytest
import torch

from tests.util import make_grad, make_param, rel_l2

pytestmark = pytest.mark.gpu


def _assert_one_bf16_rounding(out: torch.Tensor, want: torch.Tensor) -> None:
    """`out` (bf16) is one rounding of an fp32-accumulated result whose exact value is `want` (fp32):
    per element |err| <= 2^-8 |want| + 2^-9 rms(want). A dropped K-slice, a wrong tile or a missing
    beta*C term is far outside this."""
    want = want.float()
    err = (out.float() - want).abs()
    bound = want.abs() * 2.0 ** -8 + float(want.square().mean().sqrt()) * 2.0 ** -9
    worst = float((err - bound).max())
    assert worst <= 0.0, "largest excess over the rounding bound: {:.3e}".format(worst)

SHAPES = [(128, 256), (256, 128), (192, 192), (64, 1536)]


@pytest.mark.parametrize("dtype,nesterov", [(torch.bfloat16, True), (torch.bfloat16, False), (torch.float32, True)])
def test_muon_steps_match_oracle(oracle, cuda_device, dtype, nesterov):
    from gefen_b200 import GefenMuon
    from oracle.ref_loop import OracleGefenMuon

    cpu = [make_param(s, 0, i, dtype) for i, s in enumerate(SHAPES)]
    gpu = [torch.nn.Parameter(p.clone().to(cuda_device)) for p in cpu]
    ref = OracleGefenMuon(cpu, lr=0.02, weight_decay=0.1, momentum=0.95, nesterov=nesterov)
    opt = GefenMuon(gpu, lr=0.02, weight_decay=0.1, momentum=0.95, nesterov=nesterov)
    for step in range(4):
        grads = [make_grad(s, 0, i, step, dtype, tau=0.5) for i, s in enumerate(SHAPES)]
        for p, g in zip(gpu, grads):
            p.grad = g.to(cuda_device)
        opt.step()
        ref.step(grads)
    assert torch.equal(opt._gefen_codebook.cpu(), ref.codebook)
    for p, pc, st in zip(gpu, cpu, ref.state):
        assert opt.state[p]["automatic_period"] == st["automatic_period"]
        assert "vmean" not in opt.state[p]
        codes = opt.state[p]["m_codebook"].cpu().reshape(-1).int()
        diff = (codes - st["m_codebook"].reshape(-1).int()).abs()
        assert float((diff == 0).float().mean()) >= 0.9999 and int(diff.max()) <= 1
        assert torch.equal(opt.state[p]["m_magnitude"].cpu().reshape(-1), st["m_magnitude"].reshape(-1))
        assert rel_l2(p.detach().cpu(), pc) <= 1e-2
        assert opt.state[p]["step"] == 4


def test_muon_rejects_non_matrices(cuda_device):
    from gefen_b200 import GefenMuon

    with pytest.raises(ValueError):
        GefenMuon([torch.nn.Parameter(torch.zeros(8, device=cuda_device))])
    with pytest.raises(ValueError):
        GefenMuon([torch.nn.Parameter(torch.zeros(4, 4, device=cuda_device))], adjust_lr_fn="nope")


def test_newton_schulz_orthogonalises(cuda_device):
    from gefen_b200.newton_schulz import zeropower_via_newtonschulz

    torch.manual_seed(0)
    for shape in [(256, 512), (512, 256), (384, 384)]:
        g = torch.randn(shape, device=cuda_device).bfloat16()
        x = zeropower_via_newtonschulz(g, (3.4445, -4.7750, 2.0315), 5, 1e-7).float()
        small = x if shape[0] <= shape[1] else x.T
        sv = torch.linalg.svdvals(small)
        # five steps push the bulk of the singular values into the band around 1 (the smallest ones of
        # a square random matrix start near zero and need more steps)
        assert float(sv.max()) < 1.3 and 0.6 < float(sv.median()) < 1.25


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 1024), (384, 640, 200), (2048, 2048, 512), (96, 72, 136),
                                   (1024, 1024, 2048),
                                   # more tiles than SMs: persistent CTAs, two accumulator buffers, ragged last round
                                   (2048, 5120, 192), (2200, 4104, 72)])
def test_tcgen05_gemm_against_fp32_matmul(cuda_device, M, N, K):
    """The tensor-core GEMM against an fp32 torch reference on the same bf16 inputs: one rounding to
    bf16 of an fp32-accumulated result, so the error is half a bf16 ulp of the result plus fp32
    accumulation noise (see _assert_one_bf16_rounding)."""
    from gefen_b200.newton_schulz import check_status, gemm_tn

    gen = torch.Generator(device=cuda_device).manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=gen, device=cuda_device) / K ** 0.5).bfloat16()
    b = torch.randn(N, K, generator=gen, device=cuda_device).bfloat16()
    c = torch.randn(M, N, generator=gen, device=cuda_device).bfloat16()
    want = 0.75 * (a.float() @ b.float().T) - 1.25 * c.float()
    out_t = torch.empty(N, M, dtype=torch.bfloat16, device=cuda_device)
    out = gemm_tn(a, b, c=c, alpha=0.75, beta=-1.25, out_t=out_t)
    check_status(cuda_device)
    _assert_one_bf16_rounding(out, want)
    assert torch.equal(out_t, out.T.contiguous())
    plain = gemm_tn(a, b)
    _assert_one_bf16_rounding(plain, a.float() @ b.float().T)


def test_newton_schulz_matches_library_gemms(cuda_device):
    """Same iteration on torch's GEMMs (the reference's GPU path): bf16-level agreement."""
    from gefen_b200 import newton_schulz as ns

    torch.manual_seed(1)
    for shape in [(256, 512), (512, 256), (384, 384), (1024, 2048)]:
        g = (torch.randn(shape, device=cuda_device) * 1e-3).bfloat16()
        mine = ns.zeropower_via_newtonschulz(g, (3.4445, -4.7750, 2.0315), 5, 1e-7).float()
        ns.check_status(cuda_device)
        x = g / g.norm().clamp(min=1e-7)
        if shape[0] > shape[1]:
            x = x.T
        for _ in range(5):
            gram = x @ x.T
            x = torch.addmm(x, torch.addmm(gram, gram, gram, beta=-4.7750, alpha=2.0315), x, beta=3.4445)
        want = (x.T if shape[0] > shape[1] else x).float()
        assert mine.shape == want.shape
        assert float((mine - want).norm() / want.norm()) <= 2e-2


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 1024), (384, 640, 200), (2048, 6144, 2048), (96, 72, 136)])
def test_tcgen05_gemm_with_row_major_b(cuda_device, M, N, K):
    """B given as [K, N] row-major: an MN-major tensor-core operand, no transposed copy."""
    from gefen_b200.newton_schulz import check_status, gemm_nn

    gen = torch.Generator(device=cuda_device).manual_seed(M * 3 + N + K)
    a = (torch.randn(M, K, generator=gen, device=cuda_device) / K ** 0.5).bfloat16()
    b = torch.randn(K, N, generator=gen, device=cuda_device).bfloat16()
    c = torch.randn(M, N, generator=gen, device=cuda_device).bfloat16()
    want = 1.5 * (a.float() @ b.float()) + 0.5 * c.float()
    out = gemm_nn(a, b, c=c, alpha=1.5, beta=0.5)
    check_status(cuda_device)
    _assert_one_bf16_rounding(out, want)


@pytest.mark.parametrize("m,k", [(128, 256), (384, 200), (2048, 1024), (1000, 512), (4224, 128), (6144, 64)])
def test_tcgen05_gemm_symmetric_output(cuda_device, m, k):
    """Gram matrix with only the upper-triangle tiles computed and mirrored: bit-identical to the full product."""
    from gefen_b200.newton_schulz import check_status, gemm_tn

    gen = torch.Generator(device=cuda_device).manual_seed(m + k)
    x = (torch.randn(m, k, generator=gen, device=cuda_device) / k ** 0.5).bfloat16()
    full = gemm_tn(x, x)
    sym = torch.full((m, m), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    gemm_tn(x, x, out=sym, symmetric=True)
    check_status(cuda_device)
    assert torch.equal(sym, full)
    assert torch.equal(sym, sym.T.contiguous())
    poly_full = gemm_tn(full, full, c=full, alpha=2.0315, beta=-4.775)
    poly_sym = torch.full((m, m), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    gemm_tn(full, full, c=full, alpha=2.0315, beta=-4.775, out=poly_sym, symmetric=True)
    check_status(cuda_device)
    assert torch.equal(poly_sym, poly_full)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(256, 512), (1000, 3), (8,), (5,)])
def test_fused_apply_matches_the_two_torch_kernels(cuda_device, dtype, shape):
    """gefen_b200_muon_apply against the reference's tail (gefen_muon.py:326-329): `p.mul_(1 - lr*wd)` then
    `p.add_(update, alpha=-adjusted_lr)`, each rounding to the parameter dtype. The only freedom is whether
    the second step is one fused multiply-add: within one rounding of the parameter dtype."""
    from gefen_b200 import _lib

    lib = _lib.load()
    gen = torch.Generator(device=cuda_device).manual_seed(sum(shape))
    p = (torch.randn(shape, generator=gen, device=cuda_device) * 0.02).to(dtype)
    u = torch.randn(shape, generator=gen, device=cuda_device).to(dtype)
    for wd_mul, alpha in ((1 - 0.02 * 0.1, -0.02 * 1.4142), (1.0, -0.5)):
        want = p.clone()
        if wd_mul != 1.0:
            want.mul_(wd_mul)
        want.add_(u, alpha=alpha)
        got = p.clone()
        _lib.check(lib.gefen_b200_muon_apply(_lib.ptr(got), _lib.ptr(u), _lib.dtype_tag(dtype), got.numel(), wd_mul, alpha,
                                             None, 0, _lib.current_stream(cuda_device)))
        ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -24}[dtype]
        err = (got.float() - want.float()).abs()
        assert bool((err <= ulp * want.float().abs() * 1.01 + 1e-30).all())
