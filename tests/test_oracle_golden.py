"""CPU: the oracle against outputs of the reference itself (tests/golden/reference_golden.pt, made by
tests/golden/make_golden.py from the reference's own code)."""
from pathlib import Path

import torch

from tests.util import make_grad, make_param, rel_l2

GOLDEN = torch.load(Path(__file__).resolve().parent / "golden" / "reference_golden.pt", weights_only=False)


def test_nearest_entry_rule(oracle):
    g = GOLDEN["nearest"]
    assert torch.equal(oracle.nearest_indices(g["codebook"], g["x"]), g["index"])


def test_exact_dp_bit_exact(oracle):
    edges = torch.linspace(-1, 1, 4097)
    centers = 0.5 * (edges[:-1] + edges[1:])
    for case in GOLDEN["exact_dp"]:
        m = case["counts"] > 0
        got = oracle.exact_dp(centers[m], case["counts"][m], case["k"], case["force"])
        assert torch.equal(got, case["codebook"]), (case["k"], case["force"])


def test_period_decisions(oracle):
    for case in GOLDEN["periods"]:
        dtype = torch.bfloat16 if "bfloat16" in case["dtype"] else torch.float32
        g = make_grad(case["shape"], case["seed"], case["index"], 0, dtype)
        assert oracle.find_period(g, cuda_kernel_semantics=False) == case["period"], case
        # the CUDA backend squares in fp64 instead of fp32; on structured gradients the decision is the same
        if len(case["shape"]) == 2:
            assert oracle.find_period(g, cuda_kernel_semantics=True) == case["period"], case


def test_ten_steps_against_the_reference_cpu_path(oracle):
    """The reference's CPU path (lerp, rounded-magnitude normalisation) and its CUDA kernels (which
    the oracle restates) are different roundings of the same algorithm: periods and the codebook
    are identical, codes agree on >= 99.99 % of the elements and differ by at most 2 after ten
    free-running steps, parameters agree to 5e-5 relative L2 (the two reference paths themselves drift
    apart by about 1e-5 over ten steps: lerp against fma, sqrt(v)/sqrt(bc2) against sqrt(v/bc2)).
    The bit-level pin of the kernel arithmetic is the GPU comparison with the reference's own CUDA
    build, tests/test_reference_kernels_gpu.py."""
    from oracle.ref_loop import OracleGefen

    ref = GOLDEN["ten_steps_fp32"]
    shapes = ref["shapes"]
    params = [make_param(s, 0, i) if len(s) == 2 else torch.ones(s) for i, s in enumerate(shapes)]
    opt = OracleGefen(params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    for step in range(10):
        opt.step([make_grad(s, 0, i, step) for i, s in enumerate(shapes)])
    assert [st["automatic_period"] for st in opt.state] == ref["periods"]
    assert torch.equal(opt.codebook, ref["codebook"])
    total = agree = 0
    for p, st, rp, rc in zip(params, opt.state, ref["params"], ref["codes"]):
        diff = (st["m_codebook"].int() - rc.int()).abs()
        assert int(diff.max()) <= 2
        total += diff.numel()
        agree += int((diff == 0).sum())
        assert rel_l2(p, rp) <= 5e-5
    assert agree / total >= 0.9999


def test_contraction_modes_differ_only_in_rounding(oracle):
    from tests.util import reference_like_codebook

    cb = reference_like_codebook()
    g = make_grad((32, 512), 1, 0, 0)
    outs = []
    for mode in (0, 1):
        oracle.set_contraction(mode)
        p = make_param((32, 512), 1, 0)
        codes = torch.zeros(32, 512, dtype=torch.uint8)
        mag = torch.zeros(32, 1)
        v = torch.full((32, 1), 1e-6)
        oracle.automatic_gefen_fused_update_from_vmean(p, g, codes, mag, v, cb, False, 0.9, 1e-3, 0.1, 0.001, 1e-8)
        outs.append((p, codes))
    oracle.set_contraction(1)
    assert float((outs[0][1] == outs[1][1]).float().mean()) > 0.999
    assert rel_l2(outs[0][0], outs[1][0]) < 1e-6


def test_one_pass_period_scores_equal_the_per_period_function(oracle):
    """The oracle scores all candidate periods of a tensor from one array of logarithms; the sums are
    added in the same order as by the per-period restatement of the reference kernel, so the scores
    must be bit-identical (and the decisions with them)."""
    import torch

    from tests.util import make_grad

    for shape, dtype in [((96, 768), torch.float32), ((64, 2304), torch.bfloat16), ((1000,), torch.float32), ((37, 12), torch.bfloat16)]:
        g = make_grad(shape, 4, 2, 0, dtype).reshape(-1).contiguous()
        cands = oracle.candidate_periods(g.numel())
        many = oracle.adjacent_log_scores(g, cands, False, 1e-12)
        single = [oracle.average_adjacent_log_block_mean_difference(g, p, False, 1e-12) for p in cands]
        assert many == single
