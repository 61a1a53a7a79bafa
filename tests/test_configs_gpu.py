"""GPU: the benchmark configurations at their real sizes.

Config 1 (GPT-2 125M, fp32, 148 tensors, 10 steps) is small enough for the CPU oracle to follow in
full. The larger ones are checked through properties that do not need the oracle at full size: a
multi-tensor step must equal the same tensors stepped one by one, sharded ownership must not change
a bit, and magnitudes must equal the absmax that torch computes from the dequantised state."""
import pytest
import torch

from gefen_b200 import workloads
from tests.util import rel_l2

pytestmark = pytest.mark.gpu


def test_config1_gpt2_125m_ten_steps_against_oracle(oracle, cuda_device):
    from gefen_b200 import Gefen
    from oracle.ref_loop import OracleGefen

    shapes = workloads.gpt2_125m()
    cpu = [workloads.init_param(n, s, i, torch.float32, torch.device("cpu")) for i, (n, s) in enumerate(shapes)]
    gpu = [torch.nn.Parameter(p.clone().to(cuda_device)) for p in cpu]
    opt = Gefen([(n, p) for (n, _), p in zip(shapes, gpu)], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    ref = OracleGefen(cpu, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    for step in range(10):
        grads = [workloads.make_grad(s, i, step, torch.float32, torch.device("cpu")) for i, (_, s) in enumerate(shapes)]
        for p, g in zip(gpu, grads):
            p.grad = g.to(cuda_device)
        opt.step()
        ref.step(grads)
        if step == 0:
            got = [opt.state[p]["automatic_period"] for p in gpu]
            want = [st["automatic_period"] for st in ref.state]
            assert got == want                                  # partition assignments: bit-exact
            assert torch.equal(opt._gefen_codebook.cpu(), ref.codebook)   # histogram + exact DP: bit-exact
    total = agree = 0
    for p, pc, st in zip(gpu, cpu, ref.state):
        diff = (opt.state[p]["m_codebook"].cpu().int() - st["m_codebook"].int()).abs()
        assert int(diff.max()) <= 1
        total += diff.numel()
        agree += int((diff == 0).sum())
        assert rel_l2(p.detach().cpu(), pc) <= 1e-5
    assert agree / total >= 0.9999
    assert opt._optimizer_state_memory_bytes() < 0.14 * 8 * sum(p.numel() for p in gpu)   # ~8x below AdamW's m+v


@pytest.mark.parametrize("log2n", [20, 24])
def test_config3_flat_tensor_against_oracle(oracle, cuda_device, log2n):
    """One flat fp32 tensor, gradient N(0,1) x lognormal(0,1) per 4096-element run: calibration pass
    (period, histogram, codebook) and one fused step, against the oracle."""
    from gefen_b200 import Gefen
    from oracle.ref_loop import OracleGefen

    n = 1 << log2n
    gen = torch.Generator().manual_seed(log2n)
    scale = torch.exp(torch.randn(n // 4096, 1, generator=gen))
    grad = (torch.randn(n // 4096, 4096, generator=gen) * scale).reshape(-1)
    p_cpu = torch.randn(n, generator=gen) * 0.02
    p_gpu = torch.nn.Parameter(p_cpu.clone().to(cuda_device))
    opt = Gefen([p_gpu], lr=1e-3)
    ref = OracleGefen([p_cpu], lr=1e-3)
    p_gpu.grad = grad.to(cuda_device)
    opt.step()
    ref.step([grad])
    assert opt.state[p_gpu]["automatic_period"] == ref.state[0]["automatic_period"] == 2048
    assert torch.equal(opt._gefen_codebook.cpu(), ref.codebook)
    assert torch.equal(opt.state[p_gpu]["m_codebook"].cpu(), ref.state[0]["m_codebook"])
    assert torch.equal(opt.state[p_gpu]["m_magnitude"].cpu(), ref.state[0]["m_magnitude"])
    assert rel_l2(p_gpu.detach().cpu(), p_cpu) <= 1e-6


@pytest.mark.parametrize("log2n", [28, 30])
def test_config3_flat_large_properties(cuda_device, log2n):
    """2^28 and 2^30 elements: too slow for the CPU oracle, so the invariants of one step are checked with torch
    on the GPU: stored magnitude == absmax of beta1*0 + (1-beta1)*g per block (first step), codes
    dequantise to within half a codebook gap of the normalised momentum, parameters move against the
    sign of the gradient."""
    from gefen_b200 import Gefen

    n = 1 << log2n
    gen = torch.Generator(device=cuda_device).manual_seed(log2n)
    scale = torch.exp(torch.randn(n // 4096, 1, generator=gen, device=cuda_device))
    grad = (torch.randn(n // 4096, 4096, generator=gen, device=cuda_device) * scale).reshape(-1)
    p = torch.nn.Parameter(torch.zeros(n, device=cuda_device))
    p.grad = grad
    opt = Gefen([p], lr=1e-3)
    opt.step()
    st = opt.state[p]
    assert st["automatic_period"] == 2048
    m = (1.0 - torch.tensor(0.9, dtype=torch.float32)).item() * grad.view(-1, 2048)
    assert torch.equal(st["m_magnitude"].view(-1), m.abs().amax(dim=1))
    cb = opt._gefen_codebook
    gap = float((cb[1:] - cb[:-1]).max())
    moved = p.detach().view(-1, 2048)
    rows = m.shape[0]
    for r0 in range(0, rows, 1 << 15):          # in slices: the int64 index tensor of 2^30 codes would not fit
        sl = slice(r0, min(rows, r0 + (1 << 15)))
        deq = cb[st["m_codebook"][sl].long()]
        x = m[sl] / st["m_magnitude"][sl]
        assert float((deq - x).abs().max()) <= 0.5 * gap + 1e-6
        big = m[sl].abs() > 0.3 * st["m_magnitude"][sl]
        assert bool((torch.sign(moved[sl][big]) == -torch.sign(m[sl][big])).all())


def test_config2_llama_layer_multi_tensor_equals_per_tensor(cuda_device):
    """bf16, weight decay: one multi-tensor fused launch over a Llama-1.5B layer plus an embedding
    slice must give bit-identical codes and magnitudes to stepping each tensor with the per-tensor
    (reference-shaped) entry points, and parameters within what one bf16 rounding of a block's second moment
    can move them (observed: identical; bound 1e-4 relative L2, against the north-star's 1e-2)."""
    from gefen_b200 import Gefen

    shapes = [("embed", (8192, 2048))] + workloads.llama_1_5b()[1:10]
    params_a = [torch.nn.Parameter(workloads.init_param(n, s, i, torch.bfloat16, cuda_device)) for i, (n, s) in enumerate(shapes)]
    params_b = [torch.nn.Parameter(p.detach().clone()) for p in params_a]
    fused = Gefen(params_a, lr=3e-4, weight_decay=0.1, fused=True)
    per_tensor = Gefen(params_b, lr=3e-4, weight_decay=0.1, fused=False)
    for step in range(3):
        for i, (pa, pb, (_, s)) in enumerate(zip(params_a, params_b, shapes)):
            g = workloads.make_grad(s, i, step, torch.bfloat16, cuda_device)
            pa.grad, pb.grad = g, g.clone()
        fused.step()
        per_tensor.step()
    assert torch.equal(fused._gefen_codebook, per_tensor._gefen_codebook)
    worst = 0.0
    for pa, pb in zip(params_a, params_b):
        sa, sb = fused.state[pa], per_tensor.state[pb]
        assert sa["automatic_period"] == sb["automatic_period"]
        assert torch.equal(sa["m_codebook"], sb["m_codebook"])
        assert torch.equal(sa["m_magnitude"], sb["m_magnitude"])
        err = rel_l2(pa.detach().float().cpu(), pb.detach().float().cpu())
        worst = max(worst, err)
        assert err <= 1e-4, "parameters differ by {:.3e} (relative L2)".format(err)


def test_config4_llama_32b_layer_multi_tensor_equals_per_tensor(cuda_device):
    """One layer of the Llama-32B set (6656-wide projections, 17920-wide MLP: periods 1664 and 1120, not
    powers of two) plus its norms, bf16: the multi-tensor launch against the per-tensor entry points."""
    from gefen_b200 import Gefen

    shapes = workloads.llama_32b()[1:10]
    params_a = [torch.nn.Parameter(workloads.init_param(n, s, i, torch.bfloat16, cuda_device)) for i, (n, s) in enumerate(shapes)]
    params_b = [torch.nn.Parameter(p.detach().clone()) for p in params_a]
    fused = Gefen(params_a, lr=1.5e-4, weight_decay=0.1, fused=True)
    per_tensor = Gefen(params_b, lr=1.5e-4, weight_decay=0.1, fused=False)
    for step in range(2):
        for i, (pa, pb, (_, s)) in enumerate(zip(params_a, params_b, shapes)):
            g = workloads.make_grad(s, i, step, torch.bfloat16, cuda_device)
            pa.grad, pb.grad = g, g.clone()
        fused.step()
        per_tensor.step()
    assert torch.equal(fused._gefen_codebook, per_tensor._gefen_codebook)
    periods = set()
    worst = 0.0
    for pa, pb in zip(params_a, params_b):
        sa, sb = fused.state[pa], per_tensor.state[pb]
        periods.add(sa["automatic_period"])
        assert sa["automatic_period"] == sb["automatic_period"]
        assert torch.equal(sa["m_codebook"], sb["m_codebook"])
        assert torch.equal(sa["m_magnitude"], sb["m_magnitude"])
        err = rel_l2(pa.detach().float().cpu(), pb.detach().float().cpu())
        worst = max(worst, err)
        assert err <= 1e-4, "parameters differ by {:.3e} (relative L2)".format(err)
    assert periods & {1664, 1120, 3328, 2240, 6656, 8960, 17920} or max(periods) > 1024
