"""End-to-end: the `Gefen` optimizer on the GPU against the oracle's restatement of the reference
loop, on a small transformer-shaped parameter set with the benchmark's gradient distribution."""
import copy

import pytest
import torch

from tests.util import make_grad, make_param, rel_l2

pytestmark = pytest.mark.gpu

SHAPES = [(96, 64), (64,), (64, 192), (192,), (64, 256), (256, 64), (64,), (1,), (40, 36)]


def _setup(dtype, device):
    params_cpu = [make_param(s, 0, i, dtype) if len(s) == 2 else torch.ones(s, dtype=dtype) for i, s in enumerate(SHAPES)]
    params_gpu = [torch.nn.Parameter(p.clone().to(device)) for p in params_cpu]
    return params_cpu, params_gpu


def _grads(step, dtype):
    return [make_grad(s, 0, i, step, dtype) for i, s in enumerate(SHAPES)]


@pytest.mark.parametrize("dtype,wd,fused", [(torch.float32, 0.0, True), (torch.float32, 0.0, False),
                                            (torch.bfloat16, 0.1, True), (torch.bfloat16, 0.1, False),
                                            (torch.float16, 0.01, True)])
def test_ten_steps_match_oracle(oracle, cuda_device, dtype, wd, fused):
    from gefen_b200 import Gefen
    from oracle.ref_loop import OracleGefen

    params_cpu, params_gpu = _setup(dtype, cuda_device)
    ref = OracleGefen(params_cpu, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd)
    opt = Gefen([("p{}".format(i), p) for i, p in enumerate(params_gpu)], lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                weight_decay=wd, fused=fused)
    for step in range(10):
        grads = _grads(step, dtype)
        for p, g in zip(params_gpu, grads):
            p.grad = g.to(cuda_device)
        opt.step()
        ref.step(grads)
        if step == 0:
            # calibration: partition assignments and the codebook are bit-exact
            for p, st in zip(params_gpu, ref.state):
                assert opt.state[p]["automatic_period"] == st["automatic_period"]
            assert torch.equal(opt._gefen_codebook.cpu(), ref.codebook)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for p, pc, st in zip(params_gpu, params_cpu, ref.state):
        codes = opt.state[p]["m_codebook"].cpu().int()
        diff = (codes - st["m_codebook"].int()).abs()
        assert float((diff == 0).float().mean()) >= 0.9999 and int(diff.max()) <= 1
        assert rel_l2(p.detach().cpu(), pc) <= tol
        assert rel_l2(opt.state[p]["vmean"].cpu().float(), st["vmean"].float()) <= (1e-5 if dtype == torch.float32 else 1e-2)
        assert opt.state[p]["m_magnitude"].dtype == st["m_magnitude"].dtype
        assert opt.state[p]["step"] == 10


def test_state_dict_round_trip(cuda_device):
    from gefen_b200 import Gefen

    dtype = torch.bfloat16
    _, params = _setup(dtype, cuda_device)
    opt = Gefen(params, lr=1e-3, weight_decay=0.1)
    for step in range(2):
        for p, g in zip(params, _grads(step, dtype)):
            p.grad = g.to(cuda_device)
        opt.step()
    sd = copy.deepcopy(opt.state_dict())
    assert sd["gefen_global_step"] == 2 and sd["gefen_codebook"].numel() == 256
    keys = set(sd["state"][0].keys())
    assert {"automatic_period", "step", "m_codebook_shape", "m_codebook", "m_magnitude", "vmean"} <= keys

    params2 = [torch.nn.Parameter(p.detach().clone()) for p in params]
    opt2 = Gefen(params2, lr=1e-3, weight_decay=0.1)
    opt2.load_state_dict(sd)
    assert opt2.state[params2[0]]["m_codebook"].dtype == torch.uint8  # torch's cast was undone
    assert opt2.state[params2[0]]["vmean"].dtype == dtype
    grads = _grads(2, dtype)
    for p, p2, g in zip(params, params2, grads):
        p.grad = g.to(cuda_device)
        p2.grad = g.to(cuda_device)
    opt.step()
    opt2.step()
    for p, p2 in zip(params, params2):
        assert torch.equal(p.detach(), p2.detach())
        assert torch.equal(opt.state[p]["m_codebook"], opt2.state[p2]["m_codebook"])


def test_codebook_relearned_from_restored_periods(cuda_device):
    from gefen_b200 import Gefen

    _, params = _setup(torch.float32, cuda_device)
    opt = Gefen(params, lr=1e-3)
    for p, g in zip(params, _grads(0, torch.float32)):
        p.grad = g.to(cuda_device)
    opt.step()
    sd = copy.deepcopy(opt.state_dict())
    sd["gefen_codebook"] = None
    opt2 = Gefen([torch.nn.Parameter(p.detach().clone()) for p in params], lr=1e-3)
    opt2.load_state_dict(sd)
    for p, g in zip(opt2.param_groups, _grads(0, torch.float32)):
        p["params"][0].grad = g.to(cuda_device)
    opt2.step()
    assert torch.equal(opt2._gefen_codebook, opt._gefen_codebook)


def test_missing_library_is_loud(monkeypatch, cuda_device, tmp_path):
    from gefen_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_lib.GefenB200Error):
        _lib.load()


def test_loads_a_checkpoint_written_by_the_reference(cuda_device):
    """A state_dict produced by the reference optimizer (CPU, three steps; tests/golden) is loaded as
    is; two more steps here must land where the reference itself lands (its CPU arithmetic differs
    from its kernels' by rounding only)."""
    from pathlib import Path

    from gefen_b200 import Gefen

    golden = torch.load(Path(__file__).resolve().parent / "golden" / "reference_golden.pt", weights_only=False)
    ck = golden["checkpoint"]
    shapes = golden["ten_steps_fp32"]["shapes"]
    params = [torch.nn.Parameter(p.clone().to(cuda_device)) for p in ck["params"]]
    opt = Gefen([("p{}".format(i), p) for i, p in enumerate(params)], lr=1e-3, weight_decay=0.01)
    opt.load_state_dict(ck["state_dict"])
    assert opt._gefen_global_step == 3
    st = opt.state[params[0]]
    assert st["m_codebook"].dtype == torch.uint8 and st["m_codebook"].device.type == "cuda"
    assert st["step"] == 3 and isinstance(st["automatic_period"], int)
    for step in range(3, 5):
        for i, (p, s) in enumerate(zip(params, shapes)):
            p.grad = make_grad(s, 0, i, step).to(cuda_device)
        opt.step()
    total = agree = 0
    for p, want, codes in zip(params, ck["params_after_two_more"], ck["codes_after_two_more"]):
        assert rel_l2(p.detach().cpu(), want) <= 2e-5
        diff = (opt.state[p]["m_codebook"].cpu().int() - codes.int()).abs()
        assert int(diff.max()) <= 1
        total += diff.numel()
        agree += int((diff == 0).sum())
    assert agree / total >= 0.999
    # and back: the reference's loader only needs the same keys
    sd = opt.state_dict()
    assert set(sd["state"][0]) == set(ck["state_dict"]["state"][0])


def test_host_streamed_step_equals_plain_step(cuda_device):
    """Gradients from pinned host memory, parameters back to pinned host memory, bucket by bucket on
    three streams: same results as copying everything, stepping, copying everything back."""
    from gefen_b200 import Gefen, HostStreamedGefen

    # (the 600 x 2048 tensor is larger than a bucket: it is cut between blocks and spread over several)
    shapes = [(64, 512), (2048,), (96, 768), (600, 2048), (33, 24), (128, 1024), (7,), (256, 256)]

    def build():
        params = [torch.nn.Parameter(make_param(s, 3, i, torch.bfloat16).to(cuda_device)) for i, s in enumerate(shapes)]
        for p in params:
            p.grad = torch.zeros_like(p)
        return params, Gefen([("p{}".format(i), p) for i, p in enumerate(params)], lr=1e-3, weight_decay=0.1)

    plain_params, plain = build()
    stream_params, streamed_opt = build()
    host_g = [torch.empty(s, dtype=torch.bfloat16).pin_memory() for s in shapes]
    host_p = [torch.empty(s, dtype=torch.bfloat16).pin_memory() for s in shapes]
    streamed = HostStreamedGefen(streamed_opt, host_g, host_p, buckets=4)
    for step in range(4):
        grads = [make_grad(s, 3, i, step, torch.bfloat16) for i, s in enumerate(shapes)]
        for p, g, h in zip(plain_params, grads, host_g):
            p.grad.copy_(g.to(cuda_device))
            h.copy_(g)
        plain.step()
        streamed.step()
        torch.cuda.synchronize()
        for p, q, h in zip(plain_params, stream_params, host_p):
            assert torch.equal(p.detach(), q.detach())
            assert torch.equal(h, p.detach().cpu())
    for p, q in zip(plain_params, stream_params):
        assert torch.equal(plain.state[p]["m_codebook"], streamed_opt.state[q]["m_codebook"])
        assert torch.equal(plain.state[p]["vmean"], streamed_opt.state[q]["vmean"])
        assert plain.state[p]["step"] == streamed_opt.state[q]["step"] == 4
    assert plain._gefen_global_step == streamed_opt._gefen_global_step == 4
    # the buckets cover every block of every tensor exactly once, and the large tensor is cut
    assert len(streamed.buckets) == 4
    covered = {}
    for bucket in streamed.buckets:
        for i, b0, b1, whole in bucket:
            covered.setdefault(i, []).append((b0, b1))
    assert sorted(covered) == list(range(len(shapes)))
    for i, runs in covered.items():
        runs.sort()
        assert runs[0][0] == 0 and all(a[1] == b[0] for a, b in zip(runs, runs[1:]))
    assert len(covered[3]) >= 2


class _ShardedParam(torch.nn.Parameter):
    """Stands in for a DTensor parameter: the optimizer must go through to_local() (and may get a
    non-contiguous local shard, which only objects with `placements` are allowed to hand over)."""
    placements = ("Shard(0)",)

    def to_local(self):
        return self._local_view


class _AsyncGrad(torch.Tensor):
    """Stands in for a gradient that is still the handle of an asynchronous collective."""

    def wait(self):
        return self.as_subclass(torch.Tensor)


def test_dtensor_like_parameters_and_async_gradients(cuda_device):
    """reference: gefen.py:692-706, 1287-1322. Duck-typed unwrapping of DTensor-like parameters
    (to_local, non-contiguous local shard copied in and out) and of gradients with wait()."""
    from gefen_b200 import Gefen

    shape = (48, 512)
    base = make_param(shape, 4, 0, torch.bfloat16).to(cuda_device)
    plain = torch.nn.Parameter(base.clone())
    # the "local shard" is a transposed view of a [512, 48] buffer: same values, not contiguous
    storage = base.clone().t().contiguous()
    sharded = _ShardedParam(torch.zeros(shape, device=cuda_device, dtype=torch.bfloat16))   # its own data is never used
    sharded._local_view = storage.t()
    assert not sharded._local_view.is_contiguous()
    opt_plain = Gefen([("w", plain)], lr=1e-3, weight_decay=0.1)
    opt_sharded = Gefen([("w", sharded)], lr=1e-3, weight_decay=0.1)
    for step in range(3):
        g = make_grad(shape, 4, 0, step, torch.bfloat16).to(cuda_device)
        plain.grad = g.clone()
        sharded.grad = g.clone().as_subclass(_AsyncGrad)
        opt_plain.step()
        opt_sharded.step()
    torch.cuda.synchronize()
    assert torch.equal(sharded.to_local(), plain.detach())
    assert torch.equal(opt_sharded.state[sharded]["m_codebook"], opt_plain.state[plain]["m_codebook"])


def test_steady_state_path_equals_the_general_path(cuda_device):
    """A training loop whose tensors stay at the same addresses takes `Gefen._step_steady` (only the step
    counters and the scalars derived from them are refreshed). Same results as the general path, also across the
    events that must send a call back to it: a learning-rate change (stays steady, new scalars), gradients in
    new tensors, a gradient that disappears and comes back, a parameter that joins late."""
    from gefen_b200 import Gefen

    dtype = torch.bfloat16

    def build():
        _, params = _setup(dtype, cuda_device)
        for p in params:
            p.grad = torch.zeros_like(p)
        return params, Gefen([("p{}".format(i), p) for i, p in enumerate(params)], lr=1e-3, weight_decay=0.1)

    fast_params, fast = build()
    slow_params, slow = build()
    took_steady = 0
    for step in range(12):
        grads = [g.to(cuda_device) for g in _grads(step, dtype)]
        for k, (params, opt) in enumerate(((fast_params, fast), (slow_params, slow))):
            for i, (p, g) in enumerate(zip(params, grads)):
                if step in (5, 6) and i == 2:
                    p.grad = None                      # a tensor without a gradient for two steps
                elif step in (3, 8) or p.grad is None or (step < 2 and i == 4):
                    p.grad = g.clone()                 # gradients in new tensors
                else:
                    p.grad.copy_(g)                    # the steady state: same tensors, new values
            if step < 2:
                params[4].grad = None                  # a parameter that joins at step 2
            if step == 7:
                for group in opt.param_groups:
                    group["lr"] = 5e-4
            if k == 1:
                opt._steady = None                     # the general path, every step
            else:
                before = opt._steady
            opt.step()
            if k == 0 and before is not None and opt._steady is before:
                took_steady += 1
        torch.cuda.synchronize()
        for p, q in zip(fast_params, slow_params):
            assert torch.equal(p.detach(), q.detach()), step
    assert took_steady >= 4        # (the steady path did run: it leaves its cache object in place)
    for p, q in zip(fast_params, slow_params):
        a, b = fast.state[p], slow.state[q]
        assert a["step"] == b["step"]
        for key in ("m_codebook", "m_magnitude", "vmean"):
            assert torch.equal(a[key], b[key])
