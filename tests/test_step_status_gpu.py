"""GPU: the step kernels' error status. Every wait inside the kernels is bounded; when the wait for
the staged codebook tables runs out, a CTA returns without doing its share of the step and raises a
status word that the host reads. The test makes the wait run out by granting it zero polls (a test
hook of the C ABI): nothing faults, traps or hangs, the kernels simply return."""
import pytest
import torch

from tests.util import make_grad, make_param, reference_like_codebook

pytestmark = pytest.mark.gpu


@pytest.fixture
def zero_polls():
    from gefen_b200 import _lib

    lib = _lib.load()
    _lib.check(lib.gefen_b200_debug_set_stage_spin_limit(0))
    yield lib
    _lib.check(lib.gefen_b200_debug_set_stage_spin_limit(-1))


@pytest.mark.parametrize("nb,period", [(64, 2048), (40, 128), (30, 24)])   # staged kernel (long and short blocks), generic kernel
def test_timed_out_staging_is_reported_and_nothing_is_half_done(cuda_device, zero_polls, nb, period):
    from gefen_b200 import _lib
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    assert _lib.step_status(cuda_device) == 0
    cb = reference_like_codebook().to(cuda_device)
    dtype = torch.bfloat16
    p = make_param((nb, period), 1, 0, dtype).to(cuda_device)
    g = make_grad((nb, period), 1, 0, 0, dtype).to(cuda_device)
    codes = torch.randint(0, 256, (nb, period), dtype=torch.uint8, device=cuda_device)
    mag = (torch.rand(nb, 1, device=cuda_device) * 2e-3).to(dtype)
    v = (torch.rand(nb, 1, device=cuda_device) * 1e-6 + 1e-9).to(dtype)
    before = [t.clone() for t in (p, codes, mag)]
    automatic_gefen_fused_update_from_vmean_cuda(p, g, codes, mag, v, cb, False, 0.9, 3e-4, 0.1, 0.001, 1e-8)
    torch.cuda.synchronize()     # the kernel came back by itself
    for was, now in zip(before, (p, codes, mag)):
        assert torch.equal(was, now)
    assert _lib.step_status(cuda_device, clear=False) != 0
    with pytest.raises(_lib.GefenB200Error, match="gave up waiting"):
        _lib.check_step_status(cuda_device)
    assert _lib.step_status(cuda_device) == 0          # reading cleared it

    # with the default limit the same call works and leaves the status clear
    _lib.check(zero_polls.gefen_b200_debug_set_stage_spin_limit(-1))
    automatic_gefen_fused_update_from_vmean_cuda(p, g, codes, mag, v, cb, False, 0.9, 3e-4, 0.1, 0.001, 1e-8)
    assert _lib.step_status(cuda_device) == 0
    assert not torch.equal(before[1], codes)


def test_optimizer_check_raises_after_a_timed_out_step(cuda_device, zero_polls):
    from gefen_b200 import Gefen, _lib

    params = [torch.nn.Parameter(make_param((32, 512), 2, i, torch.float32).to(cuda_device)) for i in range(2)]
    opt = Gefen(params, lr=1e-3)
    _lib.check(zero_polls.gefen_b200_debug_set_stage_spin_limit(-1))
    for p in params:
        p.grad = make_grad((32, 512), 2, 0, 0, torch.float32).to(cuda_device)
    opt.step()                    # calibrates and steps normally
    opt.check()
    _lib.check(zero_polls.gefen_b200_debug_set_stage_spin_limit(0))
    opt.step()
    with pytest.raises(_lib.GefenB200Error):
        opt.check()
    _lib.check(zero_polls.gefen_b200_debug_set_stage_spin_limit(-1))
    opt.step()
    opt.check()
    opt.state_dict()
