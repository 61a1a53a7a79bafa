"""GPU: real `torch.distributed.tensor.DTensor` parameters and gradients (what FSDP2 hands an optimizer)
through `Gefen` and `GefenMuon`, on a one-rank process group with a one-device mesh, against the same run
on plain tensors. Reference behaviour: the optimizer works on `to_local()` shards (gefen.py:692-706), a
non-contiguous local shard is stepped on a contiguous copy and copied back (gefen.py:1287-1322), and the
parameter object stays the DTensor it was. Also: a flat (1-D) partition of a 2-D parameter, as ZeRO-style
callers hand it over, gives the 2-D result."""
import socket

import pytest
import torch

from tests.util import make_grad, make_param

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mesh(cuda_device):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    if dist.is_initialized():
        pytest.skip("a process group already exists in this process")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    torch.cuda.set_device(cuda_device)
    dist.init_process_group("cpu:gloo,cuda:nccl", init_method="tcp://127.0.0.1:{}".format(port), rank=0, world_size=1,
                            device_id=cuda_device)
    try:
        yield init_device_mesh("cuda", (1,))
    finally:
        dist.destroy_process_group()


def _dtensor(local, mesh):
    from torch.distributed.tensor import DTensor, Shard

    return DTensor.from_local(local, mesh, [Shard(0)], run_check=False)


@pytest.mark.parametrize("contiguous", [True, False])
def test_gefen_on_real_dtensors(cuda_device, mesh, contiguous):
    from torch.distributed.tensor import DTensor, Shard

    from gefen_b200 import Gefen

    shapes = [(48, 512), (64, 2048), (512,)]
    plain, sharded = [], []
    for i, s in enumerate(shapes):
        base = make_param(s, 6, i, torch.bfloat16).to(cuda_device)
        plain.append(torch.nn.Parameter(base.clone()))
        if contiguous or len(s) == 1:
            local = base.clone()
        else:   # a transposed view of a [cols, rows] buffer: same values, not contiguous
            local = base.clone().t().contiguous().t()
            assert not local.is_contiguous()
        sharded.append(torch.nn.Parameter(_dtensor(local, mesh)))
    opt_plain = Gefen(plain, lr=1e-3, weight_decay=0.1)
    opt_dt = Gefen(sharded, lr=1e-3, weight_decay=0.1)
    for step in range(3):
        for i, s in enumerate(shapes):
            g = make_grad(s, 6, i, step, torch.bfloat16).to(cuda_device)
            plain[i].grad = g.clone()
            sharded[i].grad = _dtensor(g.clone(), mesh)
        opt_plain.step()
        opt_dt.step()
    torch.cuda.synchronize()
    for a, b in zip(plain, sharded):
        assert isinstance(b.data, DTensor) and b.placements == (Shard(0),)    # still the caller's DTensor
        assert torch.equal(b.to_local(), a.detach())
        sa, sb = opt_plain.state[a], opt_dt.state[b]
        assert sa["automatic_period"] == sb["automatic_period"]
        for key in ("m_codebook", "m_magnitude", "vmean"):
            assert torch.equal(sa[key], sb[key])
    # checkpoints carry plain tensors, as the reference's do
    sd = opt_dt.state_dict()
    assert all(not isinstance(v, DTensor) for st in sd["state"].values() for v in st.values() if torch.is_tensor(v))


def test_gefen_muon_on_real_dtensors(cuda_device, mesh):
    from gefen_b200 import GefenMuon

    shapes = [(256, 512), (512, 256)]
    plain = [torch.nn.Parameter(make_param(s, 7, i, torch.bfloat16).to(cuda_device)) for i, s in enumerate(shapes)]
    sharded = [torch.nn.Parameter(_dtensor(p.detach().clone(), mesh)) for p in plain]
    opt_plain = GefenMuon(plain, lr=0.02, weight_decay=0.1)
    opt_dt = GefenMuon(sharded, lr=0.02, weight_decay=0.1)
    for step in range(3):
        for i, s in enumerate(shapes):
            g = make_grad(s, 7, i, step, torch.bfloat16).to(cuda_device)
            plain[i].grad = g.clone()
            sharded[i].grad = _dtensor(g.clone(), mesh)
        opt_plain.step()
        opt_dt.step()
    opt_dt.check()
    for a, b in zip(plain, sharded):
        assert torch.equal(b.to_local(), a.detach())
        assert torch.equal(opt_plain.state[a]["m_codebook"], opt_dt.state[b]["m_codebook"])


def test_flat_partition_of_a_matrix_gives_the_matrix_result(cuda_device):
    """ZeRO-style callers hand the optimizer a 1-D partition of a parameter. The period search and the blocks
    work on the flattened tensor in any case (reference: partitioning.py:147, gefen.py:1270-1275), so the
    flat form of a matrix must reproduce the matrix form bit for bit."""
    from gefen_b200 import Gefen

    shape = (96, 1024)
    base = make_param(shape, 8, 0, torch.float32).to(cuda_device)
    matrix = torch.nn.Parameter(base.clone())
    flat = torch.nn.Parameter(base.clone().reshape(-1))
    opt_m, opt_f = Gefen([matrix], lr=1e-3, weight_decay=0.01), Gefen([flat], lr=1e-3, weight_decay=0.01)
    for step in range(3):
        g = make_grad(shape, 8, 0, step, torch.float32).to(cuda_device)
        matrix.grad, flat.grad = g.clone(), g.clone().reshape(-1)
        opt_m.step()
        opt_f.step()
    assert opt_m.state[matrix]["automatic_period"] == opt_f.state[flat]["automatic_period"] == 1024
    assert torch.equal(matrix.detach().reshape(-1), flat.detach())
    assert torch.equal(opt_m.state[matrix]["m_codebook"], opt_f.state[flat]["m_codebook"])
