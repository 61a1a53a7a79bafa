"""ZeRO-1 on two GPUs of one machine. The step with the all-gather fused into the kernels (peer
stores into the other rank's parameter buffer) must leave every rank with exactly the parameters
that the NCCL all-gather leaves; with the reduce-scatter fused in as well (peer loads of the other
rank's gradients) it must equal a run that is fed the rank-order fp32 mean of the gradients; and the
multicast mode, both collectives on the NVSwitch multicast mapping of the buffers (multimem.ld_reduce /
multimem.st), must agree with that run within the rounding of the switch's sum.
Skipped with fewer than two GPUs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    from gefen_b200.zero1 import Zero1Gefen
    from tests.util import make_grad, make_param

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dev = torch.device("cuda", rank)
    shapes = [(96, 512), (64, 2048), (2048,), (40, 768), (33, 24), (7,), (128, 1024)]

    def grad_of(r, i, s, step):
        return make_grad(s, 5 + r, i, step, torch.bfloat16)

    def averaged(i, s, step):   # what the fused reduce-scatter computes: fp32 sum in rank order, scaled, rounded
        acc = torch.zeros(s, dtype=torch.float32)
        for r in range(world):
            acc += grad_of(r, i, s, step).float()
        return (acc * (1.0 / world)).to(torch.bfloat16)

    results = {}
    # own gradients + NCCL / own gradients + fused all-gather / pre-averaged gradients + fused all-gather /
    # own gradients + both collectives fused
    # ... / both collectives on the switch's multicast (where the machine has it; otherwise the defaults)
    # ... / gradients pushed to their owners by device-to-device copies and summed by the step kernels
    for name, fused_ag, fused_rs, pre_averaged, mc in (("nccl", False, False, False, False), ("fused_ag", True, False, False, False),
                                                       ("averaged_inputs", True, False, True, False),
                                                       ("fused_both", True, True, False, False),
                                                       ("multicast", None, None, False, True),
                                                       ("push", True, None, False, False)):
        params = [torch.nn.Parameter(make_param(s, 5, i, torch.bfloat16).to(dev)) for i, s in enumerate(shapes)]
        named = [("p{}".format(i), p) for i, p in enumerate(params)]
        for i, (p, s) in enumerate(zip(params, shapes)):
            p.grad = torch.zeros(s, dtype=torch.bfloat16, device=dev)
        opt = Zero1Gefen(named, lr=1e-3, weight_decay=0.1, fused_all_gather=fused_ag, fused_reduce_scatter=fused_rs,
                         multicast=mc, push_reduce_scatter=(name == "push"))
        for step in range(4):
            for i, (p, s) in enumerate(zip(params, shapes)):
                g = averaged(i, s, step) if pre_averaged else grad_of(rank, i, s, step)
                p.grad.copy_(g.to(dev))
            opt.step()
        torch.cuda.synchronize()
        results[name] = (opt.all_gather_mode, opt.reduce_scatter_mode, dict(opt.fused_errors),
                         opt.flat_param.detach().cpu().clone())
    torch.save(results, os.path.join(out_dir, "rank{}.pt".format(rank)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_collectives_equal_nccl_collectives(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranks = [torch.load(tmp_path / "rank{}.pt".format(r), weights_only=False) for r in range(world)]
    for r in range(world):
        res = ranks[r]
        assert res["nccl"][:2] == ("nccl all_gather", "nccl reduce_scatter")
        assert res["fused_ag"][:2] == ("peer stores from the step kernels", "nccl reduce_scatter"), res["fused_ag"][2]
        assert res["fused_both"][:2] == ("peer stores from the step kernels", "peer loads in the step kernels"), \
            res["fused_both"][2]
        # the all-gather done by the kernels' peer stores leaves what NCCL's leaves
        assert torch.equal(res["fused_ag"][3], res["nccl"][3])
        # the average done by the kernels' peer loads is the fp32 rank-order mean rounded to bf16
        assert torch.equal(res["fused_both"][3], res["averaged_inputs"][3])
        # and it is close to NCCL's own bf16 average
        assert (res["fused_both"][3].float() - res["nccl"][3].float()).abs().max() < 1e-2
        # pushed copies summed by the kernels: the same rank-order mean
        assert res["push"][1].startswith("device-to-device pushes"), res["push"][2]
        assert torch.equal(res["push"][3], res["averaged_inputs"][3])
        # both collectives on the switch's multicast, where the machine offers it: the switch's sum is rounded
        # its own way (not the fp32 rank-order sum rounded to nearest even, even for two ranks), so this
        # is a tolerance check against the rank-order mean and against NCCL's average
        if res["multicast"][1].startswith("multimem"):
            assert res["multicast"][0] == "multimem.st from the step kernels"
        assert (res["multicast"][3].float() - res["averaged_inputs"][3].float()).abs().max() < 1e-2
        assert (res["multicast"][3].float() - res["nccl"][3].float()).abs().max() < 1e-2
    print("collectives with the defaults:", ranks[0]["multicast"][:3])
    for name in ("nccl", "fused_ag", "fused_both", "multicast", "push"):
        assert torch.equal(ranks[0][name][3], ranks[1][name][3]), name
    assert float(ranks[0]["fused_both"][3].float().abs().sum()) > 0


def _muon_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    from gefen_b200 import GefenMuon
    from gefen_b200.zero1 import Zero1GefenMuon
    from tests.util import make_grad, make_param

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dev = torch.device("cuda", rank)
    shapes = [(256, 512), (512, 256), (384, 384), (128, 1024), (640, 128)]

    def build():
        params = [torch.nn.Parameter(make_param(s, 9, i, torch.bfloat16).to(dev)) for i, s in enumerate(shapes)]
        for p in params:
            p.grad = torch.zeros_like(p)
        return params, [("w{}".format(i), p) for i, p in enumerate(params)]

    sharded_params, named = build()
    sharded = Zero1GefenMuon(named, lr=0.02, weight_decay=0.1)
    single_params, named1 = build()
    single = GefenMuon(named1, lr=0.02, weight_decay=0.1)
    for step in range(3):
        for i, s in enumerate(shapes):   # the same gradient on every rank: its average is itself
            g = make_grad(s, 9, i, step, torch.bfloat16).to(dev)
            sharded_params[i].grad.copy_(g)
            single_params[i].grad.copy_(g)
        sharded.step()
        single.step()
    torch.cuda.synchronize()
    same = all(torch.equal(a.detach(), b.detach()) for a, b in zip(sharded_params, single_params))
    owned = sorted(pc.tensor for pc in sharded.pieces)
    torch.save({"same": same, "owned": owned}, os.path.join(out_dir, "muon_rank{}.pt".format(rank)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_muon_equals_single_process(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_muon_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranks = [torch.load(tmp_path / "muon_rank{}.pt".format(r), weights_only=False) for r in range(world)]
    assert all(r["same"] for r in ranks)
    assert sorted(ranks[0]["owned"] + ranks[1]["owned"]) == list(range(5))
    assert ranks[0]["owned"] and ranks[1]["owned"]
