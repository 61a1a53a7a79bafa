"""CPU, gloo, world size 2: the ZeRO-1 host logic (flat layout, reduce-scatter / all-gather plumbing,
period agreement, global histogram merge) with the device work replaced by the CPU oracle. Two ranks
must reproduce a single process bit for bit."""
import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
SHAPES = [(96, 64), (64,), (64, 192), (192,), (300, 256), (256, 64), (1,), (40, 36)]


class OracleOps:
    """The calibration and step of gefen_b200.zero1 on the CPU oracle (test double for GpuOps)."""

    def predict_periods(self, grads):
        from oracle import oracle as O

        return [1 if g.numel() == 1 else O.find_period(g, cuda_kernel_semantics=True) for g in grads]

    def histograms(self, flats_and_periods, bins):
        from oracle import oracle as O

        rows = torch.zeros((len(flats_and_periods), bins), dtype=torch.int64)
        for row, (flat, period) in zip(rows, flats_and_periods):
            O.gefen_exact_histogram(flat.contiguous(), period, row)
        return rows

    def fit_codebook(self, bin_counts, num_codebooks, device):
        from oracle import oracle as O

        centers, counts = O.histogram_stats(bin_counts)
        return O.exact_dp(centers, counts, num_codebooks, True)

    def make_optimizer(self, named_pieces, lr, betas, eps, weight_decay):
        from oracle.ref_loop import OracleGefen

        class Adapter:
            def __init__(self):
                self.params = [p for _, p in named_pieces]
                self.inner = OracleGefen([p.data for p in self.params], lr=lr, betas=betas, eps=eps,
                                         weight_decay=weight_decay)
                self.state = {p: st for p, st in zip(self.params, self.inner.state)}

            @property
            def _gefen_codebook(self):
                return self.inner.codebook

            @_gefen_codebook.setter
            def _gefen_codebook(self, value):
                self.inner.codebook = value

            def step(self):
                self.inner.step([p.grad for p in self.params])

        return Adapter()


def _grads(step, rank, world):
    from tests.util import make_grad

    # every rank sees different gradients; their average is what one process would see
    return [make_grad(s, 10 + rank, i, step) for i, s in enumerate(SHAPES)]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gefen_b200.zero1 import Zero1Gefen
    from tests.util import make_param

    params = [torch.nn.Parameter(make_param(s, 0, i) if len(s) == 2 else torch.ones(s)) for i, s in enumerate(SHAPES)]
    named = [("p{}".format(i), p) for i, p in enumerate(params)]
    opt = Zero1Gefen(named, lr=1e-3, weight_decay=0.1, ops=OracleOps())
    for step in range(4):
        for p, g in zip(params, _grads(step, rank, world)):
            p.grad.copy_(g)
        opt.step()
    torch.save({"params": [p.detach().clone() for p in params], "periods": opt.periods, "codebook": opt.codebook,
                "mismatches": opt.period_mismatches,
                "pieces": [(pc.tensor, pc.row0, pc.rows) for pc in opt.pieces]}, os.path.join(out_dir, "rank{}.pt".format(rank)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_one_process(tmp_path, oracle):
    from oracle.ref_loop import OracleGefen
    from tests.util import make_param

    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(tmp_path / "rank{}.pt".format(r), weights_only=False) for r in range(world)]

    # single process on the averaged gradients
    params = [make_param(s, 0, i) if len(s) == 2 else torch.ones(s) for i, s in enumerate(SHAPES)]
    ref = OracleGefen(params, lr=1e-3, weight_decay=0.1)
    for step in range(4):
        per_rank = [_grads(step, r, world) for r in range(world)]
        grads = [(a + b) / world for a, b in zip(*per_rank)]
        ref.step(grads)
    for out in outs:
        assert out["mismatches"] == []
        assert [out["periods"][t] for t in range(len(SHAPES))] == [st["automatic_period"] for st in ref.state]
        assert torch.equal(out["codebook"], ref.codebook)
        for p, q in zip(out["params"], params):
            assert torch.equal(p, q)
    # both ranks own something, and at least one tensor is split between them
    owned = [set(t for t, _, _ in out["pieces"]) for out in outs]
    assert owned[0] and owned[1] and (owned[0] & owned[1])


def _reshard_worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gefen_b200.zero1 import Zero1Gefen
    from tests.util import make_param

    params = [torch.nn.Parameter(make_param(s, 0, i) if len(s) == 2 else torch.ones(s)) for i, s in enumerate(SHAPES)]
    opt = Zero1Gefen([("p{}".format(i), p) for i, p in enumerate(params)], lr=1e-3, weight_decay=0.1, ops=OracleOps())
    for step in range(3):
        for p, g in zip(params, _grads(step, rank, world)):
            p.grad.copy_(g)
        opt.step()
    full = opt.full_state_dict()
    params_at_three = [p.detach().clone() for p in params]
    for step in range(3, 5):
        for p, g in zip(params, _grads(step, rank, world)):
            p.grad.copy_(g)
        opt.step()
    torch.save({"full": full, "params_at_three": params_at_three, "params_at_five": [p.detach().clone() for p in params]},
               os.path.join(out_dir, "reshard{}.pt".format(rank)))
    dist.barrier()
    dist.destroy_process_group()


def test_full_state_moves_between_world_sizes(tmp_path, oracle):
    """State saved by two ranks (whole-model layout, identical on both) is loaded by a single process,
    which then reaches the same parameters as the two ranks did; and loading it back into the pieces of
    the single process reproduces the pieces' state."""
    from gefen_b200.zero1 import Zero1Gefen

    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_reshard_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(tmp_path / "reshard{}.pt".format(r), weights_only=False) for r in range(world)]
    full = outs[0]["full"]
    other = outs[1]["full"]
    assert full["periods"] == other["periods"] and torch.equal(full["gefen_codebook"], other["gefen_codebook"])
    assert sorted(full["state"]) == list(range(len(SHAPES)))
    for t in full["state"]:
        for k, v in full["state"][t].items():
            if torch.is_tensor(v):
                assert torch.equal(v, other["state"][t][k])
        n = 1
        for d in SHAPES[t]:
            n *= d
        assert full["state"][t]["m_codebook"].numel() == n and full["state"][t]["step"] == 3
    # one process (no process group) continues from the two ranks' checkpoint
    params = [torch.nn.Parameter(p.clone()) for p in outs[0]["params_at_three"]]
    single = Zero1Gefen([("p{}".format(i), p) for i, p in enumerate(params)], lr=1e-3, weight_decay=0.1, ops=OracleOps())
    single.load_full_state_dict(full)
    for step in range(3, 5):
        per_rank = [_grads(step, r, world) for r in range(world)]
        for p, a, b in zip(params, *per_rank):
            p.grad.copy_((a + b) / world)
        single.step()
    for p, want in zip(params, outs[0]["params_at_five"]):
        assert torch.equal(p.detach(), want)
    again = single.full_state_dict()
    assert again["gefen_global_step"] == 5
