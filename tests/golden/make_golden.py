"""Generates tests/golden/reference_golden.pt by RUNNING the reference (its PyTorch CPU path, its
numba exact-DP and its numpy period search) on small seeded inputs. The reference ships no tests or
golden vectors of its own, so these outputs are what pins the oracle.

    python tests/golden/make_golden.py /path/to/reference

The reference package maps the package name `gefen` to its repository root, so it is imported
through a temporary directory holding a symlink of that name.
"""
import os
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from tests.util import make_grad, make_param  # noqa: E402

SHAPES = [(96, 64), (64,), (64, 192), (192,), (64, 256), (256, 64), (1,), (40, 36)]
PERIOD_SHAPES = [(768, 768), (64, 2304), (2048, 512), (1000,), (37, 12), (96, 1536), (7,), (3,), (50, 40)]


def main(reference_root: str) -> None:
    tmp = tempfile.mkdtemp()
    os.symlink(reference_root, os.path.join(tmp, "gefen"))
    sys.path.insert(0, tmp)
    import gefen.gefen as rg
    import gefen.partitioning as rp
    import gefen.quantization as rq
    from gefen import Gefen

    out = {}
    # 1. nearest-entry rule
    torch.manual_seed(0)
    cb = torch.sort(torch.cat([torch.tensor([-1.0, 1.0]), torch.tanh(torch.randn(254) * 0.6)])).values.float()
    x = torch.cat([torch.rand(20000) * 2 - 1, cb, 0.5 * (cb[1:] + cb[:-1])])
    out["nearest"] = {"codebook": cb, "x": x, "index": rg.gefen_nearest_codebook_indices(cb, x)}

    # 2. exact DP on histograms of several densities and sizes
    dps = []
    for k, force, active, seed in [(256, True, 4096, 1), (256, True, 600, 2), (16, True, 300, 3), (32, False, 900, 4),
                                   (256, True, 90, 5)]:
        gen = torch.Generator().manual_seed(seed)
        bins = 4096
        counts = torch.zeros(bins)
        idx = torch.randperm(bins, generator=gen)[:active]
        counts[idx] = torch.floor(torch.exp(-((idx.float() - 2048) / 500.0) ** 2) * 1e5 * torch.rand(active, generator=gen)) + 1
        edges = torch.linspace(-1, 1, bins + 1)
        centers = 0.5 * (edges[:-1] + edges[1:])
        m = counts > 0
        cbk = rq.exact_dp({"active_centers": centers[m], "active_counts": counts[m]}, k, force)
        dps.append({"k": k, "force": force, "counts": counts, "codebook": cbk})
    out["exact_dp"] = dps

    # 3. period decisions of the CPU backend (squares in fp32, as gefen.py:813 does)
    periods = []
    for i, shape in enumerate(PERIOD_SHAPES):
        for dtype in (torch.float32, torch.bfloat16):
            g = make_grad(shape, 7, i, 0, dtype)
            if g.numel() == 1:
                continue
            sq = g.detach().float().square().reshape(-1).cpu().numpy()
            period = rp.find_period_by_block_variance(sq, print_results=False, backend="cpu", input_is_squared=True)
            periods.append({"shape": shape, "dtype": str(dtype), "seed": 7, "index": i, "period": int(period)})
    out["periods"] = periods

    # 4. ten steps of the reference optimizer on CPU (fused=False is forced there), fp32
    params = [torch.nn.Parameter(make_param(s, 0, i) if len(s) == 2 else torch.ones(s)) for i, s in enumerate(SHAPES)]
    opt = Gefen([("p{}".format(i), p) for i, p in enumerate(params)], lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                weight_decay=0.0, fused=False)
    for step in range(10):
        for i, (p, s) in enumerate(zip(params, SHAPES)):
            p.grad = make_grad(s, 0, i, step)
        opt.step()
    out["ten_steps_fp32"] = {
        "shapes": SHAPES,
        "params": [p.detach().clone() for p in params],
        "periods": [opt.state[p]["automatic_period"] for p in params],
        "codes": [opt.state[p]["m_codebook"].clone() for p in params],
        "magnitude": [opt.state[p]["m_magnitude"].clone() for p in params],
        "vmean": [opt.state[p]["vmean"].clone() for p in params],
        "codebook": opt._gefen_codebook.clone(),
    }
    # 5. checkpoint interchange: the reference's state_dict after three steps, and where the reference
    #    itself gets to after two more steps from that checkpoint
    import copy

    params = [torch.nn.Parameter(make_param(s, 0, i) if len(s) == 2 else torch.ones(s)) for i, s in enumerate(SHAPES)]
    opt = Gefen([("p{}".format(i), p) for i, p in enumerate(params)], lr=1e-3, weight_decay=0.01, fused=False)
    for step in range(3):
        for i, (p, s) in enumerate(zip(params, SHAPES)):
            p.grad = make_grad(s, 0, i, step)
        opt.step()
    checkpoint = {"state_dict": copy.deepcopy(opt.state_dict()), "params": [p.detach().clone() for p in params]}
    for step in range(3, 5):
        for i, (p, s) in enumerate(zip(params, SHAPES)):
            p.grad = make_grad(s, 0, i, step)
        opt.step()
    checkpoint["params_after_two_more"] = [p.detach().clone() for p in params]
    checkpoint["codes_after_two_more"] = [opt.state[p]["m_codebook"].clone() for p in params]
    out["checkpoint"] = checkpoint
    torch.save(out, HERE / "reference_golden.pt")
    print("wrote", HERE / "reference_golden.pt")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/the/reference/checkout")
    main(sys.argv[1])
