"""CPU: host-side logic of the package and the C-ABI surface (no compute calls)."""
import re
import subprocess
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    from gefen_b200 import _lib

    _lib.load()
    header = (ROOT / "include" / "gefen_b200.h").read_text()
    declared = set(re.findall(r"\b(gefen_b200_[a-z0-9_]+)\s*\(", header))
    declared.discard("gefen_b200_step_tensor")
    assert len(declared) >= 20
    nm = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True, check=True)
    exported = set(re.findall(r"\b(gefen_b200_[a-z0-9_]+)\b", nm.stdout))
    assert declared <= exported, sorted(declared - exported)
    assert declared == set(_lib.EXPORTED_SYMBOLS), sorted(declared ^ set(_lib.EXPORTED_SYMBOLS))


def test_argument_errors_without_a_gpu():
    from gefen_b200 import _lib

    lib = _lib.load()
    assert lib.gefen_b200_version() >= 1
    with pytest.raises(ValueError):
        _lib.check(lib.gefen_b200_exact_histogram(None, 0, 16, 3, None, 4096, None))       # null bin_counts
    with pytest.raises(ValueError):
        _lib.check(lib.gefen_b200_codebook_prepare(None, 256, None, None))
    assert lib.gefen_b200_period_scratch_doubles(1024, 8) == 128 + 1 + 1024
    assert lib.gefen_b200_exact_dp_scratch_bytes(4096, 256) == 2 * 4097 * 8 + 257 * 4097 * 4 + 16


def test_divisors_and_candidates(oracle):
    from gefen_b200 import partitioning as P

    for n in [1, 2, 7, 12, 64, 768, 1000, 2048 * 512, 50257 * 768, 128256 * 2048]:
        assert P.divisors(n) == oracle.divisors(n)
        assert P.candidate_periods(n) == oracle.candidate_periods(n)
    assert P.divisors(12) == [1, 2, 3, 4, 6, 12]
    assert P.divisors(1) == []
    assert P.divisors(36, max_divisor=6) == [1, 2, 3, 4, 6]


def test_decision_sublist_gives_the_same_period(oracle):
    """Scoring only the candidates that can matter must not change the decision."""
    from gefen_b200 import partitioning as P

    gen = torch.Generator().manual_seed(0)
    for n in [64, 192, 768 * 768, 2 ** 20, 3 * 5 * 7 * 11 * 13, 2048 * 8192, 8 * 1009, 4 * 1013]:
        cands = P.candidate_periods(n)
        for trial in range(20):
            scores = torch.rand(len(cands), generator=gen).tolist()
            if trial % 4 == 0:
                scores = sorted(scores)
            full = list(zip(cands, scores))
            want = oracle.choose_period(full, n)
            assert P._finalize_period_results(full, False, n) == want
            sub = P.decision_periods(cands)
            got = P._finalize_period_results([(p, s) for p, s in full if p in set(sub)], False, n) if sub else 1
            assert got == want


def test_constructor_mirrors_the_reference_grouping():
    from gefen_b200 import Gefen

    a = torch.nn.Parameter(torch.zeros(4, 4))
    b = torch.nn.Parameter(torch.zeros(3))
    frozen = torch.nn.Parameter(torch.zeros(2), requires_grad=False)
    opt = Gefen([("Layer.A", a), b, {"params": [("C", frozen), ("D", torch.nn.Parameter(torch.ones(2)))], "lr": 0.5,
                                     "betas": (0.8, 0.9), "weight_decay": 0.2}], lr=1e-2, weight_decay=0.1)
    names = [g["name"] for g in opt.param_groups]
    assert names == ["layer.a", "param_1", "d"]
    assert all(len(g["params"]) == 1 for g in opt.param_groups)
    assert opt.param_groups[0]["lr"] == 1e-2 and opt.param_groups[0]["weight_decay"] == 0.1
    assert opt.param_groups[2]["lr"] == 0.5 and opt.param_groups[2]["beta1"] == 0.8 and opt.param_groups[2]["weight_decay"] == 0.2
    assert set(opt.defaults) == {"lr", "beta1", "beta2", "eps"}
    for bad in (dict(lr=-1.0), dict(betas=(1.0, 0.9)), dict(betas=(0.9, -0.1)), dict(weight_decay=-1.0), dict(eps=-1.0)):
        with pytest.raises(ValueError):
            Gefen([a], **bad)
    with pytest.raises(TypeError):
        Gefen([("x", 3)])
    sd = opt.state_dict()
    assert sd["gefen_global_step"] == 0 and sd["gefen_codebook"] is None


def test_step_without_cuda_is_loud():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from gefen_b200 import Gefen

    p = torch.nn.Parameter(torch.zeros(8, 8))
    p.grad = torch.ones(8, 8)
    with pytest.raises(Exception):
        Gefen([p]).step()


def test_quantiser_and_division_building_blocks(tmp_path, oracle):
    """The scalar code the kernels are built from, compiled for the host and swept against the
    reference rule on a DP-shaped codebook and on degenerate ones."""
    import numpy as np

    exe = tmp_path / "sweep"
    subprocess.run(["/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++", "-O2", "-fopenmp", "-ffp-contract=off",
                    "-mfma", "-mavx2", "-std=c++17", "-o", str(exe), str(ROOT / "tests" / "native" / "quant_core_sweep.cpp")],
                   check=True)
    from tests.util import reference_like_codebook

    books = {
        "dp_like": reference_like_codebook().numpy(),
        "duplicates": np.array([-1.0, -0.5, -0.5, -0.5, 0.0, 0.0, 0.25, 0.2500001, 1.0], dtype=np.float32),
        "linear": np.linspace(-1, 1, 256).astype(np.float32),
        "beyond_range": np.sort((np.random.RandomState(0).rand(256) * 2.4 - 1.2).astype(np.float32)),
        "single": np.array([0.3], dtype=np.float32),
        "max_below_one": np.linspace(-0.7, 0.6, 16).astype(np.float32),
    }
    for name, cb in books.items():
        path = tmp_path / (name + ".f32")
        cb.tofile(path)
        out = subprocess.run([str(exe), str(path), "sample"], capture_output=True, text=True, check=True).stdout.split()
        bad_lut, bad_thr, slow, bad_div, checked = (int(x) for x in out)
        assert bad_lut == 0 and bad_thr == 0 and bad_div == 0 and checked > 2_000_000, (name, out)
        if name == "dp_like":
            assert slow < 0.05 * checked  # codebooks from the exact DP rarely need the slow path


def test_flat_layout_invariants():
    from gefen_b200 import workloads
    from gefen_b200.zero1 import FlatLayout

    for fn in (workloads.llama_1_5b, workloads.gpt2_125m, workloads.qwen3_1_7b_matrices, workloads.llama_32b):
        shapes = [s for _, s in fn()]
        total = sum(workloads.numel(s) for s in shapes)
        for world in (1, 2, 3, 4, 8):
            layout = FlatLayout(shapes, world)
            by_tensor = {}
            for p in layout.pieces:
                assert p.rank * layout.segment <= p.offset and p.offset + p.numel <= (p.rank + 1) * layout.segment
                by_tensor.setdefault(p.tensor, []).append(p)
            assert len(by_tensor) == len(shapes)
            for t, ps in by_tensor.items():
                ps.sort(key=lambda q: q.row0)
                assert ps[0].row0 == 0
                assert sum(q.numel for q in ps) == workloads.numel(shapes[t])
                for a, b in zip(ps, ps[1:]):  # a split tensor stays one contiguous range
                    assert a.offset + a.numel == b.offset and a.row0 + a.rows == b.row0
            loads = [sum(p.numel for p in layout.owned(r)) for r in range(world)]
            assert max(loads) <= total / world * 1.01 + 8192


def test_whole_tensor_layout_invariants():
    from gefen_b200 import workloads
    from gefen_b200.zero1 import WholeTensorLayout

    shapes = [s for _, s in workloads.qwen3_1_7b_matrices()] + [(7, 3), (1, 8)]
    total = sum(workloads.numel(s) for s in shapes)
    for world in (1, 2, 3, 8):
        layout = WholeTensorLayout(shapes, world)
        assert layout.total == layout.segment * world
        spans = []
        for t, pc in enumerate(layout.pieces):
            assert pc.tensor == t and pc.row0 == 0 and pc.numel == workloads.numel(shapes[t])
            assert pc.offset % 8 == 0
            assert pc.rank * layout.segment <= pc.offset and pc.offset + pc.numel <= (pc.rank + 1) * layout.segment
            spans.append((pc.offset, pc.offset + pc.numel))
        spans.sort()
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
        loads = [sum(p.numel for p in layout.owned(r)) for r in range(world)]
        assert sum(loads) == total and max(loads) - min(loads) <= max(workloads.numel(s) for s in shapes)


def test_kernel_class_of_a_table_row():
    """Which kernel a tensor gets is host logic of the library (no GPU): 1 = staged path with blocks that
    take a whole warp (more than 1024 elements), 2 = staged path with several blocks per warp pass, 0 / -1 =
    generic warp / CTA per block (periods that are not multiples of 8, unaligned tensors, 4-bit codes,
    period-1 tensors)."""
    import numpy as np

    from gefen_b200 import _lib

    lib = _lib.load()

    def cls(period, dtype=_lib.BF16, flags=0, p=0x10000, g=0x20000, codes=0x30000):
        row = np.zeros(1, dtype=_lib.STEP_TENSOR_DTYPE)
        row["p"], row["g"], row["codes"], row["mag"], row["v"] = p, g, codes, 0x40000, 0x50000
        row["period"], row["num_blocks"], row["flags"] = period, 4, flags
        return lib.gefen_b200_step_tensor_class(row.ctypes.data, dtype)

    assert [cls(p) for p in (2048, 1032, 4096, 8192)] == [1, 1, 1, 1]
    assert [cls(p) for p in (8, 64, 128, 248, 256, 512, 768, 1024)] == [2, 2, 2, 2, 2, 2, 2, 2]
    assert [cls(p, _lib.F32) for p in (768, 1536)] == [2, 1]
    assert [cls(p) for p in (9, 12, 100, 2044)] == [0, 0, 0, 0]
    assert cls(4100) == -1 and cls(8200) == -1               # long blocks off the staged path: a CTA per block
    assert cls(2048, flags=_lib.STEP_PERIOD1) == 0
    assert cls(2048, flags=_lib.STEP_PACKED) == 0
    assert cls(2048, p=0x10008) == 0 and cls(2048, g=0x20002) == 0 and cls(2048, codes=0x30004) == 0
    assert cls(2048, _lib.F64) == 0
