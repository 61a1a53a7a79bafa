"""Ahead-of-time build of libgefen_b200.so (sm_100a only) with plain nvcc.

Replaces the reference's JIT loader (kernels/gefen_cuda.py:6-22, kernels/_build_notice.py:364-444):
no torch headers, no pybind, one shared library with a C ABI, built in-tree.

    python -m gefen_b200.csrc.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
ROOT = PKG.parent
LIB_PATH = PKG / "libgefen_b200.so"
OBJ_DIR = CSRC / "build"

SOURCES = [
    "codebook_lut.cu",
    "step_kernels.cu",
    "calib_kernels.cu",
    "exact_dp.cu",
    "ns_gemm.cu",
]
HEADERS = ["common.cuh", "quant_core.h", "../../include/gefen_b200.h"]

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    if candidate.exists():
        return str(candidate)
    found = shutil.which("nvcc")
    if found is None:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every .cu of the package for sm_100a and links libgefen_b200.so."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    headers = [CSRC / h for h in HEADERS] + [Path(__file__)]
    extra = ["-Xptxas", "-v"] if verbose else []
    jobs = []
    for src in SOURCES:
        src_path = CSRC / src
        obj = OBJ_DIR / (src_path.stem + ".o")
        if force or _stale(obj, [src_path] + headers):
            jobs.append((src_path, obj))

    def compile_one(job):
        src_path, obj = job
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", str(src_path), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed for {}:\n{}\n{}".format(src_path.name, res.stdout, res.stderr))
        return src_path.name, res.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
            for name, log in pool.map(compile_one, jobs):
                if verbose and log:
                    print("== {}\n{}".format(name, log))
    objs = [OBJ_DIR / (Path(s).stem + ".o") for s in SOURCES]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH)] + [str(o) for o in objs]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n{}\n{}".format(res.stdout, res.stderr))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
