"""TEST INFRASTRUCTURE - builds the reference's own CUDA extension, from its sources where they lie,
into oracle/_ref/ (git-ignored). On a GPU box the resulting module is a second checker for the
kernels (the reference's production path) and gives the reference-kernel timing quoted beside the
benchmark. Nothing is copied: the sources are compiled in place for sm_100a with the reference's own
flags (-O3; kernels/_build_notice.py:407-414), by torch.utils.cpp_extension.load called directly
because the reference's loader refuses an nvcc whose version differs from torch's CUDA version.

    python -m oracle.build_ref
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NAME = "gefen_cuda_ext_ref"
REFERENCE_KERNELS = Path(os.environ.get("GEFEN_REFERENCE_ROOT", "/root/reference")) / "kernels"
SOURCES = [
    "gefen_cuda_binding.cpp",
    "automatic_gefen_fused_kernel.cu",
    "automatic_vmean_kernel.cu",
    "exact_histogram_fused_kernel.cu",
    "period_variance_kernel.cu",
    "lloyd_max_fused_kernel.cu",
]


def built_module_path() -> Path:
    return OUT / (NAME + ".so")


def build(force: bool = False) -> Path:
    target = built_module_path()
    if target.exists() and not force:
        return target
    if not REFERENCE_KERNELS.is_dir():
        raise FileNotFoundError("reference sources not found at {}".format(REFERENCE_KERNELS))
    from torch.utils.cpp_extension import load

    OUT.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    load(
        name=NAME,
        sources=[str(REFERENCE_KERNELS / s) for s in SOURCES],
        extra_cflags=["-O3"],
        extra_cuda_cflags=["-O3"],
        build_directory=str(OUT),
        is_python_module=False,
        verbose=False,
    )
    return target


def load_module():
    """Imports the built extension (needs a CUDA-capable torch at call time). Returns None if it has
    not been built."""
    target = built_module_path()
    if not target.exists():
        return None
    import torch  # noqa: F401  (the extension links against torch)

    spec = importlib.util.spec_from_file_location(NAME, str(target))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
