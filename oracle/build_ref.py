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
# where the reference checkout lies: the environment variable GEFEN_REFERENCE_ROOT (no default path)
_ROOT = os.environ.get("GEFEN_REFERENCE_ROOT")
REFERENCE_KERNELS = Path(_ROOT) / "kernels" if _ROOT else None
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


def build(force: bool = False, reference_root=None) -> Path:
    """reference_root: the reference checkout (default: the environment variable GEFEN_REFERENCE_ROOT)."""
    target = built_module_path()
    if target.exists() and not force:
        return target
    kernels = Path(reference_root) / "kernels" if reference_root is not None else REFERENCE_KERNELS
    if kernels is None or not kernels.is_dir():
        raise FileNotFoundError("reference sources not found: pass reference_root or set GEFEN_REFERENCE_ROOT to the "
                                "reference checkout (got {})".format(kernels))
    from torch.utils.cpp_extension import load

    OUT.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    load(
        name=NAME,
        sources=[str(kernels / s) for s in SOURCES],
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
    roots = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(force="--force" in sys.argv, reference_root=roots[0] if roots else None))
