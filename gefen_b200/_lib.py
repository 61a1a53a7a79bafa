"""ctypes binding of libgefen_b200.so, the C-ABI library that replaces the reference's pybind11
extension (kernels/gefen_cuda_binding.cpp:107-217) and its JIT loader (kernels/gefen_cuda.py:6-22).

There is no CPU path behind this module: if the library is missing or a call fails, it raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np
import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libgefen_b200.so"

F32, F16, BF16, F64 = 0, 1, 2, 3
_DTYPE_TAG = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.float64: F64}

OK, EINVAL, ECUDA, ERUNTIME, EUNSUPPORTED = 0, -1, -2, -3, -4

CODEBOOK_WS_BYTES = 34848

STEP_FUSE_VMEAN = 1
STEP_WEIGHT_DECAY = 2
STEP_PERIOD1 = 4
STEP_MUON = 8
STEP_NESTEROV = 16
STEP_PACKED = 32

# numpy mirror of gefen_b200_step_tensor_t (include/gefen_b200.h)
STEP_TENSOR_DTYPE = np.dtype(
    [
        ("p", "<u8"), ("g", "<u8"), ("codes", "<u8"), ("mag", "<u8"), ("v", "<u8"),
        ("first_block", "<i8"), ("num_blocks", "<i8"), ("period", "<i8"),
        ("beta1", "<f4"), ("beta2", "<f4"), ("lr", "<f4"), ("bc1", "<f4"), ("bc2", "<f4"), ("eps", "<f4"),
        ("wd_mul", "<f4"),
        ("flags", "<u4"), ("mag_dtype", "<i4"), ("v_dtype", "<i4"), ("reserved", "<i4", (2,)),
    ]
)

_lib = None


class GefenB200Error(RuntimeError):
    pass


def dtype_tag(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_TAG[dtype]
    except KeyError:
        raise ValueError("gefen_b200 supports float32, float16, bfloat16 and float64 tensors, got {}".format(dtype))


def _declare(lib):
    c = ctypes
    vp, i32, i64, dbl = c.c_void_p, c.c_int, c.c_int64, c.c_double
    sig = {
        "gefen_b200_last_error": (c.c_char_p, []),
        "gefen_b200_version": (i32, []),
        "gefen_b200_codebook_prepare": (i32, [vp, i32, vp, vp]),
        "gefen_b200_automatic_vmean_update": (i32, [vp, i32, vp, i32, i64, i64, dbl, vp]),
        "gefen_b200_automatic_gefen_fused_update_from_vmean": (
            i32, [vp, vp, i32, vp, vp, i32, vp, i32, vp, i32, vp, i32, i64, i64, dbl, dbl, dbl, dbl, dbl, vp]),
        "gefen_b200_automatic_gefen_fused_update_from_vmean_static_ws": (
            i32, [vp, vp, i32, vp, vp, i32, vp, i32, vp, i32, i32, i64, i64, dbl, dbl, dbl, dbl, dbl, vp]),
        "gefen_b200_automatic_gefen_fused_update": (
            i32, [vp, vp, i32, vp, vp, i32, vp, vp, i32, vp, i32, i64, i64, dbl, dbl, vp]),
        "gefen_b200_automatic_gefen_period1_update": (
            i32, [vp, vp, i32, vp, vp, i32, vp, i32, vp, i32, vp, i64, i64, dbl, dbl, dbl, dbl, dbl, dbl, vp]),
        "gefen_b200_automatic_gefen_muon_momentum": (
            i32, [vp, i32, vp, vp, i32, vp, i32, vp, vp, i32, i64, i64, dbl, vp]),
        "gefen_b200_multi_tensor_step": (i32, [vp, vp, i32, i32, vp, vp]),
        "gefen_b200_multi_tensor_step_peers": (i32, [vp, vp, i32, i32, vp, vp, i32, vp, i32, dbl, vp]),
        "gefen_b200_multi_tensor_step_multicast": (i32, [vp, vp, i32, i32, vp, vp, i32, vp, i32, dbl, i64, i64, vp]),
        "gefen_b200_multicast_sum": (i32, [vp, vp, i32, i64, dbl, vp]),
        "gefen_b200_muon_apply": (i32, [vp, vp, i32, i64, dbl, dbl, vp, i32, vp]),
        "gefen_b200_step_tensor_size": (i32, []),
        "gefen_b200_step_tensor_class": (i32, [vp, i32]),
        "gefen_b200_step_status": (i32, [vp, i32]),
        "gefen_b200_debug_set_stage_spin_limit": (i32, [i64]),
        "gefen_b200_exact_histogram": (i32, [vp, i32, i64, i64, vp, i32, vp]),
        "gefen_b200_average_within_block_variance": (i32, [vp, i32, i64, i64, i32, vp, vp]),
        "gefen_b200_average_within_block_coefficient_of_variation": (i32, [vp, i32, i64, i64, i32, vp, vp]),
        "gefen_b200_period_scratch_doubles": (i64, [i64, i64]),
        "gefen_b200_average_adjacent_log_block_mean_difference": (i32, [vp, i32, i64, i64, i32, dbl, vp, vp, vp]),
        "gefen_b200_period_scan_scratch_doubles": (i64, [i64, vp, i32]),
        "gefen_b200_period_scan": (i32, [vp, i32, i64, i32, dbl, vp, i32, vp, vp, vp]),
        "gefen_b200_lloyd_accumulate": (i32, [vp, i32, i64, i64, vp, i32, vp, vp, vp, vp]),
        "gefen_b200_lloyd_mse": (i32, [vp, i32, i64, i64, vp, vp, i32, vp, vp, vp, vp]),
        "gefen_b200_exact_dp_scratch_bytes": (i64, [i32, i32]),
        "gefen_b200_exact_dp": (i32, [vp, vp, vp, i32, i32, i32, vp, vp, vp]),
        "gefen_b200_ns_gemm_tn": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i64, dbl, dbl, i32, vp, vp]),
        "gefen_b200_newton_schulz": (i32, [vp, vp, vp, vp, i32, i32, i32, dbl, dbl, dbl, vp, vp]),
        "gefen_b200_ns_gemm_nn": (i32, [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, dbl, dbl, vp, vp]),
        "gefen_b200_ns_gemm_tt": (i32, [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, dbl, dbl, i32, vp, vp]),
    }
    for name, (restype, argtypes) in sig.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return sig


EXPORTED_SYMBOLS = None


def load():
    """Loads the library once. Raises if it has not been built (python -m gefen_b200.csrc.build)."""
    global _lib, EXPORTED_SYMBOLS
    if _lib is None:
        if not LIB_PATH.exists():
            raise GefenB200Error(
                "{} is missing: build it with `python -m gefen_b200.csrc.build`; gefen_b200 has no fallback path".format(
                    LIB_PATH))
        lib = ctypes.CDLL(str(LIB_PATH))
        EXPORTED_SYMBOLS = sorted(_declare(lib).keys())
        if lib.gefen_b200_step_tensor_size() != STEP_TENSOR_DTYPE.itemsize:
            raise GefenB200Error("step-tensor layout mismatch between the library and its Python mirror")
        _lib = lib
    return _lib


def check(rc: int) -> None:
    """Maps status codes to the exceptions the reference raises (ValueError for std::invalid_argument,
    RuntimeError otherwise)."""
    if rc == OK:
        return
    msg = load().gefen_b200_last_error().decode("utf-8", "replace")
    if rc == EINVAL:
        raise ValueError(msg)
    if rc == EUNSUPPORTED:
        raise NotImplementedError(msg)
    raise GefenB200Error(msg)


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def step_status(device, clear: bool = True) -> int:
    """Status word of the step kernels on `device` (synchronises it): non-zero when a bounded wait
    inside a step kernel ran out since the last clear, i.e. a step was left incomplete."""
    value = ctypes.c_int(0)
    with device_guard(device):
        check(load().gefen_b200_step_status(ctypes.byref(value), int(clear)))
    return int(value.value)


def check_step_status(device) -> None:
    """Raises GefenB200Error if a step kernel on `device` gave up a bounded wait (synchronises)."""
    if step_status(device, clear=True) != 0:
        raise GefenB200Error("a Gefen step kernel gave up waiting for its staged codebook tables; the optimizer "
                             "state and parameters of that step are incomplete")


def current_stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class device_guard:
    """Makes `device` current for the duration of a call (reference: c10::cuda::CUDAGuard)."""

    def __init__(self, device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        self.prev = torch.cuda.current_device()
        if self.prev != self.idx:
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev != self.idx:
            torch.cuda.set_device(self.prev)
        return False


# ------------------------------------------------------------------ codebook workspaces
_WORKSPACES = {}   # id(codebook tensor) -> (tag, workspace, event, stream handle, weak reference)


def codebook_workspace(codebook: torch.Tensor) -> torch.Tensor:
    """Device workspace (thresholds + lookup table) for `codebook`. It is kept for as long as the tensor
    object lives and rebuilt when the tensor is modified in place (its version counter moves) or
    reallocated. The tables are built on the stream that is current at that moment; an event recorded behind
    the build makes every later consumer on another stream wait for it."""
    import weakref

    key = id(codebook)
    tag = (codebook._version, codebook.data_ptr(), codebook.numel())
    hit = _WORKSPACES.get(key)
    stream = torch.cuda.current_stream(codebook.device)
    if hit is not None and hit[0] == tag and hit[4]() is codebook:
        if hit[3] != stream.cuda_stream:
            stream.wait_event(hit[2])
        return hit[1]
    ws = torch.empty(CODEBOOK_WS_BYTES, dtype=torch.uint8, device=codebook.device)
    with device_guard(codebook.device):
        check(load().gefen_b200_codebook_prepare(ptr(codebook), codebook.numel(), ptr(ws),
                                                 current_stream(codebook.device)))
    built = torch.cuda.Event()
    built.record(stream)
    _WORKSPACES[key] = (tag, ws, built, stream.cuda_stream, weakref.ref(codebook, lambda _ref, k=key: _WORKSPACES.pop(k, None)))
    return ws
