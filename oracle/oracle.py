"""TEST INFRASTRUCTURE - Python face of the CPU oracle (oracle/gefen_oracle.c plus the host-side
calibration logic). Only tests, the smoke check and bench.py's cpu_baseline leg import this.

The functions mirror, on CPU tensors, the operations of the reference's CUDA extension
(kernels/gefen_cuda_binding.cpp:107-217) and of its calibration pipeline (partitioning.py,
quantization.py, gefen.py:305-419), mutating their arguments in place like the originals.
"""
from __future__ import annotations

import ctypes
import math
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libgefen_oracle.so"
_lib = None

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.float64: 3}


def build(force: bool = False) -> Path:
    src = _HERE / "gefen_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libgefen_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.oracle_adjacent_log_score.restype = ctypes.c_double
        _lib.oracle_exact_dp.restype = ctypes.c_int
        _lib.oracle_adjacent_log_scores_many.restype = ctypes.c_int
        _lib.oracle_nearest_index.restype = ctypes.c_int
        _lib.oracle_get_contraction.restype = ctypes.c_int
    return _lib


def set_contraction(mode: int) -> None:
    lib().oracle_set_contraction(ctypes.c_int(mode))


def _ptr(t: torch.Tensor):
    assert t.device.type == "cpu" and t.is_contiguous(), "oracle works on contiguous CPU tensors"
    return ctypes.c_void_p(t.data_ptr())


def _d(x: float):
    return ctypes.c_double(float(x))


def _i64(x: int):
    return ctypes.c_int64(int(x))


# ----------------------------------------------------------------------------- kernels
def nearest_indices(codebook: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    xf = x.detach().float().contiguous().reshape(-1)
    out = torch.empty(xf.numel(), dtype=torch.uint8)
    lib().oracle_nearest_indices(_ptr(xf), _i64(xf.numel()), _ptr(codebook), ctypes.c_int(codebook.numel()), _ptr(out))
    return out.view(x.shape)


def _unpack_nibbles(m_sign: torch.Tensor, numel: int) -> torch.Tensor:
    """4-bit codes, two per byte, low nibble first (reference: automatic_gefen_fused_kernel.cu:14-27)."""
    flat = m_sign.reshape(-1)
    both = torch.stack([flat & 0x0F, (flat >> 4) & 0x0F], dim=1).reshape(-1)
    return both[:numel].contiguous()


def _pack_nibbles(codes: torch.Tensor, m_sign: torch.Tensor) -> None:
    """Writes the codes back in place; an odd tail leaves the unused high nibble as it was."""
    flat = m_sign.reshape(-1)
    c = codes.reshape(-1)
    pairs = c.numel() // 2
    flat[:pairs] = (c[0:2 * pairs:2] & 0x0F) | ((c[1:2 * pairs:2] & 0x0F) << 4)
    if c.numel() % 2:
        flat[pairs] = (flat[pairs] & 0xF0) | (c[-1] & 0x0F)


class _Codes:
    """Byte-per-code view of m_sign for the C kernels, packed back on exit when needed."""

    def __init__(self, m_sign, shape, packed):
        self.m_sign, self.packed = m_sign, packed
        numel = 1
        for d in shape:
            numel *= d
        self.codes = _unpack_nibbles(m_sign, numel).view(shape) if packed else m_sign

    def __enter__(self):
        return self.codes

    def __exit__(self, *exc):
        if self.packed:
            _pack_nibbles(self.codes, self.m_sign)
        return False


def automatic_vmean_update(vmean, grad_view, beta2):
    nb, period = grad_view.shape
    lib().oracle_vmean_update(_ptr(vmean), _DT[vmean.dtype], _ptr(grad_view), _DT[grad_view.dtype], _i64(nb),
                              _i64(period), _d(beta2))


def automatic_gefen_fused_update_from_vmean(p, grad_view, m_sign, m_magnitude, vmean, codebook, packed_indices,
                                            beta1, lr, bias_correction_1, bias_correction_2, eps):
    nb, period = grad_view.shape
    with _Codes(m_sign, (nb, period), packed_indices) as codes:
        lib().oracle_fused_update_from_vmean(_ptr(p), _ptr(grad_view), _DT[p.dtype], _ptr(codes), _ptr(m_magnitude),
                                             _DT[m_magnitude.dtype], _ptr(vmean), _DT[vmean.dtype], _ptr(codebook),
                                             ctypes.c_int(codebook.numel()), _i64(nb), _i64(period), _d(beta1), _d(lr),
                                             _d(bias_correction_1), _d(bias_correction_2), _d(eps))


def automatic_gefen_fused_update(p, grad_view, m_sign, m_magnitude, stepsize, codebook, packed_indices, beta1, lr):
    nb, period = grad_view.shape
    with _Codes(m_sign, (nb, period), packed_indices) as codes:
        lib().oracle_fused_update(_ptr(p), _ptr(grad_view), _DT[p.dtype], _ptr(codes), _ptr(m_magnitude),
                                  _DT[m_magnitude.dtype], _ptr(stepsize), _ptr(codebook), ctypes.c_int(codebook.numel()),
                                  _i64(nb), _i64(period), _d(beta1), _d(lr))


def automatic_gefen_period1_update(p, grad_flat, m_sign, m_magnitude, vmean, codebook, period_one_divisor, beta1,
                                   beta2, lr, bias_correction_1, bias_correction_2, eps):
    lib().oracle_period1_update(_ptr(p), _ptr(grad_flat), _DT[p.dtype], _ptr(m_sign), _ptr(m_magnitude),
                                _DT[m_magnitude.dtype], _ptr(vmean), _DT[vmean.dtype], _ptr(codebook),
                                ctypes.c_int(codebook.numel()), _i64(grad_flat.numel()), _i64(period_one_divisor),
                                _d(beta1), _d(beta2), _d(lr), _d(bias_correction_1), _d(bias_correction_2), _d(eps))


def automatic_gefen_muon_momentum(grad_view, m_sign, m_magnitude, codebook, momentum_update, packed_indices, beta1):
    nb, period = grad_view.shape
    with _Codes(m_sign, (nb, period), packed_indices) as codes:
        lib().oracle_muon_momentum(_ptr(grad_view), _DT[grad_view.dtype], _ptr(codes), _ptr(m_magnitude),
                                   _DT[m_magnitude.dtype], _ptr(codebook), ctypes.c_int(codebook.numel()),
                                   _ptr(momentum_update), _i64(nb), _i64(period), _d(beta1))


def weight_decay(p, lr, wd):
    lib().oracle_weight_decay(_ptr(p), _DT[p.dtype], _i64(p.numel()), _d(lr), _d(wd))


def gefen_exact_histogram(grad_flat, period, bin_counts):
    lib().oracle_histogram(_ptr(grad_flat), _DT[grad_flat.dtype], _i64(grad_flat.numel()), _i64(period),
                           _ptr(bin_counts), ctypes.c_int(bin_counts.numel()))


def average_adjacent_log_block_mean_difference(values, period, input_is_squared, epsilon):
    invalid = ctypes.c_double(0.0)
    score = lib().oracle_adjacent_log_score(_ptr(values), _DT[values.dtype], _i64(values.numel()), _i64(period),
                                            ctypes.c_int(1 if input_is_squared else 0), _d(epsilon),
                                            ctypes.byref(invalid))
    if invalid.value > 0:
        raise RuntimeError("Expected values plus epsilon to be positive before log transform.")
    return score


def adjacent_log_scores(values, periods, input_is_squared, epsilon):
    """Scores of several candidate periods of one tensor: the logarithms are taken once, the sums are
    added in the order of `average_adjacent_log_block_mean_difference` (bit-identical scores)."""
    arr = (ctypes.c_int64 * len(periods))(*[int(p) for p in periods])
    out = (ctypes.c_double * len(periods))()
    invalid = ctypes.c_double(0.0)
    rc = lib().oracle_adjacent_log_scores_many(_ptr(values), _DT[values.dtype], _i64(values.numel()), arr,
                                               ctypes.c_int(len(periods)), ctypes.c_int(1 if input_is_squared else 0),
                                               _d(epsilon), out, ctypes.byref(invalid))
    if rc != 0:
        raise MemoryError("oracle: no memory for the logarithm scratch of {} elements".format(values.numel()))
    if invalid.value > 0:
        raise RuntimeError("Expected values plus epsilon to be positive before log transform.")
    return [float(x) for x in out]


def block_moments(values, period, input_is_squared, cov):
    stats = torch.zeros(3, dtype=torch.float64)
    lib().oracle_block_moments(_ptr(values), _DT[values.dtype], _i64(values.numel()), _i64(period),
                               ctypes.c_int(1 if input_is_squared else 0), ctypes.c_int(1 if cov else 0), _ptr(stats))
    return stats


def gefen_lloyd_accumulate(grad_flat, codebook, period, sums, counts):
    """sums: float64[K] (order-free yardstick for the kernels' fp32 atomics), counts: int64[K]."""
    lib().oracle_lloyd_accumulate(_ptr(grad_flat), _DT[grad_flat.dtype], _i64(grad_flat.numel()), _i64(period),
                                  _ptr(codebook), ctypes.c_int(codebook.numel()), _ptr(sums), _ptr(counts))


def gefen_lloyd_mse(grad_flat, old_codebook, new_codebook, period):
    out = torch.zeros(2, dtype=torch.float64)
    lib().oracle_lloyd_mse(_ptr(grad_flat), _DT[grad_flat.dtype], _i64(grad_flat.numel()), _i64(period),
                           _ptr(old_codebook), _ptr(new_codebook), ctypes.c_int(old_codebook.numel()), _ptr(out))
    return out


# ----------------------------------------------------------------------------- calibration host logic
DMNB = 4          # minimum number of blocks (reference: partitioning.py:6)
PERIOD_CAP = 1024  # reference: partitioning.py:328


def divisors(n: int, max_divisor=None):
    """Divisors of n below n, ascending (reference: partitioning.py:13-30)."""
    small, large = [], []
    for i in range(1, math.isqrt(n) + 1):
        if n % i == 0:
            if i != n and (max_divisor is None or i <= max_divisor):
                small.append(i)
            j = n // i
            if j != i and (max_divisor is None or j <= max_divisor):
                large.append(j)
    return small + large[::-1]


def candidate_periods(n: int, max_period=None, min_num_blocks: int = DMNB):
    return [p for p in divisors(n, max_period) if n // p >= min_num_blocks]


def choose_period(periods_and_scores, flattened_length: int) -> int:
    """The local-maximum rule and the >1024 cap (reference: partitioning.py:277-347)."""
    ps = list(periods_and_scores)
    if not ps:
        raise ValueError("Expected at least one valid period candidate.")
    last_period = ps[-1][0]
    best = None
    for idx in range(1, len(ps) - 1):
        p, score = ps[idx]
        if p <= 8 or p == last_period:
            continue
        if score <= ps[idx - 1][1] or score <= ps[idx + 1][1]:
            continue
        if best is None or (score, p) > best:
            best = (score, p)
    if best is None:
        return 1
    if not math.isfinite(best[0]):
        raise ValueError("Expected finite best score, got {}.".format(best[0]))
    period = best[1]
    if period > PERIOD_CAP:
        period = min(q for q in divisors(flattened_length) if PERIOD_CAP < q <= period and period % q == 0)
    return period


def find_period(grad: torch.Tensor, *, cuda_kernel_semantics: bool = True, max_period=None, epsilon: float = 1e-12) -> int:
    """Period of one gradient tensor.

    cuda_kernel_semantics=True squares in fp64 from the fp32 value (the reference's CUDA backend,
    period_variance_kernel.cu:128-131); False squares in fp32 first (its CPU backend, gefen.py:813).
    """
    flat = grad.detach().reshape(-1)
    n = flat.numel()
    if n == 1:
        return 1
    cands = candidate_periods(n, max_period)
    if not cands:
        return 1
    if cuda_kernel_semantics:
        values, squared = flat.contiguous(), False
    else:
        values, squared = flat.float().square().contiguous(), True
    scores = list(zip(cands, adjacent_log_scores(values, cands, squared, epsilon)))
    return choose_period(scores, n)


def exact_dp(active_centers: torch.Tensor, active_counts: torch.Tensor, num_codebooks: int,
             force_endpoints: bool = True) -> torch.Tensor:
    """Sorted float32 codebook (reference: quantization.py:206-258, padded path :68-81)."""
    centers = active_centers.detach().cpu().float()
    counts = active_counts.detach().cpu().float()
    if centers.numel() == 0:
        raise ValueError("Cannot run exact DP on an empty histogram.")
    if num_codebooks > centers.numel():
        cb = torch.empty(num_codebooks, dtype=torch.float32)
        cb[: centers.numel()] = centers
        cb[centers.numel():] = centers[-1]
        if force_endpoints:
            cb[0], cb[-1] = -1.0, 1.0
        return cb.sort().values
    n = centers.numel()
    w = counts.double()
    x = centers.double()
    pw = torch.zeros(n + 1, dtype=torch.float64)
    pwx = torch.zeros(n + 1, dtype=torch.float64)
    pwx2 = torch.zeros(n + 1, dtype=torch.float64)
    pw[1:] = torch.cumsum(w, 0)
    pwx[1:] = torch.cumsum(w * x, 0)
    pwx2[1:] = torch.cumsum(w * x.square(), 0)
    out = torch.empty(num_codebooks, dtype=torch.float32)
    rc = lib().oracle_exact_dp(_ptr(pw), _ptr(pwx), _ptr(pwx2), ctypes.c_int(n), ctypes.c_int(num_codebooks),
                               ctypes.c_int(1 if force_endpoints else 0), _ptr(out))
    if rc != 0:
        raise RuntimeError("oracle exact_dp failed with code {}".format(rc))
    return out.sort().values


def histogram_stats(bin_counts_f32: torch.Tensor):
    bins = bin_counts_f32.numel()
    edges = torch.linspace(-1.0, 1.0, steps=bins + 1, dtype=torch.float32)
    centers = 0.5 * (edges[:-1] + edges[1:])
    active = bin_counts_f32 > 0
    return centers[active], bin_counts_f32[active]


def learn_codebook(grads_and_periods, num_codebooks: int = 256, force_endpoints: bool = True):
    """grads_and_periods: iterable of (flat CPU gradient, period). Accumulates the per-tensor int64
    histograms in float32 in the given order (reference: gefen.py:329-347) and fits the codebook."""
    bins = num_codebooks * 16
    total = torch.zeros(bins, dtype=torch.float32)
    seen = 0
    for flat, period in grads_and_periods:
        counts = torch.zeros(bins, dtype=torch.int64)
        gefen_exact_histogram(flat.contiguous(), period, counts)
        total.add_(counts.to(torch.float32))
        seen += flat.numel()
    if seen == 0:
        return None
    centers, counts = histogram_stats(total)
    return exact_dp(centers, counts, num_codebooks, force_endpoints)
