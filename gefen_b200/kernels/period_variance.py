"""Block-period scores (reference: kernels/period_variance.py:10-161). Each function returns a
Python float like the reference wrappers; `period_scan` scores every candidate period of a tensor
with one host synchronisation instead of one per candidate (reference: partitioning.py:259-268)."""
from __future__ import annotations

import numpy as np
import torch

from .. import _lib


def _check(values: torch.Tensor, period: int) -> torch.Tensor:
    if not isinstance(values, torch.Tensor):
        raise TypeError("Expected torch.Tensor, got {}".format(type(values).__name__))
    if values.device.type != "cuda":
        raise ValueError("Expected a CUDA tensor, got device {}".format(values.device))
    if values.numel() == 0:
        raise ValueError("Expected a non-empty tensor.")
    if period <= 0:
        raise ValueError("Expected a positive period, got {}".format(period))
    if values.numel() % period != 0:
        raise ValueError("Expected length {} to be divisible by period {}.".format(values.numel(), period))
    if not values.is_floating_point():
        raise ValueError("Expected a floating-point tensor.")
    return values.detach().reshape(-1).contiguous()


def average_within_block_variance_cuda_kernel(values: torch.Tensor, period: int, *, input_is_squared: bool) -> float:
    flat = _check(values, period)
    stats = torch.empty(1, dtype=torch.float64, device=flat.device)
    with _lib.device_guard(flat.device):
        _lib.check(_lib.load().gefen_b200_average_within_block_variance(
            _lib.ptr(flat), _lib.dtype_tag(flat.dtype), flat.numel(), int(period), int(bool(input_is_squared)),
            _lib.ptr(stats), _lib.current_stream(flat.device)))
    # reference post-op: result.div_(logical_blocks).sqrt_() (period_variance_kernel.cu:242)
    return float((stats[0] / float(flat.numel() // period)).sqrt().item())


def average_within_block_coefficient_of_variation_cuda_kernel(values: torch.Tensor, period: int, *,
                                                              input_is_squared: bool) -> float:
    flat = _check(values, period)
    stats = torch.empty(3, dtype=torch.float64, device=flat.device)
    with _lib.device_guard(flat.device):
        _lib.check(_lib.load().gefen_b200_average_within_block_coefficient_of_variation(
            _lib.ptr(flat), _lib.dtype_tag(flat.dtype), flat.numel(), int(period), int(bool(input_is_squared)),
            _lib.ptr(stats), _lib.current_stream(flat.device)))
    host = stats.cpu()
    # reference post-ops and errors: period_variance_kernel.cu:311-317
    if host[2].item() > 0.0:
        raise RuntimeError("Expected non-negative block means for coefficient of variation.")
    if host[1].item() == 0.0:
        raise RuntimeError("Encountered only zero block means, cannot compute coefficient of variation.")
    return float((host[0] / host[1]).item())


def average_adjacent_log_block_mean_difference_cuda_kernel(values: torch.Tensor, period: int, *,
                                                           input_is_squared: bool, epsilon: float) -> float:
    flat = _check(values, period)
    if epsilon <= 0.0:
        raise ValueError("Expected a positive epsilon, got {}".format(epsilon))
    if flat.numel() // period < 2:
        raise ValueError("Expected at least two blocks to compare adjacent block means.")
    return period_scan(flat, [int(period)], input_is_squared=input_is_squared, epsilon=epsilon)[0]


def period_scan_async(flat: torch.Tensor, periods, *, input_is_squared: bool, epsilon: float) -> torch.Tensor:
    """Enqueues the scores of all `periods`; returns the device tensor [len(periods), 2] of
    (score, invalid count) without synchronising."""
    lib = _lib.load()
    host_periods = np.ascontiguousarray(np.asarray(periods, dtype=np.int64))
    n = int(host_periods.size)
    stats = torch.empty((n, 2), dtype=torch.float64, device=flat.device)
    if n == 0:
        return stats
    scratch_len = lib.gefen_b200_period_scan_scratch_doubles(flat.numel(), host_periods.ctypes.data, n)
    scratch = torch.empty(scratch_len, dtype=torch.float64, device=flat.device)
    with _lib.device_guard(flat.device):
        _lib.check(lib.gefen_b200_period_scan(
            _lib.ptr(flat), _lib.dtype_tag(flat.dtype), flat.numel(), int(bool(input_is_squared)), float(epsilon),
            host_periods.ctypes.data, n, _lib.ptr(stats), _lib.ptr(scratch), _lib.current_stream(flat.device)))
    return stats


def scores_from_stats(stats_host: torch.Tensor):
    """Applies the reference's error rule (period_variance_kernel.cu:392-394) to fetched stats."""
    if stats_host.numel() and bool((stats_host[:, 1] > 0).any()):
        raise RuntimeError("Expected values plus epsilon to be positive before log transform.")
    return [float(s) for s in stats_host[:, 0].tolist()]


def period_scan(flat: torch.Tensor, periods, *, input_is_squared: bool, epsilon: float):
    return scores_from_stats(period_scan_async(flat, periods, input_is_squared=input_is_squared,
                                               epsilon=epsilon).cpu())


# The reference registers its variance score as an opaque custom operator so that graph capture treats it
# as one node (kernels/period_variance.py:49-72); the same registration under this package's namespace.
if hasattr(torch.library, "custom_op"):

    @torch.library.custom_op("gefen_b200::average_within_block_variance_cuda", mutates_args=())
    def _average_within_block_variance_cuda_opaque(values: torch.Tensor, period: int, input_is_squared: bool) -> torch.Tensor:
        score = average_within_block_variance_cuda_kernel(values, period, input_is_squared=input_is_squared)
        return torch.tensor(score, dtype=torch.float64, device=values.device)

    @_average_within_block_variance_cuda_opaque.register_fake
    def _average_within_block_variance_cuda_opaque_fake(values: torch.Tensor, period: int, input_is_squared: bool) -> torch.Tensor:
        del period, input_is_squared
        return values.new_empty((), dtype=torch.float64)

    _OPAQUE_OP_AVAILABLE = True
else:
    _OPAQUE_OP_AVAILABLE = False
