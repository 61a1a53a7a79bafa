"""Exact integer histogram of block-normalised gradients
(reference: kernels/exact_histogram_fused.py:10-58)."""
from __future__ import annotations

import torch

from .. import _lib
from ._common import require_cuda_tensors


def gefen_exact_histogram_cuda(grad_flat: torch.Tensor, period: int, bin_counts: torch.Tensor) -> None:
    """bin_counts[b] += number of elements whose g/absmax(block) falls in bin b; int64, added to."""
    require_cuda_tensors({"grad_flat": grad_flat, "bin_counts": bin_counts})
    if grad_flat.dim() != 1:
        raise ValueError("Expected grad_flat to be 1D, got dim={}".format(grad_flat.dim()))
    if bin_counts.dim() != 1:
        raise ValueError("Expected bin_counts to be 1D, got dim={}".format(bin_counts.dim()))
    if bin_counts.dtype != torch.int64:
        raise ValueError("Expected bin_counts to be int64, got {}".format(bin_counts.dtype))
    if period <= 0:
        raise ValueError("Expected period to be positive, got {}".format(period))
    if grad_flat.numel() % period != 0:
        raise ValueError("Expected grad_flat.numel()={} to be divisible by period={}.".format(
            grad_flat.numel(), period))
    if bin_counts.numel() <= 0 or bin_counts.numel() > 4096:
        raise ValueError("Expected histogram bins in [1, 4096], got {}".format(bin_counts.numel()))
    if not bin_counts.is_contiguous():
        raise ValueError("Expected bin_counts to be contiguous.")
    grad_flat = grad_flat.contiguous()
    with _lib.device_guard(grad_flat.device):
        _lib.check(_lib.load().gefen_b200_exact_histogram(
            _lib.ptr(grad_flat), _lib.dtype_tag(grad_flat.dtype), grad_flat.numel(), int(period),
            _lib.ptr(bin_counts), bin_counts.numel(), _lib.current_stream(grad_flat.device)))
