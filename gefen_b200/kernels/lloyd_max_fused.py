"""Lloyd-Max E-step and logging MSE (reference: kernels/lloyd_max_fused.py:10-143), plus the
iteration loop the reference no longer ships (its research path was removed, cf. the error text at
gefen.py:319-327); the loop here is therefore not pinned by the reference."""
from __future__ import annotations

import torch

from .. import _lib
from ._common import require_cuda_tensors


def _check_flat_and_codebook(grad_flat, codebook, period):
    if grad_flat.dim() != 1:
        raise ValueError("Expected grad_flat to be 1D, got dim={}".format(grad_flat.dim()))
    if codebook.dim() != 1:
        raise ValueError("Expected codebook to be 1D, got dim={}".format(codebook.dim()))
    if codebook.dtype != torch.float32:
        raise ValueError("Expected codebook to be float32, got {}".format(codebook.dtype))
    if period <= 0:
        raise ValueError("Expected period to be positive, got {}".format(period))
    if grad_flat.numel() % period != 0:
        raise ValueError("Expected grad_flat.numel()={} to be divisible by period={}.".format(
            grad_flat.numel(), period))
    if codebook.numel() > 256 or codebook.numel() < 1:
        raise ValueError("Expected codebook to have at most 256 entries, got {}".format(codebook.numel()))


def gefen_lloyd_accumulate_cuda(grad_flat, codebook, period: int, sums, counts) -> None:
    """sums[e] += sum of normalised values nearest to entry e; counts[e] += their number."""
    require_cuda_tensors({"grad_flat": grad_flat, "codebook": codebook, "sums": sums, "counts": counts})
    _check_flat_and_codebook(grad_flat, codebook, period)
    if sums.dim() != 1 or sums.numel() != codebook.numel():
        raise ValueError("Expected sums to be 1D with one entry per codebook value.")
    if counts.dim() != 1 or counts.numel() != codebook.numel():
        raise ValueError("Expected counts to be 1D with one entry per codebook value.")
    if sums.dtype != torch.float32:
        raise ValueError("Expected sums to be float32, got {}".format(sums.dtype))
    if counts.dtype != torch.int64:
        raise ValueError("Expected counts to be int64, got {}".format(counts.dtype))
    grad_flat = grad_flat.contiguous()
    codebook = codebook.contiguous()
    with _lib.device_guard(grad_flat.device):
        _lib.check(_lib.load().gefen_b200_lloyd_accumulate(
            _lib.ptr(grad_flat), _lib.dtype_tag(grad_flat.dtype), grad_flat.numel(), int(period),
            _lib.ptr(codebook), codebook.numel(), _lib.ptr(_lib.codebook_workspace(codebook)), _lib.ptr(sums),
            _lib.ptr(counts), _lib.current_stream(grad_flat.device)))


def gefen_lloyd_mse_cuda(grad_flat, old_codebook, new_codebook, period: int, mse_normalized_sum,
                         mse_original_sum) -> None:
    """Adds the squared error of assigning with old_codebook and reconstructing with new_codebook,
    in normalised and in original scale, to the two one-element fp32 accumulators."""
    require_cuda_tensors({"grad_flat": grad_flat, "old_codebook": old_codebook, "new_codebook": new_codebook,
                          "mse_normalized_sum": mse_normalized_sum, "mse_original_sum": mse_original_sum})
    _check_flat_and_codebook(grad_flat, old_codebook, period)
    if new_codebook.dim() != 1 or new_codebook.numel() != old_codebook.numel():
        raise ValueError("Expected new_codebook to be 1D with the size of old_codebook.")
    if new_codebook.dtype != torch.float32:
        raise ValueError("Expected new_codebook to be float32, got {}".format(new_codebook.dtype))
    for name, t in (("mse_normalized_sum", mse_normalized_sum), ("mse_original_sum", mse_original_sum)):
        if t.numel() != 1 or t.dtype != torch.float32:
            raise ValueError("Expected {} to be a one-element float32 tensor.".format(name))
    grad_flat = grad_flat.contiguous()
    old_codebook = old_codebook.contiguous()
    new_codebook = new_codebook.contiguous()
    with _lib.device_guard(grad_flat.device):
        _lib.check(_lib.load().gefen_b200_lloyd_mse(
            _lib.ptr(grad_flat), _lib.dtype_tag(grad_flat.dtype), grad_flat.numel(), int(period),
            _lib.ptr(old_codebook), _lib.ptr(new_codebook), old_codebook.numel(),
            _lib.ptr(_lib.codebook_workspace(old_codebook)), _lib.ptr(mse_normalized_sum),
            _lib.ptr(mse_original_sum), _lib.current_stream(grad_flat.device)))


def lloyd_max_fit(grads_and_periods, codebook: torch.Tensor, iterations: int = 10,
                  force_endpoints: bool = True) -> torch.Tensor:
    """Iterates E-step (kernel) and M-step: entry <- sums/counts where counts > 0, the two end
    entries pinned to -1 and +1 when force_endpoints, then re-sorted. Returns a new codebook."""
    cb = codebook.detach().clone().float().contiguous()
    k = cb.numel()
    for _ in range(iterations):
        sums = torch.zeros(k, dtype=torch.float32, device=cb.device)
        counts = torch.zeros(k, dtype=torch.int64, device=cb.device)
        for flat, period in grads_and_periods:
            gefen_lloyd_accumulate_cuda(flat, cb, period, sums, counts)
        filled = counts > 0
        new_cb = torch.where(filled, sums / counts.clamp(min=1).float(), cb)
        if force_endpoints:
            new_cb[0] = -1.0
            new_cb[-1] = 1.0
        cb = new_cb.sort().values.contiguous()
    return cb
