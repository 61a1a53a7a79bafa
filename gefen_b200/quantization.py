"""Codebook fit: exact 1-D k-means by dynamic programming, run on the GPU
(reference: quantization.py:55-258)."""
from __future__ import annotations

import torch

from . import _lib


def _build_padded_codebook(active_centers: torch.Tensor, num_codebooks: int, force_endpoints: bool) -> torch.Tensor:
    """Fewer active bins than entries: the centres themselves, the tail repeated (reference :68-81)."""
    n = int(active_centers.numel())
    codebook = torch.empty(num_codebooks, dtype=torch.float32)
    codebook[:n] = active_centers
    codebook[n:] = active_centers[-1]
    if force_endpoints:
        codebook[0] = -1.0
        codebook[-1] = 1.0
    return codebook.sort().values


def exact_dp(histogram_stats: dict, num_codebooks: int, force_endpoints: bool = True,
             device: torch.device | None = None) -> torch.Tensor:
    """Returns the sorted float32 codebook on the CPU, like the reference (:206-258). The prefix
    sums are formed on the host in the reference's order (sequential fp64 cumsum); the O(B^2 K)
    recurrence runs on `device` (default: the current CUDA device)."""
    active_centers = histogram_stats["active_centers"].detach().cpu().to(torch.float32)
    active_counts = histogram_stats["active_counts"].detach().cpu().to(torch.float32)
    if active_centers.numel() == 0:
        raise ValueError("Cannot run exact DP on an empty histogram.")
    if not torch.all(active_counts > 0):
        raise ValueError("exact DP expects strictly positive counts for all active histogram bins.")
    if num_codebooks > active_centers.numel():
        return _build_padded_codebook(active_centers, num_codebooks, force_endpoints)

    n = int(active_centers.numel())
    w = active_counts.to(torch.float64)
    x = active_centers.to(torch.float64)
    prefix = torch.zeros(3, n + 1, dtype=torch.float64)
    prefix[0, 1:] = torch.cumsum(w, dim=0)
    prefix[1, 1:] = torch.cumsum(w * x, dim=0)
    prefix[2, 1:] = torch.cumsum(w * x.square(), dim=0)

    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    lib = _lib.load()
    prefix_dev = prefix.to(device)
    scratch = torch.empty(lib.gefen_b200_exact_dp_scratch_bytes(n, num_codebooks), dtype=torch.uint8, device=device)
    out = torch.empty(num_codebooks, dtype=torch.float32, device=device)
    with _lib.device_guard(device):
        _lib.check(lib.gefen_b200_exact_dp(
            _lib.ptr(prefix_dev[0]), _lib.ptr(prefix_dev[1]), _lib.ptr(prefix_dev[2]), n, int(num_codebooks),
            int(bool(force_endpoints)), _lib.ptr(scratch), _lib.ptr(out), _lib.current_stream(device)))
    # the last 16 bytes of the scratch hold the status word of the backtrack (0 = a complete path)
    tail = torch.cat([out.view(torch.uint8), scratch[-16:]]).cpu()
    codebook = tail[: num_codebooks * 4].view(torch.float32).clone()
    status = int(tail[num_codebooks * 4:].view(torch.int32)[0])
    if status != 0:
        raise RuntimeError("exact DP could not trace a complete partition back (status {})".format(status))
    if not bool(torch.isfinite(codebook).all()):
        raise RuntimeError("exact DP produced a non-finite codebook")
    return codebook.sort().values
