"""Block-shared second moment (reference: kernels/automatic_vmean.py:10-55)."""
from __future__ import annotations

import torch

from .. import _lib
from ._common import require_block_column, require_state_dtype


def automatic_vmean_update_cuda(vmean: torch.Tensor, grad_view: torch.Tensor, beta2: float) -> None:
    """vmean[b] <- beta2 * vmean[b] + (1 - beta2) * mean(grad_view[b, :]^2), in place."""
    if not isinstance(vmean, torch.Tensor):
        raise TypeError("Expected vmean to be a torch.Tensor.")
    if not isinstance(grad_view, torch.Tensor):
        raise TypeError("Expected grad_view to be a torch.Tensor.")
    if vmean.device.type != "cuda":
        raise ValueError("Expected vmean to be on CUDA, got device {}.".format(vmean.device))
    if grad_view.device.type != "cuda":
        raise ValueError("Expected grad_view to be on CUDA, got device {}.".format(grad_view.device))
    if grad_view.dim() != 2:
        raise ValueError("Expected grad_view to be 2D, got dim={}.".format(grad_view.dim()))
    require_block_column("vmean", vmean)
    if grad_view.shape[0] != vmean.shape[0]:
        raise ValueError("Expected grad_view and vmean to have the same number of blocks.")
    require_state_dtype("vmean", vmean)
    if not 0.0 <= beta2 <= 1.0:
        raise ValueError("Expected beta2 to be in [0, 1], got {}.".format(beta2))
    if not vmean.is_contiguous():
        raise ValueError("Expected vmean to be contiguous.")
    grad_view = grad_view.contiguous()
    with _lib.device_guard(vmean.device):
        _lib.check(_lib.load().gefen_b200_automatic_vmean_update(
            _lib.ptr(vmean), _lib.dtype_tag(vmean.dtype), _lib.ptr(grad_view), _lib.dtype_tag(grad_view.dtype),
            grad_view.shape[0], grad_view.shape[1], float(beta2), _lib.current_stream(vmean.device)))
