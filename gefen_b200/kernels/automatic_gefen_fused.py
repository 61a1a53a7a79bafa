"""The fused Gefen step, its period-1 and GefenMuon forms
(reference: kernels/automatic_gefen_fused.py:11-489)."""
from __future__ import annotations

import torch

from .. import _lib
from ._common import (
    require_block_column,
    require_codebook,
    require_contiguous,
    require_cuda_tensors,
    require_index_count,
    require_state_dtype,
)


def _ws(codebook: torch.Tensor):
    return _lib.ptr(_lib.codebook_workspace(codebook))


def automatic_gefen_fused_update_cuda(p, grad_view, m_sign, m_magnitude, stepsize, codebook, packed_indices: bool,
                                      beta1: float, lr: float) -> None:
    """Step with a precomputed per-block fp32 stepsize (reference wrapper :11-117)."""
    require_cuda_tensors({"p": p, "grad_view": grad_view, "m_sign": m_sign, "m_magnitude": m_magnitude,
                          "stepsize": stepsize, "codebook": codebook})
    if grad_view.dim() != 2:
        raise ValueError("Expected grad_view to be 2D, got dim={}".format(grad_view.dim()))
    if grad_view.dtype != p.dtype:
        raise ValueError("Expected grad_view dtype {} to match p dtype {}.".format(grad_view.dtype, p.dtype))
    require_block_column("m_magnitude", m_magnitude)
    require_block_column("stepsize", stepsize)
    if grad_view.shape[0] != m_magnitude.shape[0]:
        raise ValueError("Expected grad_view and m_magnitude to have the same number of blocks.")
    if grad_view.shape[0] != stepsize.shape[0]:
        raise ValueError("Expected grad_view and stepsize to have the same number of blocks.")
    require_state_dtype("m_magnitude", m_magnitude)
    if stepsize.dtype != torch.float32:
        raise ValueError("Expected stepsize to be float32, got {}".format(stepsize.dtype))
    require_codebook(codebook)
    require_index_count(m_sign, grad_view.numel(), packed_indices)
    if p.numel() != grad_view.numel():
        raise ValueError("Expected p.numel() to match grad_view.numel().")
    grad_view = grad_view.contiguous()
    stepsize = stepsize.contiguous()
    codebook = codebook.contiguous()
    require_contiguous({"p": p, "m_sign": m_sign, "m_magnitude": m_magnitude})
    with _lib.device_guard(p.device):
        _lib.check(_lib.load().gefen_b200_automatic_gefen_fused_update(
            _lib.ptr(p), _lib.ptr(grad_view), _lib.dtype_tag(p.dtype), _lib.ptr(m_sign), _lib.ptr(m_magnitude),
            _lib.dtype_tag(m_magnitude.dtype), _lib.ptr(stepsize), _lib.ptr(codebook), codebook.numel(),
            _ws(codebook), int(bool(packed_indices)), grad_view.shape[0], grad_view.shape[1], float(beta1),
            float(lr), _lib.current_stream(p.device)))


def automatic_gefen_fused_update_from_vmean_cuda(p, grad_view, m_sign, m_magnitude, vmean, codebook,
                                                 packed_indices: bool, beta1: float, lr: float,
                                                 bias_correction_1: float, bias_correction_2: float,
                                                 eps: float) -> None:
    """The production step for period > 1 (reference wrapper :120-249)."""
    require_cuda_tensors({"p": p, "grad_view": grad_view, "m_sign": m_sign, "m_magnitude": m_magnitude,
                          "vmean": vmean, "codebook": codebook})
    if grad_view.dim() != 2:
        raise ValueError("Expected grad_view to be 2D, got dim={}".format(grad_view.dim()))
    if grad_view.dtype != p.dtype:
        raise ValueError("Expected grad_view dtype {} to match p dtype {}.".format(grad_view.dtype, p.dtype))
    require_block_column("m_magnitude", m_magnitude)
    require_block_column("vmean", vmean)
    if grad_view.shape[0] != m_magnitude.shape[0]:
        raise ValueError("Expected grad_view and m_magnitude to have the same number of blocks.")
    if grad_view.shape[0] != vmean.shape[0]:
        raise ValueError("Expected grad_view and vmean to have the same number of blocks.")
    require_state_dtype("m_magnitude", m_magnitude)
    require_state_dtype("vmean", vmean)
    require_codebook(codebook)
    require_index_count(m_sign, grad_view.numel(), packed_indices)
    if bias_correction_1 <= 0.0:
        raise ValueError("Expected bias_correction_1 to be positive, got {}".format(bias_correction_1))
    if bias_correction_2 <= 0.0:
        raise ValueError("Expected bias_correction_2 to be positive, got {}".format(bias_correction_2))
    if eps < 0.0:
        raise ValueError("Expected eps to be non-negative, got {}".format(eps))
    if p.numel() != grad_view.numel():
        raise ValueError("Expected p.numel() to match grad_view.numel().")
    grad_view = grad_view.contiguous()
    vmean = vmean.contiguous()
    codebook = codebook.contiguous()
    require_contiguous({"p": p, "m_sign": m_sign, "m_magnitude": m_magnitude})
    with _lib.device_guard(p.device):
        _lib.check(_lib.load().gefen_b200_automatic_gefen_fused_update_from_vmean(
            _lib.ptr(p), _lib.ptr(grad_view), _lib.dtype_tag(p.dtype), _lib.ptr(m_sign), _lib.ptr(m_magnitude),
            _lib.dtype_tag(m_magnitude.dtype), _lib.ptr(vmean), _lib.dtype_tag(vmean.dtype), _lib.ptr(codebook),
            codebook.numel(), _ws(codebook), int(bool(packed_indices)), grad_view.shape[0], grad_view.shape[1],
            float(beta1), float(lr), float(bias_correction_1), float(bias_correction_2), float(eps),
            _lib.current_stream(p.device)))


def automatic_gefen_period1_update_cuda(p, grad_flat, m_sign, m_magnitude, vmean, codebook,
                                        period_one_divisor: int, beta1: float, beta2: float, lr: float,
                                        bias_correction_1: float, bias_correction_2: float, eps: float) -> None:
    """Period-1 tensors: per-element second moment, one magnitude per `period_one_divisor`
    elements (reference wrapper :252-388)."""
    require_cuda_tensors({"p": p, "grad_flat": grad_flat, "m_sign": m_sign, "m_magnitude": m_magnitude,
                          "vmean": vmean, "codebook": codebook})
    if grad_flat.dim() != 1:
        raise ValueError("Expected grad_flat to be 1D, got dim={}".format(grad_flat.dim()))
    if grad_flat.dtype != p.dtype:
        raise ValueError("Expected grad_flat dtype {} to match p dtype {}.".format(grad_flat.dtype, p.dtype))
    if not isinstance(period_one_divisor, int) or period_one_divisor <= 0:
        raise ValueError("Expected period_one_divisor to be a positive int, got {}".format(period_one_divisor))
    total = grad_flat.numel()
    if total % period_one_divisor != 0:
        raise ValueError("Expected period_one_divisor {} to divide grad_flat.numel()={}.".format(
            period_one_divisor, total))
    require_block_column("m_magnitude", m_magnitude)
    require_block_column("vmean", vmean)
    if m_magnitude.shape[0] != total // period_one_divisor:
        raise ValueError("Expected m_magnitude to have {} rows, got {}.".format(
            total // period_one_divisor, m_magnitude.shape[0]))
    if vmean.shape[0] != total:
        raise ValueError("Expected vmean to have one row per element.")
    require_state_dtype("m_magnitude", m_magnitude)
    require_state_dtype("vmean", vmean)
    require_codebook(codebook)
    require_index_count(m_sign, total, False)
    if p.numel() != total:
        raise ValueError("Expected p.numel() to match grad_flat.numel().")
    if bias_correction_1 <= 0.0:
        raise ValueError("Expected bias_correction_1 to be positive, got {}".format(bias_correction_1))
    if bias_correction_2 <= 0.0:
        raise ValueError("Expected bias_correction_2 to be positive, got {}".format(bias_correction_2))
    if eps < 0.0:
        raise ValueError("Expected eps to be non-negative, got {}".format(eps))
    grad_flat = grad_flat.contiguous()
    codebook = codebook.contiguous()
    require_contiguous({"p": p, "m_sign": m_sign, "m_magnitude": m_magnitude, "vmean": vmean})
    with _lib.device_guard(p.device):
        _lib.check(_lib.load().gefen_b200_automatic_gefen_period1_update(
            _lib.ptr(p), _lib.ptr(grad_flat), _lib.dtype_tag(p.dtype), _lib.ptr(m_sign), _lib.ptr(m_magnitude),
            _lib.dtype_tag(m_magnitude.dtype), _lib.ptr(vmean), _lib.dtype_tag(vmean.dtype), _lib.ptr(codebook),
            codebook.numel(), _ws(codebook), total, period_one_divisor, float(beta1), float(beta2), float(lr),
            float(bias_correction_1), float(bias_correction_2), float(eps), _lib.current_stream(p.device)))


def automatic_gefen_muon_momentum_cuda(grad_view, m_sign, m_magnitude, codebook, momentum_update,
                                       packed_indices: bool, beta1: float) -> None:
    """GefenMuon's quantised momentum: writes the dequantised new momentum into `momentum_update`
    (reference wrapper :391-489)."""
    require_cuda_tensors({"grad_view": grad_view, "m_sign": m_sign, "m_magnitude": m_magnitude,
                          "codebook": codebook, "momentum_update": momentum_update})
    if grad_view.dim() != 2:
        raise ValueError("Expected grad_view to be 2D, got dim={}".format(grad_view.dim()))
    if momentum_update.shape != grad_view.shape:
        raise ValueError("Expected momentum_update shape {} to match grad_view shape {}.".format(
            tuple(momentum_update.shape), tuple(grad_view.shape)))
    if momentum_update.dtype != grad_view.dtype:
        raise ValueError("Expected momentum_update dtype {} to match grad_view dtype {}.".format(
            momentum_update.dtype, grad_view.dtype))
    require_block_column("m_magnitude", m_magnitude)
    if grad_view.shape[0] != m_magnitude.shape[0]:
        raise ValueError("Expected grad_view and m_magnitude to have the same number of blocks.")
    require_state_dtype("m_magnitude", m_magnitude)
    require_codebook(codebook)
    require_index_count(m_sign, grad_view.numel(), packed_indices)
    if not 0.0 <= beta1 <= 1.0:
        raise ValueError("Expected beta1 to be in [0, 1], got {}".format(beta1))
    grad_view = grad_view.contiguous()
    codebook = codebook.contiguous()
    require_contiguous({"m_sign": m_sign, "m_magnitude": m_magnitude, "momentum_update": momentum_update})
    with _lib.device_guard(grad_view.device):
        _lib.check(_lib.load().gefen_b200_automatic_gefen_muon_momentum(
            _lib.ptr(grad_view), _lib.dtype_tag(grad_view.dtype), _lib.ptr(m_sign), _lib.ptr(m_magnitude),
            _lib.dtype_tag(m_magnitude.dtype), _lib.ptr(codebook), codebook.numel(), _ws(codebook),
            _lib.ptr(momentum_update), int(bool(packed_indices)), grad_view.shape[0], grad_view.shape[1],
            float(beta1), _lib.current_stream(grad_view.device)))
