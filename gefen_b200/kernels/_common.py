"""Argument checks shared by the kernel wrappers."""
from __future__ import annotations

import torch

STATE_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def require_cuda_tensors(tensors: dict) -> None:
    for name, tensor in tensors.items():
        if not isinstance(tensor, torch.Tensor):
            raise TypeError("Expected {} to be a torch.Tensor.".format(name))
        if tensor.device.type != "cuda":
            raise ValueError("Expected {} to be on CUDA, got device {}.".format(name, tensor.device))


def require_contiguous(tensors: dict) -> None:
    for name, tensor in tensors.items():
        if not tensor.is_contiguous():
            raise ValueError("Expected {} to be contiguous.".format(name))


def require_state_dtype(name: str, tensor: torch.Tensor) -> None:
    if tensor.dtype not in STATE_DTYPES:
        raise ValueError("Expected {} to be float32, float16, or bfloat16, got {}".format(name, tensor.dtype))


def require_block_column(name: str, tensor: torch.Tensor) -> None:
    if tensor.dim() != 2 or tensor.shape[1] != 1:
        raise ValueError("Expected {} to have shape [num_blocks, 1], got {}".format(name, tuple(tensor.shape)))


def require_codebook(codebook: torch.Tensor) -> None:
    if codebook.dtype != torch.float32:
        raise ValueError("Expected codebook to be float32, got {}".format(codebook.dtype))
    if codebook.numel() > 256 or codebook.numel() < 1:
        raise ValueError("Expected codebook to have between 1 and 256 entries, got {}".format(codebook.numel()))


def require_index_count(m_sign: torch.Tensor, numel: int, packed_indices: bool) -> None:
    if m_sign.dtype != torch.uint8:
        raise ValueError("Expected m_sign to be uint8, got {}".format(m_sign.dtype))
    expected = (numel + 1) // 2 if packed_indices else numel
    if m_sign.numel() != expected:
        raise ValueError("Expected {} m_sign.numel()={} for grad_view.numel()={}, got {}.".format(
            "packed" if packed_indices else "unpacked", expected, numel, m_sign.numel()))
