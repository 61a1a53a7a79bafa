"""Seeded synthetic inputs shaped like the benchmark configurations: parameters ~ N(0, 0.02),
gradients ~ N(0, sigma) times a per-row log-normal scale that is fixed across steps (this gives
the block structure the period search looks for)."""
from __future__ import annotations

import torch


def generator(seed: int, tensor_index: int, step: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed * 1_000_000 + 1000 * tensor_index + step)
    return g


def row_scale(shape, seed: int, tensor_index: int, tau: float) -> torch.Tensor:
    g = generator(seed, tensor_index, 999)
    rows = shape[0] if len(shape) == 2 else 1
    return torch.exp(torch.randn(rows, 1, generator=g) * tau)


def make_grad(shape, seed: int, tensor_index: int, step: int, dtype=torch.float32, sigma: float = 1e-3,
              tau: float = 1.0) -> torch.Tensor:
    g = generator(seed, tensor_index, step)
    base = torch.randn(*shape, generator=g) * sigma
    scale = row_scale(shape, seed, tensor_index, tau)
    out = base * scale if len(shape) == 2 else base * scale.reshape(())
    return out.to(dtype)


def make_param(shape, seed: int, tensor_index: int, dtype=torch.float32) -> torch.Tensor:
    g = generator(seed, tensor_index, 998)
    return (torch.randn(*shape, generator=g) * 0.02).to(dtype)


def reference_like_codebook(seed: int = 0, k: int = 256) -> torch.Tensor:
    """A codebook of the shape the exact DP produces: sorted, endpoints -1/+1, dense around 0."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    inner = torch.sort(torch.tanh(torch.randn(k - 2, generator=g) * 0.6)).values
    return torch.cat([torch.tensor([-1.0]), inner, torch.tensor([1.0])]).float().contiguous()


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().reshape(-1)
    b = b.double().reshape(-1)
    denom = float(b.norm())
    return float((a - b).norm()) / (denom if denom > 0 else 1.0)
