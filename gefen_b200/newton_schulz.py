"""Newton-Schulz orthogonalisation used by GefenMuon (reference: gefen_muon.py:16-51).

X <- X / max(||X||_F, eps); then `steps` times: A = X X^T, B = b*A + c*A*A, X <- a*X + B*X, all in
bf16 with fp32 accumulation, on the wide orientation (rows <= cols; taller inputs are transposed).
Each product rounds its result to bf16 once, as the reference's torch.addmm / `@` calls do.

The products run on the library's tcgen05 GEMM (`gefen_b200_ns_gemm_tn`, K-major operands). Keeping
X and X^T side by side makes every product of the iteration K-major: the third GEMM writes its
result in both orientations. Shapes the kernel does not take (a dimension that is not a multiple
of 8) use torch's GEMMs.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import _lib

_STATUS = {}
USE_TCGEN05 = os.environ.get("GEFEN_B200_NS", "tcgen05") != "torch"


_SCRATCH = {}


def _scratch(device, numel: int) -> torch.Tensor:
    """Per-device bf16 scratch for the iteration (Gram matrix, polynomial, second iterate), grown on demand.
    Work on one stream is ordered, so successive matrices can share it."""
    t = _SCRATCH.get(device.index)
    if t is None or t.numel() < numel:
        t = torch.empty(numel, dtype=torch.bfloat16, device=device)
        _SCRATCH[device.index] = t
    return t[:numel]


def _status(device) -> torch.Tensor:
    t = _STATUS.get(device.index)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device.index] = t
    return t


def check_status(device) -> None:
    """Raises if a bounded wait inside a GEMM kernel ran out since the last check (synchronises)."""
    t = _STATUS.get(device.index)
    if t is not None and int(t.item()) != 0:
        t.zero_()
        raise _lib.GefenB200Error("a tcgen05 GEMM gave up waiting on one of its barriers; results are incomplete")


def gemm_tn(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
            out: Optional[torch.Tensor] = None, out_t: Optional[torch.Tensor] = None, symmetric: bool = False) -> torch.Tensor:
    """out[M,N] = alpha * a[M,K] @ b[N,K]^T + beta * c[M,N]; out_t[N,M] = out^T if given. bf16, row-major.
    symmetric=True promises a symmetric result (a is b, c symmetric): half of the tiles are computed."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    for t in (a, b, c, out, out_t):
        if t is not None and (t.dtype != torch.bfloat16 or t.stride(-1) != 1):
            raise ValueError("gemm_tn expects bf16 matrices with unit inner stride")
    with _lib.device_guard(a.device):
        _lib.check(_lib.load().gefen_b200_ns_gemm_tn(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.ptr(out), _lib.ptr(out_t), M, N, K, a.stride(0), b.stride(0),
            0 if c is None else c.stride(0), out.stride(0), 0 if out_t is None else out_t.stride(0), float(alpha),
            float(beta), int(symmetric), _lib.ptr(_status(a.device)), _lib.current_stream(a.device)))
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M,N] = alpha * a[M,K] @ b[K,N] + beta * c[M,N]. bf16, row-major."""
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    for t in (a, b, c, out):
        if t is not None and (t.dtype != torch.bfloat16 or t.stride(-1) != 1):
            raise ValueError("gemm_nn expects bf16 matrices with unit inner stride")
    with _lib.device_guard(a.device):
        _lib.check(_lib.load().gefen_b200_ns_gemm_nn(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0),
            0 if c is None else c.stride(0), out.stride(0), float(alpha), float(beta), _lib.ptr(_status(a.device)),
            _lib.current_stream(a.device)))
    return out


def gemm_tt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, symmetric: bool = False) -> torch.Tensor:
    """out[M,N] = a[K,M]^T @ b[K,N]. bf16, row-major."""
    K, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    with _lib.device_guard(a.device):
        _lib.check(_lib.load().gefen_b200_ns_gemm_tt(
            _lib.ptr(a), _lib.ptr(b), None, _lib.ptr(out), M, N, K, a.stride(0), b.stride(0), 0, out.stride(0), 1.0, 0.0,
            int(symmetric), _lib.ptr(_status(a.device)), _lib.current_stream(a.device)))
    return out


def _supported(m: int, n: int) -> bool:
    return USE_TCGEN05 and m % 8 == 0 and n % 8 == 0


def zeropower_via_newtonschulz(grad: torch.Tensor, ns_coefficients: Tuple[float, float, float], ns_steps: int,
                               eps: float) -> torch.Tensor:
    if ns_steps >= 100:
        raise ValueError("Number of steps must be less than 100 for computational efficiency")
    if len(grad.shape) != 2:
        raise ValueError("Input tensor gradient must be a 2D matrix")
    if len(ns_coefficients) != 3:
        raise ValueError("Coefficients must be a tuple of exactly 3 values")
    if grad.device.type != "cuda":
        raise ValueError("gefen_b200 runs Newton-Schulz on the GPU only, got device {}".format(grad.device))
    a, b, c = ns_coefficients
    x = grad.bfloat16()
    rows, cols = x.shape
    if not _supported(rows, cols) or ns_steps == 0:
        transposed = rows > cols
        if transposed:
            x = x.T
        x = x / x.norm().clamp(min=eps)
        for _ in range(ns_steps):
            gram = x @ x.T
            gram_update = torch.addmm(gram, gram, gram, beta=b, alpha=c)
            x = torch.addmm(x, gram_update, x, beta=a)
        return x.T if transposed else x

    # bf16 norm and quotient, as the reference's div_ (the Frobenius norm does not care about orientation).
    # Both iterates live in the per-device scratch: the same addresses for every matrix of a shape, which
    # lets the native driver replay the chain of products as one graph.
    m = min(rows, cols)
    scratch = _scratch(x.device, 2 * m * m + 2 * rows * cols)
    gram = scratch[: m * m]
    poly = scratch[m * m: 2 * m * m]
    nxt = scratch[2 * m * m: 2 * m * m + rows * cols].view(rows, cols)
    first = scratch[2 * m * m + rows * cols: 2 * m * m + 2 * rows * cols].view(rows, cols)
    x = torch.div(x, x.norm().clamp(min=eps), out=first)
    with _lib.device_guard(x.device):
        _lib.check(_lib.load().gefen_b200_newton_schulz(
            _lib.ptr(x), _lib.ptr(nxt), _lib.ptr(gram), _lib.ptr(poly), rows, cols, int(ns_steps), float(a), float(b),
            float(c), _lib.ptr(_status(x.device)), _lib.current_stream(x.device)))
    return (x if ns_steps % 2 == 0 else nxt).clone()
