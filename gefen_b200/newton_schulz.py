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
            out: Optional[torch.Tensor] = None, out_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M,N] = alpha * a[M,K] @ b[N,K]^T + beta * c[M,N]; out_t[N,M] = out^T if given. bf16, row-major."""
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
            float(beta), _lib.ptr(_status(a.device)), _lib.current_stream(a.device)))
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
    transposed = grad.size(0) > grad.size(1)
    if transposed:
        x = x.T
    x = x / x.norm().clamp(min=eps)          # bf16 norm and quotient, as the reference's div_
    m, n = x.shape
    if not _supported(m, n) or ns_steps == 0:
        for _ in range(ns_steps):
            gram = x @ x.T
            gram_update = torch.addmm(gram, gram, gram, beta=b, alpha=c)
            x = torch.addmm(x, gram_update, x, beta=a)
        return x.T if transposed else x

    # wide X [m, n] and its transpose [n, m], both contiguous
    if transposed:
        xt = x.T.contiguous()       # the original orientation
        xw = x.contiguous()
    else:
        xw = x.contiguous()
        xt = x.T.contiguous()
    dev = x.device
    gram = torch.empty((m, m), dtype=torch.bfloat16, device=dev)
    poly = torch.empty((m, m), dtype=torch.bfloat16, device=dev)
    xw_next = torch.empty_like(xw)
    xt_next = torch.empty_like(xt)
    for _ in range(ns_steps):
        gemm_tn(xw, xw, out=gram)                                          # G = X X^T
        gemm_tn(gram, gram, c=gram, alpha=c, beta=b, out=poly)              # B = b G + c G G   (G symmetric)
        gemm_tn(poly, xt, c=xw, alpha=1.0, beta=a, out=xw_next, out_t=xt_next)   # X' = a X + B X, and X'^T
        xw, xw_next = xw_next, xw
        xt, xt_next = xt_next, xt
    return xt if transposed else xw
