"""Newton-Schulz orthogonalisation used by GefenMuon (reference: gefen_muon.py:16-51).

X <- X / max(||X||_F, eps); then `steps` times: A = X X^T, B = b*A + c*A*A, X <- a*X + B*X, all in
bf16 with fp32 accumulation, on the wide orientation (rows <= cols; taller inputs are transposed).
Each product rounds its result to bf16 once, as the reference's torch.addmm / `@` calls do.

The products run on the library's tcgen05 GEMMs (`gefen_b200_newton_schulz`: K-major and MN-major
operands, so no transposed copy is ever made). The kernels take dimensions that are multiples of 8
(16-byte rows); any other matrix is padded with zero rows and columns, which the iteration maps to
zero rows and columns (they add nothing to X X^T), and the result is cut back. There is no library
GEMM behind this module.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

_STATUS = {}


_SCRATCH = {}
LANES = 2   # matrices orthogonalised side by side (see `orthogonalize_all`)


def _scratch(device, numel: int, lane: int = 0) -> torch.Tensor:
    """Per-device, per-lane bf16 scratch for the iteration (Gram matrix, polynomial, both iterates), grown on
    demand. Work on one stream is ordered, so successive matrices of a lane can share it."""
    key = (device.index, lane)
    t = _SCRATCH.get(key)
    if t is None or t.numel() < numel:
        t = torch.empty(numel, dtype=torch.bfloat16, device=device)
        _SCRATCH[key] = t
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


def _newton_schulz_into_scratch(grad: torch.Tensor, ns_coefficients, ns_steps: int, eps: float, lane: int) -> torch.Tensor:
    """The iteration on the current stream; returns a VIEW of the lane's scratch that holds the result (valid
    until the lane's next matrix is enqueued)."""
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
    if rows == 0 or cols == 0:
        return x
    # bf16 norm and quotient, as the reference's div_ (the Frobenius norm does not care about orientation).
    # Both iterates live in the lane's scratch: the same addresses for every matrix of a shape, which lets
    # the native driver replay the chain of products as one graph.
    prow, pcol = (rows + 7) // 8 * 8, (cols + 7) // 8 * 8
    m = min(prow, pcol)
    scratch = _scratch(x.device, 2 * m * m + 2 * prow * pcol, lane)
    gram = scratch[: m * m]
    poly = scratch[m * m: 2 * m * m]
    nxt = scratch[2 * m * m: 2 * m * m + prow * pcol].view(prow, pcol)
    first = scratch[2 * m * m + prow * pcol: 2 * m * m + 2 * prow * pcol].view(prow, pcol)
    if (prow, pcol) != (rows, cols):
        first.zero_()
        nxt.zero_()
    torch.div(x, x.norm().clamp(min=eps), out=first[:rows, :cols])
    if ns_steps > 0:
        with _lib.device_guard(x.device):
            _lib.check(_lib.load().gefen_b200_newton_schulz(
                _lib.ptr(first), _lib.ptr(nxt), _lib.ptr(gram), _lib.ptr(poly), prow, pcol, int(ns_steps), float(a), float(b),
                float(c), _lib.ptr(_status(x.device)), _lib.current_stream(x.device)))
    result = first if ns_steps % 2 == 0 else nxt
    return result[:rows, :cols]


def zeropower_via_newtonschulz(grad: torch.Tensor, ns_coefficients: Tuple[float, float, float], ns_steps: int,
                               eps: float) -> torch.Tensor:
    """reference: gefen_muon.py:16-51. Returns a new tensor."""
    return _newton_schulz_into_scratch(grad, ns_coefficients, ns_steps, eps, 0).clone()


_LANE_STREAMS = {}


def _lane_streams(device):
    streams = _LANE_STREAMS.get(device.index)
    if streams is None:
        streams = _LANE_STREAMS[device.index] = [torch.cuda.Stream(device) for _ in range(LANES)]
    return streams


def orthogonalize_all(items, consume) -> None:
    """Newton-Schulz for many matrices, LANES of them side by side.

    items: list of (matrix, ns_coefficients, ns_steps, eps); consume(i, ortho) is called with the
    orthogonalised matrix i (a view of scratch memory: use it at once, on the current stream). The two
    symmetric products of an iteration have fewer output tiles than the GPU has SMs (72 tiles of 128 x 256
    for a 2048-row Gram matrix); running the chains of two matrices on two streams lets those launches
    share the SMs. Every lane stream starts after the work already on the caller's stream and the caller's
    stream waits for all lanes at the end, so to the caller this is one ordered piece of work."""
    if not items:
        return
    device = items[0][0].device
    cur = torch.cuda.current_stream(device)
    streams = _lane_streams(device)
    start = torch.cuda.Event()
    start.record(cur)
    for lane, stream in enumerate(streams):
        stream.wait_event(start)
    for i, (matrix, coefficients, steps, eps) in enumerate(items):
        lane = i % LANES
        with torch.cuda.stream(streams[lane]):
            consume(i, _newton_schulz_into_scratch(matrix, coefficients, steps, eps, lane))
    for stream in streams:
        done = torch.cuda.Event()
        done.record(stream)
        cur.wait_event(done)
