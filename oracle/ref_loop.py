"""TEST INFRASTRUCTURE - the reference's optimizer loop restated on the CPU oracle kernels.

`OracleGefen` walks the same sequence as the reference's fused (CUDA) path, one tensor at a time:
calibration before the first step (period per tensor, global histogram, exact-DP codebook;
reference gefen.py:969-980, :882-946), then per step and tensor: second-moment update, step
counter, decoupled weight decay in the parameter dtype, bias corrections in Python doubles and
the fused kernel (reference gefen.py:1270-1322). `OracleGefenMuon` does the same for
gefen_muon.py:216-329 with torch's CPU matmuls for Newton-Schulz.
Tensors live on the CPU; parameters are plain tensors with a `.grad` attribute set by the caller.
"""
from __future__ import annotations

import math

import torch

from . import oracle as O


def state_dtype(grad: torch.Tensor) -> torch.dtype:
    return grad.dtype if grad.dtype in (torch.float16, torch.bfloat16) else torch.float32


def largest_divisor_at_most(value: int, limit: int) -> int:
    if value <= limit:
        return value
    return O.divisors(value, max_divisor=limit)[-1]


class OracleGefen:
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        self.params = list(params)
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.state = [dict() for _ in self.params]
        self.codebook = None

    def calibrate(self, grads):
        items = []
        for st, g in zip(self.state, grads):
            flat = g.reshape(-1)
            if "automatic_period" not in st:
                st["automatic_period"] = 1 if flat.numel() == 1 else O.find_period(g, cuda_kernel_semantics=True)
            items.append((flat, st["automatic_period"]))
        self.codebook = O.learn_codebook(items)

    def _init_state(self, st, g):
        period = st["automatic_period"]
        n = g.numel()
        nb = n // period
        st["step"] = 0
        st["m_codebook"] = torch.zeros(nb, period, dtype=torch.uint8)
        sd = state_dtype(g)
        if period == 1:
            st["period_one_divisor"] = largest_divisor_at_most(n, 256)
            st["m_magnitude"] = torch.zeros(n // st["period_one_divisor"], 1, dtype=sd)
        else:
            st["m_magnitude"] = torch.zeros(nb, 1, dtype=sd)
        st["vmean"] = torch.zeros(nb, 1, dtype=sd)

    def step(self, grads):
        if self.codebook is None:
            self.calibrate(grads)
        beta1, beta2 = self.betas
        for p, st, g in zip(self.params, self.state, grads):
            if "step" not in st:
                self._init_state(st, g)
            period = st["automatic_period"]
            flat = g.reshape(-1).contiguous()
            gv = flat.view(-1, period)
            if period != 1:
                O.automatic_vmean_update(st["vmean"], gv, beta2)
            st["step"] += 1
            if self.wd > 0.0:
                O.weight_decay(p, self.lr, self.wd)
            bc1 = 1 - beta1 ** st["step"]
            bc2 = 1 - beta2 ** st["step"]
            if period == 1:
                O.automatic_gefen_period1_update(p, flat, st["m_codebook"], st["m_magnitude"], st["vmean"],
                                                 self.codebook, st["period_one_divisor"], beta1, beta2, self.lr,
                                                 bc1, bc2, self.eps)
            else:
                O.automatic_gefen_fused_update_from_vmean(p, gv, st["m_codebook"], st["m_magnitude"], st["vmean"],
                                                          self.codebook, False, beta1, self.lr, bc1, bc2, self.eps)


def newton_schulz(update: torch.Tensor, coefficients=(3.4445, -4.7750, 2.0315), steps=5, eps=1e-7) -> torch.Tensor:
    """reference: gefen_muon.py:16-51"""
    a, b, c = coefficients
    x = update.bfloat16()
    transposed = update.size(0) > update.size(1)
    if transposed:
        x = x.T
    x = x / x.norm().clamp(min=eps)
    for _ in range(steps):
        gram = x @ x.T
        gram_update = torch.addmm(gram, gram, gram, beta=b, alpha=c)
        x = torch.addmm(x, gram_update, x, beta=a)
    return x.T if transposed else x


class OracleGefenMuon(OracleGefen):
    def __init__(self, params, lr=1e-3, weight_decay=0.1, momentum=0.95, nesterov=True,
                 ns_coefficients=(3.4445, -4.7750, 2.0315), eps=1e-7, ns_steps=5):
        super().__init__(params, lr=lr, betas=(momentum, 0.0), eps=eps, weight_decay=weight_decay)
        self.momentum, self.nesterov = momentum, nesterov
        self.ns_coefficients, self.ns_steps = ns_coefficients, ns_steps

    def step(self, grads):
        if self.codebook is None:
            self.calibrate(grads)
        for p, st, g in zip(self.params, self.state, grads):
            if "step" not in st:
                self._init_state(st, g)
                del st["vmean"]
            period = st["automatic_period"]
            block = st["period_one_divisor"] if period == 1 else period
            gv = g.reshape(-1, block).contiguous()
            mom = torch.empty_like(gv)
            O.automatic_gefen_muon_momentum(gv, st["m_codebook"].view(-1, block), st["m_magnitude"], self.codebook,
                                            mom, False, self.momentum)
            st["step"] += 1
            if self.nesterov:
                mom.mul_(self.momentum).add_(gv, alpha=1 - self.momentum)
            update = newton_schulz(mom.view_as(g), self.ns_coefficients, self.ns_steps, self.eps)
            rows, cols = p.shape[:2]
            adjusted = self.lr * math.sqrt(max(1, rows / cols))
            if self.wd > 0.0:
                p.mul_(1 - self.lr * self.wd)
            p.add_(update, alpha=-adjusted)
