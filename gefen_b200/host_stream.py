"""Gefen step for models whose gradients arrive in, and whose parameters return to, pinned host
memory every step (optimizer state and a working copy of the parameters stay on the GPU).

The reference optimizer only sees tensors where they already live (gefen.py:1399-1420); moving them is
its caller's business, done whole: all gradients in, step, all parameters out. Here the model is cut
into buckets of consecutive parameters and three streams work on different buckets at once:

    copy-in stream   : gradients of bucket k+1  host -> device
    compute stream   : Gefen step of bucket k    (one multi-tensor launch per dtype and kernel class)
    copy-out stream  : parameters of bucket k-1 device -> host

PCIe carries both directions at the same time, so a step costs about one direction's transfer instead
of two plus the kernels. The arithmetic is the optimizer's own (`Gefen._step_multi_tensor` on a subset),
so results are identical to `Gefen.step()` on the same gradients.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .gefen import Gefen


class HostStreamedGefen:
    """optimizer: a `Gefen(fused=True)` over CUDA parameters that have `.grad` tensors allocated.
    host_grads / host_params: pinned host tensors, one per optimizer parameter, in the order of
    `optimizer.param_groups` (same shapes and dtypes)."""

    def __init__(self, optimizer: Gefen, host_grads: Sequence[torch.Tensor], host_params: Sequence[torch.Tensor],
                 buckets: int = 8):
        if not isinstance(optimizer, Gefen) or not optimizer.fused:
            raise ValueError("HostStreamedGefen needs a Gefen optimizer with fused=True")
        self.opt = optimizer
        self.params: List[torch.nn.Parameter] = [p for g in optimizer.param_groups for p in g["params"]]
        if len(host_grads) != len(self.params) or len(host_params) != len(self.params):
            raise ValueError("Expected one host gradient and one host parameter buffer per optimizer parameter")
        for p, hg, hp in zip(self.params, host_grads, host_params):
            if p.device.type != "cuda" or p.grad is None:
                raise ValueError("Every parameter must be a CUDA tensor with an allocated .grad")
            if hg.shape != p.shape or hp.shape != p.shape or hg.dtype != p.dtype or hp.dtype != p.dtype:
                raise ValueError("Host buffers must match their parameter's shape and dtype")
            if not (hg.is_pinned() and hp.is_pinned()):
                raise ValueError("Host buffers must be pinned (page-locked) memory")
        self.host_grads = list(host_grads)
        self.host_params = list(host_params)
        self.device = self.params[0].device
        # consecutive parameters, about equal bytes per bucket
        total = sum(p.numel() * p.element_size() for p in self.params)
        target = max(1, total // max(1, buckets))
        self.buckets: List[List[int]] = [[]]
        acc = 0
        for i, p in enumerate(self.params):
            if acc >= target and len(self.buckets) < buckets:
                self.buckets.append([])
                acc = 0
            self.buckets[-1].append(i)
            acc += p.numel() * p.element_size()
        self._ids = [set(id(self.params[i]) for i in b) for b in self.buckets]
        self._in = torch.cuda.Stream(self.device)
        self._out = torch.cuda.Stream(self.device)

    def _copy_in(self, bucket: List[int]) -> None:
        for i in bucket:
            self.params[i].grad.copy_(self.host_grads[i], non_blocking=True)

    def _copy_out(self, bucket: List[int]) -> None:
        for i in bucket:
            self.host_params[i].copy_(self.params[i].detach(), non_blocking=True)

    @torch.no_grad()
    def step(self) -> None:
        """One optimizer step. Returns with all work enqueued; the current stream is made to wait for
        the last copy-out, so an event recorded on it afterwards covers the whole step."""
        opt = self.opt
        cur = torch.cuda.current_stream(self.device)
        if opt._gefen_codebook is None:
            # the calibrating step needs every gradient at once: whole model in, step, whole model out
            for b in self.buckets:
                self._copy_in(b)
            opt.step()
            for b in self.buckets:
                self._copy_out(b)
            return
        opt._maybe_refresh_gefen_codebook()
        start = torch.cuda.Event()
        start.record(cur)
        self._in.wait_event(start)      # gradients of the previous step have been consumed
        self._out.wait_event(start)
        arrived = []
        with torch.cuda.stream(self._in):
            for b in self.buckets:
                self._copy_in(b)
                e = torch.cuda.Event()
                e.record(self._in)
                arrived.append(e)
        for k, b in enumerate(self.buckets):
            cur.wait_event(arrived[k])
            opt._step_multi_tensor(only=self._ids[k])
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self._out):
                self._out.wait_event(done)
                self._copy_out(b)
        opt._gefen_global_step += 1
        finished = torch.cuda.Event()
        finished.record(self._out)
        cur.wait_event(finished)
