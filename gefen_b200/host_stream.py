"""Gefen step for models whose gradients arrive in, and whose parameters return to, pinned host
memory every step (optimizer state and a working copy of the parameters stay on the GPU).

The reference optimizer only sees tensors where they already live (gefen.py:1399-1420); moving them is
its caller's business, done whole: all gradients in, step, all parameters out. Here the model is cut
into buckets of about equal bytes (consecutive parameters; a large tensor is cut between blocks, which
the step treats independently) and three streams work on different buckets at once:

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


def cut_buckets(numels, element_sizes, periods, n_buckets, weights=None):
    """Cuts a model, in parameter order, into at most `n_buckets` runs of about equal bytes (or, with
    `weights`, of bytes in proportion to one weight per bucket). A tensor larger than what is left of a bucket
    is cut at a block boundary (the blocks of a tensor are independent in the step), so that no bucket is much
    larger than its share. Period-1 tensors (tiny) stay whole.
    Returns a list of buckets; a bucket is a list of (parameter index, first block, end block, whole
    tensor?) in which a parameter appears at most once."""
    sizes = [n * e for n, e in zip(numels, element_sizes)]
    n_buckets = max(1, n_buckets)
    if weights is None:
        weights = [1.0] * n_buckets
    targets = [max(1, int(sum(sizes) * w / sum(weights))) for w in weights]
    buckets, cur, room = [], [], targets[0]
    for i, (numel, esize, period) in enumerate(zip(numels, element_sizes, periods)):
        nb = numel // period if period > 1 else 1
        block_bytes = (period if period > 1 else numel) * esize
        b0 = 0
        while b0 < nb:
            last = len(buckets) >= n_buckets - 1        # the last bucket takes all that is left
            fit = nb if (period <= 1 or last) else max(1, -(-room // block_bytes))   # rounds up: the bucket closes
            b1 = min(nb, b0 + fit)
            if period > 1 and nb - b1 < max(1, nb // 64):   # do not leave a sliver for the next bucket
                b1 = nb
            cur.append((i, b0, b1, b0 == 0 and b1 == nb))
            room -= (b1 - b0) * block_bytes
            b0 = b1
            if room <= 0 and not last:
                buckets.append(cur)
                cur, room = [], targets[len(buckets)]
    if cur:
        buckets.append(cur)
    return buckets


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
        self.n_buckets = max(1, int(buckets))
        self.buckets = None          # built after calibration: the cut points are block boundaries
        self._in = torch.cuda.Stream(self.device)
        self._out = torch.cuda.Stream(self.device)

    def _build_buckets(self) -> None:
        periods = [int(self.opt.state[p]["automatic_period"]) for p in self.params]
        # The first bucket's copy-in and the last bucket's copy-out are the parts of a step that nothing
        # overlaps: the buckets at both ends are small (1/8, 1/4, 1/2 of the others).
        n = self.n_buckets
        ramp = [0.125, 0.25, 0.5]
        weights = ramp + [1.0] * (n - 6) + ramp[::-1] if n >= 8 else None
        self.buckets = cut_buckets([p.numel() for p in self.params], [p.element_size() for p in self.params],
                                   periods, n, weights)
        buckets = self.buckets
        self._ids = [set(id(self.params[i]) for i, _, _, _ in b) for b in buckets]
        self._ranges = [{id(self.params[i]): (b0, b1) for i, b0, b1, whole in b if not whole} for b in buckets]
        self._advance = [set(id(self.params[i]) for i, b0, _, _ in b if b0 == 0) for b in buckets]

    def _span(self, i: int, b0: int, b1: int, whole: bool):
        if whole:
            return slice(None)
        period = int(self.opt.state[self.params[i]]["automatic_period"])
        return slice(b0 * period, b1 * period)

    def _copy_in(self, bucket) -> None:
        for i, b0, b1, whole in bucket:
            span = self._span(i, b0, b1, whole)
            self.params[i].grad.view(-1)[span].copy_(self.host_grads[i].view(-1)[span], non_blocking=True)

    def _copy_out(self, bucket) -> None:
        for i, b0, b1, whole in bucket:
            span = self._span(i, b0, b1, whole)
            self.host_params[i].view(-1)[span].copy_(self.params[i].detach().view(-1)[span], non_blocking=True)

    @torch.no_grad()
    def step(self) -> None:
        """One optimizer step. Returns with all work enqueued; the current stream is made to wait for
        the last copy-out, so an event recorded on it afterwards covers the whole step."""
        opt = self.opt
        cur = torch.cuda.current_stream(self.device)
        if opt._gefen_codebook is None:
            # the calibrating step needs every gradient at once: whole model in, step, whole model out
            for p, hg in zip(self.params, self.host_grads):
                p.grad.copy_(hg, non_blocking=True)
            opt.step()
            for p, hp in zip(self.params, self.host_params):
                hp.copy_(p.detach(), non_blocking=True)
            return
        if self.buckets is None:
            self._build_buckets()
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
            opt._step_multi_tensor(only=self._ids[k], ranges=self._ranges[k], advance=self._advance[k])
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self._out):
                self._out.wait_event(done)
                self._copy_out(b)
        opt._gefen_global_step += 1
        finished = torch.cuda.Event()
        finished.record(self._out)
        cur.wait_event(finished)
