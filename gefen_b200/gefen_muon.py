"""`GefenMuon`: Muon with Gefen's 8-bit quantised momentum (reference: gefen_muon.py:1-350).

Per 2-D parameter and step: dequantise the momentum, m <- beta*m + (1-beta)*g, re-encode it (the
same block kernel as Gefen, writing the dequantised new momentum), Nesterov blend, Newton-Schulz
orthogonalisation in bf16, decoupled weight decay and the update with the shape-adjusted learning
rate. The momentum kernel runs once for all matrices of a chunk (one multi-tensor launch, Nesterov
fused); Newton-Schulz and the apply run per matrix.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional, Tuple, Union

import numpy as np
import torch
import torch.nn as nn

from . import _lib
from .gefen import Gefen
from .newton_schulz import orthogonalize_all

EPS = 1e-7
DEFAULT_A = 3.4445
DEFAULT_B = -4.7750
DEFAULT_C = 2.0315
DEFAULT_NS_STEPS = 5
MOMENTUM_CHUNK_ELEMENTS = 1 << 28   # dense momentum scratch held at a time (elements of the parameter dtype)


def _adjust_lr(lr: float, adjust_lr_fn: Optional[str], param_shape) -> float:
    """reference: gefen_muon.py:54-67"""
    if isinstance(lr, torch.Tensor):
        lr = lr.item()
    rows, cols = param_shape[:2]
    if adjust_lr_fn is None or adjust_lr_fn == "original":
        ratio = math.sqrt(max(1, rows / cols))
    elif adjust_lr_fn == "match_rms_adamw":
        ratio = 0.2 * math.sqrt(max(rows, cols))
    else:
        ratio = 1.0
    return lr * ratio


class GefenMuon(Gefen):
    def __init__(
        self,
        params: Iterable[Union[nn.Parameter, Tuple[str, nn.Parameter]]],
        lr: Union[float, torch.Tensor] = 1e-3,
        weight_decay: float = 0.1,
        momentum: float = 0.95,
        nesterov: bool = True,
        ns_coefficients: Tuple[float, float, float] = (DEFAULT_A, DEFAULT_B, DEFAULT_C),
        eps: float = EPS,
        ns_steps: int = DEFAULT_NS_STEPS,
        adjust_lr_fn: Optional[str] = None,
        *,
        fused: bool = True,
        verbose: bool = False,
    ) -> None:
        if isinstance(lr, torch.Tensor) and lr.numel() != 1:
            raise ValueError("Tensor lr must be 1-element")
        if not 0.0 <= lr:
            raise ValueError("Learning rate should be >= 0 but is: {}".format(lr))
        if not 0.0 <= momentum:
            raise ValueError("momentum should be >= 0 but is: {}".format(momentum))
        if not 0.0 <= weight_decay:
            raise ValueError("weight decay should be >= 0 but is: {}".format(weight_decay))
        if adjust_lr_fn is not None and adjust_lr_fn not in ("original", "match_rms_adamw"):
            raise ValueError("Adjust learning rate function {} is not supported".format(adjust_lr_fn))
        super().__init__(params, lr=lr, betas=(momentum, 0.0), eps=eps, weight_decay=weight_decay, fused=fused,
                         verbose=verbose)
        for group in self.param_groups:
            group["momentum"] = momentum
            group["nesterov"] = nesterov
            group["ns_coefficients"] = ns_coefficients
            group["ns_steps"] = ns_steps
            group["adjust_lr_fn"] = adjust_lr_fn
            for p in group["params"]:
                if p.ndim != 2:
                    raise ValueError("GefenMuon only supports 2D parameters whereas we found a parameter with size: {}"
                                     .format(p.size()))
        self._scratch = None

    # ------------------------------------------------------------------ momentum
    def _momentum_scratch(self, numel: int, dtype, device) -> torch.Tensor:
        if (self._scratch is None or self._scratch.numel() < numel or self._scratch.dtype != dtype
                or self._scratch.device != device):
            self._scratch = torch.empty(numel, dtype=dtype, device=device)
        return self._scratch

    def _device_table(self, nbytes: int, device) -> torch.Tensor:
        """Device copy of the launch table, kept between steps (work on one stream is ordered)."""
        t = getattr(self, "_table", None)
        if t is None or t.numel() < nbytes or t.device != device:
            t = self._table = torch.empty(max(nbytes, 4096), dtype=torch.uint8, device=device)
        return t

    def check(self) -> None:
        """As `Gefen.check`, and also raises if a Newton-Schulz GEMM gave up one of its bounded waits."""
        super().check()
        from . import newton_schulz

        for device in {p.device for g in self.param_groups for p in g["params"] if p.device.type == "cuda"}:
            newton_schulz.check_status(device)

    def _quantized_momentum(self, chunk, scratch: torch.Tensor):
        """One multi-tensor launch: new 8-bit momentum for every matrix of `chunk`, its dequantised
        value (Nesterov-blended when asked) written into consecutive slices of `scratch`."""
        lib = _lib.load()
        rows = np.zeros(len(chunk), dtype=_lib.STEP_TENSOR_DTYPE)
        outs, offset = [], 0
        for r, (group, name, p, local_p, grad) in enumerate(chunk):
            state = self.state[p]
            period = state["automatic_period"]
            numel = grad.numel()
            block = self._period_one_divisor_from_state(state, numel) if period == 1 else period
            out = scratch[offset:offset + numel].view(grad.shape)
            offset += (numel + 7) // 8 * 8
            outs.append(out)
            momentum = group["momentum"]
            flags = _lib.STEP_MUON | (_lib.STEP_NESTEROV if group["nesterov"] else 0)
            rows[r]["p"], rows[r]["g"] = out.data_ptr(), grad.data_ptr()
            rows[r]["codes"], rows[r]["mag"] = state["m_codebook"].data_ptr(), state["m_magnitude"].data_ptr()
            rows[r]["mag_dtype"] = _lib.dtype_tag(state["m_magnitude"].dtype)
            rows[r]["v_dtype"] = _lib.F32
            rows[r]["period"], rows[r]["num_blocks"] = block, numel // block
            rows[r]["beta1"] = momentum
            rows[r]["beta2"] = 1 - momentum      # alpha of the Nesterov add_, rounded from the double
            rows[r]["bc1"] = rows[r]["bc2"] = rows[r]["wd_mul"] = 1.0
            rows[r]["flags"] = flags
            state["step"] += 1
        tag = _lib.dtype_tag(chunk[0][4].dtype)
        classes = [lib.gefen_b200_step_tensor_class(rows[r:r + 1].ctypes.data, tag) for r in range(len(chunk))]
        order = sorted(range(len(chunk)), key=lambda r: classes[r])
        rows = np.ascontiguousarray(rows[order])
        device = chunk[0][4].device
        table = self._device_table(rows.nbytes, device)
        ws = _lib.codebook_workspace(self._gefen_codebook)
        with _lib.device_guard(device):
            _lib.check(lib.gefen_b200_multi_tensor_step(rows.ctypes.data, _lib.ptr(table), len(chunk), tag, _lib.ptr(ws),
                                                        _lib.current_stream(device)))
        return outs

    # ------------------------------------------------------------------ step
    def _step_muon(self) -> None:
        work = self._collect()
        if not work:
            return
        if self._gefen_codebook is None:
            raise ValueError("Expected Gefen codebook to be initialized before fused GefenMuon update.")
        for i, (group, name, p, local_p, grad) in enumerate(work):
            if torch.is_complex(local_p):
                raise RuntimeError("GefenMuon does not support complex parameters")
            if grad.is_sparse:
                raise RuntimeError("GefenMuon does not support sparse gradients")
            if grad.ndim != 2:
                raise ValueError("GefenMuon gradient must be a 2D matrix for {}".format(name))
            self._ensure_state(name, p, local_p, grad, with_vmean=False)
            if not grad.is_contiguous():
                work[i] = (group, name, p, local_p, grad.contiguous())
        # chunks bound the dense scratch; inside a chunk all tensors share dtype and device
        chunks, cur, cur_elems = [], [], 0
        for item in work:
            n = (item[4].numel() + 7) // 8 * 8
            same = not cur or (cur[0][4].dtype == item[4].dtype and cur[0][4].device == item[4].device)
            if cur and (cur_elems + n > MOMENTUM_CHUNK_ELEMENTS or not same):
                chunks.append(cur)
                cur, cur_elems = [], 0
            cur.append(item)
            cur_elems += n
        if cur:
            chunks.append(cur)
        lib = _lib.load()
        for chunk in chunks:
            total = sum((it[4].numel() + 7) // 8 * 8 for it in chunk)
            scratch = self._momentum_scratch(total, chunk[0][4].dtype, chunk[0][4].device)
            outs = self._quantized_momentum(chunk, scratch)

            peers = getattr(self, "_peer_param_deltas", None)
            n_peers = 0 if peers is None else len(peers)

            def apply(i, ortho):
                # decoupled weight decay and the update (reference: gefen_muon.py:325-329), one kernel; for a
                # ZeRO-1 rank it also stores the updated matrix into the other ranks' parameter buffers
                group, name, p, local_p, grad = chunk[i]
                lr = group["lr"]
                adjusted_lr = _adjust_lr(lr, group["adjust_lr_fn"], p.shape)
                wd_mul = 1 - float(lr) * group["weight_decay"] if group["weight_decay"] > 0.0 else 1.0
                if ortho.dtype != local_p.dtype or not local_p.is_contiguous():
                    if wd_mul != 1.0:
                        local_p.mul_(wd_mul)
                    local_p.add_(ortho, alpha=-adjusted_lr)
                    return
                if not ortho.is_contiguous():
                    ortho = ortho.contiguous()
                with _lib.device_guard(local_p.device):
                    _lib.check(lib.gefen_b200_muon_apply(
                        _lib.ptr(local_p), _lib.ptr(ortho), _lib.dtype_tag(local_p.dtype), local_p.numel(), wd_mul,
                        -adjusted_lr, peers.ctypes.data if n_peers else None, n_peers, _lib.current_stream(local_p.device)))

            orthogonalize_all([(update, group["ns_coefficients"], group["ns_steps"], group["eps"])
                               for (group, name, p, local_p, grad), update in zip(chunk, outs)], apply)

    @torch.no_grad()
    def step(self, closure=None):
        """The closure runs before calibration here, unlike Gefen.step (reference: gefen_muon.py:331-350)."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._maybe_refresh_gefen_codebook()
        self._step_muon()
        self._gefen_global_step += 1
        return loss
