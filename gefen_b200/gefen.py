"""`Gefen`: drop-in for the reference optimizer class (reference: gefen.py:435-1420) whose step,
calibration and state layout are reproduced while every piece of device work goes through the
sm_100a kernels of libgefen_b200.so.

State per parameter (same keys, shapes and dtypes as the reference, so checkpoints interchange):
  automatic_period:int, step:int, m_codebook_shape:tuple, m_codebook: uint8 [nb, period],
  m_magnitude: state dtype [nb, 1] (period 1: [numel / period_one_divisor, 1]),
  vmean: state dtype [nb, 1] (period 1: [numel, 1]), period_one_divisor:int (period 1 only).
state_dict() adds "gefen_global_step" and "gefen_codebook".

`fused=True` (default) runs the whole step as a handful of multi-tensor launches that fuse the
second-moment update, the decoupled weight decay and the 8-bit momentum step. `fused=False` keeps
the reference's launch structure (one second-moment launch, one weight-decay multiply and one step
launch per tensor) on the same kernels; there is no CPU path.
"""
from __future__ import annotations

from itertools import chain
from typing import Iterable, Optional, Tuple, Union

import numpy as np
import torch
import torch.nn as nn

from . import _lib
from . import partitioning
from . import quantization

F_FP32 = False              # force fp32 optimizer state regardless of the gradient dtype (reference :18, :53-69)
NUM_CODEBOOK_ENTRIES = 256  # reference :937
HISTOGRAM_BINS = NUM_CODEBOOK_ENTRIES * 16  # reference :329
PERIOD_ONE_MAX_DIVISOR = 256  # reference :622-623


def automatic_partition_view(flat_tensor: torch.Tensor, period: int) -> torch.Tensor:
    """[numel] -> [numel / period, period] (reference :21-39)."""
    if flat_tensor.dim() != 1:
        raise ValueError("Automatic partition view expects a 1D tensor, got dim={}".format(flat_tensor.dim()))
    if period <= 0:
        raise ValueError("Automatic partition period must be positive, got {}".format(period))
    if flat_tensor.numel() % period != 0:
        raise ValueError("Automatic partition expects numel {} to be divisible by period {}".format(
            flat_tensor.numel(), period))
    return flat_tensor.view(-1, period)


def gefen_state_dtype_from_grad(grad_view: torch.Tensor) -> torch.dtype:
    """Optimizer-state dtype follows the gradient dtype unless F_FP32 (reference :53-69)."""
    force_fp32 = globals().get("F_FP32", False)
    if not isinstance(force_fp32, bool):
        raise TypeError("F_FP32 must be a bool, got {}".format(type(force_fp32).__name__))
    if force_fp32 or grad_view.dtype == torch.float32:
        return torch.float32
    if grad_view.dtype in (torch.float16, torch.bfloat16):
        return grad_view.dtype
    raise ValueError("Gefen state dtype is undefined for gradient dtype {}".format(grad_view.dtype))


def largest_divisor_at_most(value: int, limit: int) -> int:
    """reference :72-82"""
    if value <= 0:
        raise ValueError("Expected value to be positive, got {}".format(value))
    if limit <= 0:
        raise ValueError("Expected limit to be positive, got {}".format(limit))
    if value <= limit:
        return value
    found = partitioning.divisors(value, max_divisor=limit)
    if not found:
        raise ValueError("Could not find a positive divisor for value {}".format(value))
    return found[-1]


def _local(tensor, what: str) -> torch.Tensor:
    """DTensor / async-collective unwrapping by duck typing (reference :692-706)."""
    if hasattr(tensor, "to_local"):
        tensor = tensor.to_local()
    if hasattr(tensor, "wait"):
        tensor = tensor.wait()
    if not isinstance(tensor, torch.Tensor):
        raise TypeError("Expected {} to resolve to a torch.Tensor, got {}.".format(what, type(tensor)))
    return tensor


def learn_gefen_exact_codebook_from_grad_periods(*, grad_periods, codebook_device: torch.device,
                                                 num_codebooks: int, force_endpoints: bool,
                                                 verbose: bool = False) -> Optional[torch.Tensor]:
    """One global codebook from the gradients of all tensors (reference :305-419).

    Each tensor's exact int64 histogram is produced on the GPU into its own row; the rows are
    fetched with one copy and accumulated on the host in float32 in parameter order, which is the
    reference's arithmetic (:331, :347). The codebook is then the exact-DP fit of the active bins.
    """
    items = [(flat, period) for _, flat, period, _ in grad_periods]
    if not items:
        return None
    from .kernels.exact_histogram_fused import gefen_exact_histogram_cuda

    bins = num_codebooks * 16
    device = items[0][0].device
    rows = torch.zeros((len(items), bins), dtype=torch.int64, device=device)
    for row, (flat, period) in zip(rows, items):
        gefen_exact_histogram_cuda(flat, period, row)
    rows_host = rows.cpu()
    bin_counts = torch.zeros(bins, dtype=torch.float32)
    for row in rows_host:
        bin_counts.add_(row.to(torch.float32))

    edges = torch.linspace(-1.0, 1.0, steps=bins + 1, dtype=torch.float32)
    centers = 0.5 * (edges[:-1] + edges[1:])
    active = bin_counts > 0
    stats = {
        "bin_edges": edges,
        "bin_centers": centers,
        "bin_counts": bin_counts,
        "active_bins": active,
        "active_centers": centers[active],
        "active_counts": bin_counts[active],
        "active_sums": centers[active] * bin_counts[active],
    }
    if verbose:
        print("Gefen exact codebook: {} tensors, {} active bins".format(len(items), int(active.sum())))
    codebook = quantization.exact_dp(stats, num_codebooks, force_endpoints, device=device)
    return codebook.to(codebook_device)


class _StepPlan:
    """Cached launch tables of one optimizer: one numpy table per parameter dtype, rows ordered by
    kernel class so that each class is one launch."""

    def __init__(self):
        self.key = None
        self.tables = []  # list of dicts: dtype_tag, rows (np structured), entries, device_table


class Gefen(torch.optim.Optimizer):
    def __init__(
        self,
        params: Iterable[Union[nn.Parameter, Tuple[str, nn.Parameter]]],
        lr: Union[float, torch.Tensor] = 1e-3,
        betas: Tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 0.0,
        *,
        fused: bool = True,
        verbose: bool = False,
    ):
        def validate(g_lr, g_betas, g_eps, g_wd):
            if not 0.0 <= g_lr:
                raise ValueError("Invalid learning rate: {}".format(g_lr))
            if not 0.0 <= g_betas[0] < 1.0:
                raise ValueError("Invalid beta parameter at index 0: {}".format(g_betas[0]))
            if not 0.0 <= g_betas[1] < 1.0:
                raise ValueError("Invalid beta parameter at index 1: {}".format(g_betas[1]))
            if not 0.0 <= g_wd:
                raise ValueError("Invalid weight_decay value: {}".format(g_wd))
            if not 0.0 <= g_eps:
                raise ValueError("Invalid epsilon value: {}".format(g_eps))

        validate(lr, betas, eps, weight_decay)

        def named(group_params):
            if isinstance(group_params, torch.Tensor):
                yield None, group_params
                return
            for item in group_params:
                name, param = item if isinstance(item, tuple) else (None, item)
                if not isinstance(param, torch.Tensor):
                    raise TypeError("Gefen can only optimize Tensors, but one of the params is {}".format(
                        type(param).__name__))
                yield name, param

        # One param group per parameter, names lower-cased, frozen parameters dropped (reference :503-565).
        groups = []

        def add(name, param, g_lr, g_betas, g_eps, g_wd):
            if not param.requires_grad:
                return
            groups.append({"name": str(name).lower(), "params": param, "lr": g_lr, "beta1": g_betas[0],
                           "beta2": g_betas[1], "eps": g_eps, "weight_decay": g_wd})

        for gi, entry in enumerate(params):
            if isinstance(entry, dict):
                if "params" not in entry:
                    raise ValueError("Gefen parameter group {} is missing the 'params' key.".format(gi))
                g_lr = entry.get("lr", lr)
                g_betas = entry.get("betas", betas)
                g_eps = entry.get("eps", eps)
                g_wd = entry.get("weight_decay", weight_decay)
                validate(g_lr, g_betas, g_eps, g_wd)
                for pi, (name, param) in enumerate(named(entry["params"])):
                    add("group_{}_param_{}".format(gi, pi) if name is None else name, param, g_lr, g_betas, g_eps, g_wd)
            else:
                for name, param in named((entry,)):
                    add("param_{}".format(gi) if name is None else name, param, lr, betas, eps, weight_decay)

        self.fused = bool(fused)
        self.verbose = verbose
        self._gefen_codebook = None
        self._gefen_global_step = 0
        self._plan = _StepPlan()
        self._plans = {}
        self._steady = None
        if verbose:
            print("Initializing Gefen optimizer (fused={}).".format(self.fused))
        super().__init__(groups, dict(lr=lr, beta1=betas[0], beta2=betas[1], eps=eps))

    # ------------------------------------------------------------------ calibration
    def _gefen_codebook_device(self) -> torch.device:
        for group in self.param_groups:
            for p in group["params"]:
                return p.grad.device if p.grad is not None else p.device
        raise ValueError("Expected at least one parameter when choosing the Gefen codebook device.")

    def _period_one_divisor_for_numel(self, numel: int) -> int:
        return largest_divisor_at_most(numel, PERIOD_ONE_MAX_DIVISOR)

    def _period_one_divisor_from_state(self, state, total_numel: int) -> int:
        """reference :625-658"""
        d = state.get("period_one_divisor")
        if d is None:
            d = self._period_one_divisor_for_numel(total_numel)
            state["period_one_divisor"] = d
        elif not isinstance(d, int):
            raise TypeError("period_one_divisor must be an int, got {}".format(type(d).__name__))
        elif d <= 0:
            raise ValueError("period_one_divisor must be positive, got {}".format(d))
        elif total_numel % d != 0:
            raise ValueError("period_one_divisor {} must divide flattened tensor numel {}".format(d, total_numel))
        mag = state.get("m_magnitude")
        if torch.is_tensor(mag) and mag.shape != (total_numel // d, 1):
            raise ValueError("Expected m_magnitude shape {} for period_one_divisor {}, got {}".format(
                (total_numel // d, 1), d, tuple(mag.shape)))
        return d

    def _predict_periods(self, todo):
        """todo: list of (name, param, grad). Scores every tensor's candidate periods on the GPU,
        then fetches all scores with one copy and applies the integer rule (reference :765-828 and
        partitioning.py:225-347, without the per-divisor synchronisation)."""
        launched = []
        for name, p, grad in todo:
            if grad.device.type != "cuda":
                raise ValueError("gefen_b200 needs CUDA gradients, got device {} for {}".format(grad.device, name))
            launched.append(partitioning.launch_period_scores(grad, input_is_squared=False))
        stats = [s for _, _, s, _ in launched if s is not None]
        host = torch.cat(stats, dim=0).cpu() if stats else None
        periods, cursor = [], 0
        for n, cand, s, _ in launched:
            if s is None:
                periods.append(1)
                continue
            periods.append(partitioning.decide_period(n, cand, host[cursor:cursor + len(cand)]))
            cursor += len(cand)
        return periods

    def _iter_gefen_grad_periods(self, reuse_existing_periods: bool = False):
        """(name, flat grad, period, grad) for every parameter with a non-empty gradient; fixes
        state["automatic_period"] on the way (reference :882-924)."""
        found, todo = [], []
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = _local(p.grad, "gradient {}".format(group["name"])).detach()
                flat = grad.reshape(-1)
                if flat.numel() == 0:
                    continue
                state = self.state[p]
                if reuse_existing_periods:
                    if "automatic_period" not in state:
                        raise ValueError(
                            "Expected automatic_period to exist for {} before refreshing Gefen codebook at "
                            "optimizer step {}".format(group["name"], self._gefen_global_step))
                    period = state["automatic_period"]
                elif flat.numel() == 1:
                    period = 1
                else:
                    period = None
                    todo.append((group["name"], p, grad))
                found.append([group["name"], p, flat, period, grad])
        if todo:
            predicted = iter(self._predict_periods(todo))
            for item in found:
                if item[3] is None:
                    item[3] = next(predicted)
        for name, p, flat, period, grad in found:
            self.state[p]["automatic_period"] = period
            if flat.numel() % period != 0:
                raise ValueError(
                    "Automatic partition period {} does not divide parameter {} with numel {} while learning "
                    "Gefen codebook".format(period, name, flat.numel()))
            if self.verbose:
                print("Gefen shared-v:", name, "| shape=", tuple(p.shape), "| numel=", p.numel(),
                      "| automatic period=", period)
            yield name, flat, period, grad

    def _learn_gefen_exact_codebook(self, reuse_existing_periods: bool = False) -> Optional[torch.Tensor]:
        return learn_gefen_exact_codebook_from_grad_periods(
            grad_periods=self._iter_gefen_grad_periods(reuse_existing_periods=reuse_existing_periods),
            codebook_device=self._gefen_codebook_device(),
            num_codebooks=NUM_CODEBOOK_ENTRIES,
            force_endpoints=True,
            verbose=self.verbose,
        )

    def _has_restored_automatic_periods(self) -> bool:
        return any("automatic_period" in self.state.get(p, {}) for g in self.param_groups for p in g["params"])

    def _maybe_refresh_gefen_codebook(self) -> None:
        """Learns the codebook on the first step, or after a restore that carried periods but no
        codebook; otherwise only follows the parameters' device (reference :969-980)."""
        if self._gefen_codebook is not None:
            device = self._gefen_codebook_device()
            if self._gefen_codebook.device != device:
                self._gefen_codebook = self._gefen_codebook.to(device)
            return
        codebook = self._learn_gefen_exact_codebook(reuse_existing_periods=self._has_restored_automatic_periods())
        if codebook is not None:
            self._gefen_codebook = codebook.contiguous()

    # ------------------------------------------------------------------ state
    def _init_gefen_state(self, state, grad_view: torch.Tensor) -> None:
        """reference :1039-1062"""
        state["m_codebook_shape"] = tuple(grad_view.shape)
        state["m_codebook"] = torch.zeros(grad_view.shape, dtype=torch.uint8, device=grad_view.device)
        state_dtype = gefen_state_dtype_from_grad(grad_view)
        if grad_view.shape[1] == 1:
            d = self._period_one_divisor_for_numel(grad_view.numel())
            state["period_one_divisor"] = d
            rows = grad_view.numel() // d
        elif grad_view.shape[1] > 1:
            rows = grad_view.shape[0]
        else:
            raise ValueError("Expected grad_view second dimension to be positive, got {}".format(grad_view.shape[1]))
        state["m_magnitude"] = torch.zeros((rows, 1), dtype=state_dtype, device=grad_view.device)

    def _ensure_state(self, name: str, p, local_p: torch.Tensor, grad: torch.Tensor, with_vmean: bool = True):
        """First visit of a parameter (reference :1232-1268)."""
        state = self.state[p]
        if "step" in state:
            return state
        numel = grad.numel()
        if "automatic_period" in state:
            period = state["automatic_period"]
        elif numel == 1:
            period = 1
        else:
            period = self._predict_periods([(name, p, grad)])[0]
        if numel % period != 0:
            raise ValueError("Automatic partition period {} does not divide local shard of parameter {} with numel {}"
                             .format(period, name, numel))
        state["automatic_period"] = period
        state["step"] = 0
        grad_view = automatic_partition_view(grad.reshape(-1), period)
        self._init_gefen_state(state, grad_view)
        if with_vmean:
            state["vmean"] = torch.zeros((grad_view.shape[0], 1), dtype=gefen_state_dtype_from_grad(grad_view),
                                         device=grad_view.device)
        return state

    # ------------------------------------------------------------------ step, per-tensor launches
    def _step_automatic(self, group, name: str, p, grad) -> None:
        """The reference's launch structure on this library's kernels (reference :1208-1322)."""
        from .kernels.automatic_gefen_fused import (
            automatic_gefen_fused_update_from_vmean_cuda,
            automatic_gefen_period1_update_cuda,
        )
        from .kernels.automatic_vmean import automatic_vmean_update_cuda

        local_p = _local(p, "parameter {}".format(name))
        grad = _local(grad, "gradient {}".format(name))
        flat_grad = grad.reshape(-1)
        if local_p.numel() != flat_grad.numel():
            raise ValueError("Local parameter shard numel {} does not match local gradient numel {} for {}.".format(
                local_p.numel(), flat_grad.numel(), name))
        if flat_grad.numel() == 0:
            return
        state = self._ensure_state(name, p, local_p, grad)
        period = state["automatic_period"]
        grad_view = automatic_partition_view(flat_grad, period)
        beta1, beta2, lr, eps = group["beta1"], group["beta2"], group["lr"], group["eps"]
        if period != 1:
            automatic_vmean_update_cuda(state["vmean"], grad_view, beta2)
        state["step"] += 1
        if group["weight_decay"] > 0.0:
            local_p.mul_(1 - lr * group["weight_decay"])
        bc1 = 1 - beta1 ** state["step"]
        bc2 = 1 - beta2 ** state["step"]
        fused_p = self._contiguous_param(p, local_p, name)
        if period == 1:
            automatic_gefen_period1_update_cuda(
                fused_p, flat_grad, state["m_codebook"], state["m_magnitude"], state["vmean"], self._gefen_codebook,
                self._period_one_divisor_from_state(state, flat_grad.numel()), beta1, beta2, float(lr), bc1, bc2, eps)
        else:
            automatic_gefen_fused_update_from_vmean_cuda(
                fused_p, grad_view, state["m_codebook"], state["m_magnitude"], state["vmean"], self._gefen_codebook,
                False, beta1, float(lr), bc1, bc2, eps)
        if fused_p is not local_p:
            local_p.copy_(fused_p)

    @staticmethod
    def _contiguous_param(p, local_p: torch.Tensor, name: str) -> torch.Tensor:
        """reference :1287-1297: only DTensor shards may be non-contiguous."""
        if local_p.is_contiguous():
            return local_p
        if hasattr(p, "to_local") and hasattr(p, "placements"):
            return local_p.contiguous()
        raise ValueError("Gefen fused update requires a contiguous parameter tensor for {}.".format(name))

    # ------------------------------------------------------------------ step, multi-tensor launches
    def _collect(self):
        """(group, name, p, local_p, grad) for every parameter that takes part in this step."""
        work = []
        for group in self.param_groups:
            name = group["name"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                local_p = _local(p, "parameter {}".format(name))
                grad = _local(p.grad, "gradient {}".format(name))
                if local_p.numel() != grad.numel():
                    raise ValueError("Local parameter shard numel {} does not match local gradient numel {} for {}."
                                     .format(local_p.numel(), grad.numel(), name))
                if grad.numel() == 0:
                    continue
                if grad.dtype != local_p.dtype:
                    raise ValueError("Expected grad_view dtype {} to match p dtype {}.".format(grad.dtype, local_p.dtype))
                if grad.device.type != "cuda":
                    raise ValueError("gefen_b200 needs CUDA tensors, got device {} for {}".format(grad.device, name))
                work.append((group, name, p, local_p, grad))
        return work

    def _step_tables(self, work, muon: bool = False, ranges=None):
        """Builds (or reuses) the launch tables for `work`. Static columns are cached; the pointer
        and scalar columns are refreshed by the caller every step. ranges: {id(param): (first block, end
        block)} restricts a tensor's row to a run of its blocks (blocks are independent of each other)."""
        key = (muon,) + tuple((id(item[2]),) + tuple((ranges or {}).get(id(item[2]), ())) for item in work)
        plan = self._plans.get(key)
        if plan is not None:
            self._plan = plan
            return plan.tables
        if len(self._plans) >= 512:   # callers that keep changing the set of tensors: start over
            self._plans.clear()
        plan = self._plans[key] = self._plan = _StepPlan()
        lib = _lib.load()
        by_dtype = {}
        for idx, (group, name, p, local_p, grad) in enumerate(work):
            by_dtype.setdefault((grad.dtype, grad.device), []).append(idx)
        tables = []
        for (dtype, device), idxs in by_dtype.items():
            tag = _lib.dtype_tag(dtype)
            rows = np.zeros(len(idxs), dtype=_lib.STEP_TENSOR_DTYPE)
            for r, idx in enumerate(idxs):
                group, name, p, local_p, grad = work[idx]
                state = self.state[p]
                period = state["automatic_period"]
                numel = grad.numel()
                flags = 0
                if muon:
                    flags |= _lib.STEP_MUON
                    block = self._period_one_divisor_from_state(state, numel) if period == 1 else period
                elif period == 1:
                    flags |= _lib.STEP_PERIOD1
                    block = self._period_one_divisor_from_state(state, numel)
                else:
                    flags |= _lib.STEP_FUSE_VMEAN
                    block = period
                b0, b1 = (ranges or {}).get(id(p), (0, numel // block))
                if (b0, b1) != (0, numel // block) and (period == 1 or muon):
                    raise ValueError("block ranges are for Gefen tensors with a period above 1, got {}".format(name))
                state_bytes = state["m_magnitude"].element_size()
                rows[r]["codes"] = state["m_codebook"].data_ptr() + b0 * block
                rows[r]["mag"] = state["m_magnitude"].data_ptr() + b0 * state_bytes
                rows[r]["mag_dtype"] = _lib.dtype_tag(state["m_magnitude"].dtype)
                if muon:
                    rows[r]["v_dtype"] = _lib.F32
                else:
                    rows[r]["v"] = state["vmean"].data_ptr() + (b0 * state["vmean"].element_size() if period != 1 else 0)
                    rows[r]["v_dtype"] = _lib.dtype_tag(state["vmean"].dtype)
                rows[r]["period"] = block
                rows[r]["num_blocks"] = b1 - b0
                rows[r]["flags"] = flags
                rows[r]["p"] = local_p.data_ptr() + b0 * block * local_p.element_size()
                rows[r]["g"] = grad.data_ptr() + b0 * block * grad.element_size()
            classes = [lib.gefen_b200_step_tensor_class(rows[r:r + 1].ctypes.data, tag) for r in range(len(idxs))]
            order = sorted(range(len(idxs)), key=lambda r: classes[r])
            rows = np.ascontiguousarray(rows[order])
            tables.append({
                "tag": tag,
                "device": device,
                "rows": rows,
                "static_flags": rows["flags"].copy(),
                "entries": [idxs[r] for r in order],
                "classes": [classes[r] for r in order],
                # byte offset of each row's first element in its tensor (0 unless a block range was given)
                "offsets": [int((ranges or {}).get(id(work[idxs[r]][2]), (0, 0))[0]) * int(rows[i]["period"])
                            for i, r in enumerate(order)],
                "device_table": torch.empty(rows.nbytes, dtype=torch.uint8, device=device),
            })
        plan.key = key
        plan.tables = tables
        return tables

    def _step_multi_tensor(self, only=None, ranges=None, advance=None) -> None:
        """One multi-tensor launch per dtype and kernel class over every parameter with a gradient,
        or over those whose id() is in `only` (callers that stream the model through in pieces). Such a
        caller may also cut a tensor into runs of blocks: ranges = {id(param): (first block, end block)}
        steps only those blocks, and `advance` (a set of ids) names the tensors whose step counter moves
        in this call (the call that takes a tensor's first run); the other runs of the same optimizer step
        use the counter as that call left it."""
        if only is None and ranges is None and advance is None and self._steady is not None:
            if self._gefen_codebook is not None and self._step_steady():
                return
        work = self._collect()
        if only is not None:
            work = [item for item in work if id(item[2]) in only]
        if not work:
            return
        if self._gefen_codebook is None:
            raise ValueError("Expected Gefen codebook to be initialized before fused update.")
        copies = []
        for i, (group, name, p, local_p, grad) in enumerate(work):
            self._ensure_state(name, p, local_p, grad)
            fused_p = self._contiguous_param(p, local_p, name)
            if not grad.is_contiguous():
                grad = grad.contiguous()
            if fused_p is not local_p:
                copies.append((local_p, fused_p))
            work[i] = (group, name, p, fused_p, grad)
        ws = _lib.codebook_workspace(self._gefen_codebook)
        tables = self._step_tables(work, ranges=ranges)
        for table in tables:
            rows = table["rows"]
            n = len(table["entries"])
            cols = {k: [0.0] * n for k in ("beta1", "beta2", "lr", "bc1", "bc2", "eps", "wd_mul")}
            p_ptr, g_ptr, flags = [0] * n, [0] * n, table["static_flags"].copy()
            for r, idx in enumerate(table["entries"]):
                group, name, p, fused_p, grad = work[idx]
                state = self.state[p]
                if advance is None or id(p) in advance:
                    state["step"] += 1
                beta1, beta2, lr, wd = group["beta1"], group["beta2"], float(group["lr"]), group["weight_decay"]
                cols["beta1"][r] = beta1
                cols["beta2"][r] = beta2
                cols["lr"][r] = lr
                cols["bc1"][r] = 1 - beta1 ** state["step"]
                cols["bc2"][r] = 1 - beta2 ** state["step"]
                cols["eps"][r] = group["eps"]
                if wd > 0.0:
                    cols["wd_mul"][r] = 1 - lr * wd
                    flags[r] |= _lib.STEP_WEIGHT_DECAY
                else:
                    cols["wd_mul"][r] = 1.0
                p_ptr[r] = fused_p.data_ptr() + table["offsets"][r] * fused_p.element_size()
                g_ptr[r] = grad.data_ptr() + table["offsets"][r] * grad.element_size()
            for k, v in cols.items():
                rows[k] = v
            rows["p"] = p_ptr
            rows["g"] = g_ptr
            rows["flags"] = flags
            self._launch_table(table, ws)
        for local_p, fused_p in copies:
            local_p.copy_(fused_p)
        # A whole step over plain contiguous tensors: remember what the next call can reuse as it is.
        self._steady = None
        if only is None and ranges is None and advance is None and not copies and \
                all(type(item[2].grad) is torch.Tensor and not hasattr(item[2], "to_local") for item in work):
            in_plan = {id(item[2]) for item in work}
            self._steady = {
                "codebook": self._gefen_codebook,
                "n_groups": len(self.param_groups),
                "n_params": sum(len(g["params"]) for g in self.param_groups),
                "idle": [p for g in self.param_groups for p in g["params"] if id(p) not in in_plan],
                "tables": [(table, [(work[idx][2], self.state[work[idx][2]], work[idx][0], int(table["rows"]["g"][r]),
                                     int(table["rows"]["p"][r]), work[idx][4].numel(), work[idx][4].dtype)
                                    for r, idx in enumerate(table["entries"])])
                           for table in tables],
            }

    def _step_steady(self) -> bool:
        """The step of a training loop in its steady state: the same tensors at the same addresses as in the
        previous call, so only the step counters and the scalars derived from them change. Checks exactly
        that first (and returns False, having changed nothing, if anything differs)."""
        st = self._steady
        if st["codebook"] is not self._gefen_codebook or st["n_groups"] != len(self.param_groups) or \
                st["n_params"] != sum(len(g["params"]) for g in self.param_groups):
            return False
        for p in st["idle"]:
            if p.grad is not None:
                return False
        for table, items in st["tables"]:
            for p, state, group, g_ptr, p_ptr, numel, dtype in items:
                g = p.grad
                if g is None or type(g) is not torch.Tensor or g.data_ptr() != g_ptr or p.data_ptr() != p_ptr or \
                        g.numel() != numel or g.dtype != dtype or not g.is_contiguous() or not p.is_contiguous():
                    return False
        ws = _lib.codebook_workspace(self._gefen_codebook)
        memo = {}
        for table, items in st["tables"]:
            vals = []
            for p, state, group, g_ptr, p_ptr, numel, dtype in items:
                step = state["step"] + 1
                state["step"] = step
                key = (group["beta1"], group["beta2"], float(group["lr"]), group["weight_decay"], group["eps"], step)
                v = memo.get(key)
                if v is None:
                    beta1, beta2, lr, wd, eps, _ = key
                    v = memo[key] = (beta1, beta2, lr, 1 - beta1 ** step, 1 - beta2 ** step, eps,
                                     (1 - lr * wd) if wd > 0.0 else 1.0, 1.0 if wd > 0.0 else 0.0)
                vals.append(v)
            cols = np.array(vals, dtype=np.float64)
            rows = table["rows"]
            for c, k in enumerate(("beta1", "beta2", "lr", "bc1", "bc2", "eps", "wd_mul")):
                rows[k] = cols[:, c]
            rows["flags"] = table["static_flags"] | (cols[:, 7].astype(table["static_flags"].dtype) * _lib.STEP_WEIGHT_DECAY)
            self._launch_table(table, ws)
        return True

    def _launch_table(self, table, ws) -> None:
        """One multi-tensor call of the library for a filled table (one launch per kernel class in it)."""
        lib = _lib.load()
        rows = table["rows"]
        n = len(table["entries"])
        device = table["device"]
        # set by a ZeRO-1 wrapper whose parameter and gradient buffers are mapped between the ranks'
        # GPUs: byte distances to the peers' parameter copies, which the kernels then store to as
        # well, and to all ranks' gradient buffers, which the kernels then average themselves
        peers = getattr(self, "_peer_param_deltas", None)
        grad_srcs = getattr(self, "_grad_src_deltas", None)
        with _lib.device_guard(device):
            if (peers is not None and len(peers)) or (grad_srcs is not None and len(grad_srcs)):
                n_peers = 0 if peers is None else len(peers)
                n_srcs = 0 if grad_srcs is None else len(grad_srcs)
                # multicast (NVSwitch) addresses of the same buffers, where the wrapper found them
                param_mc = int(getattr(self, "_param_multicast_delta", 0) or 0) if n_peers else 0
                grad_mc = int(getattr(self, "_grad_multicast_delta", 0) or 0) if n_srcs else 0
                _lib.check(lib.gefen_b200_multi_tensor_step_multicast(
                    rows.ctypes.data, _lib.ptr(table["device_table"]), n, table["tag"], _lib.ptr(ws),
                    peers.ctypes.data if n_peers else None, n_peers,
                    grad_srcs.ctypes.data if n_srcs else None, n_srcs, float(getattr(self, "_grad_src_scale", 1.0)),
                    param_mc, grad_mc, _lib.current_stream(device)))
            else:
                _lib.check(lib.gefen_b200_multi_tensor_step(
                    rows.ctypes.data, _lib.ptr(table["device_table"]), n, table["tag"], _lib.ptr(ws),
                    _lib.current_stream(device)))

    def check(self) -> None:
        """Raises if a kernel of an earlier step gave up one of its bounded waits, which leaves that
        step incomplete (synchronises the devices of the parameters). The kernels never trap or spin
        for ever; this is where such a time-out becomes an exception. No counterpart in the reference,
        whose kernels wait on nothing."""
        devices = {p.device for g in self.param_groups for p in g["params"] if p.device.type == "cuda"}
        for device in devices:
            _lib.check_step_status(device)

    def _optimizer_state_memory_bytes(self) -> int:
        return sum(v.numel() * v.element_size() for s in self.state.values() for v in s.values() if torch.is_tensor(v))

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        """torch's dict plus the global step and the codebook (reference :1343-1349)."""
        self.check()   # a checkpoint of a half-done step must not look like a good one
        sd = super().state_dict()
        sd["gefen_global_step"] = self._gefen_global_step
        sd["gefen_codebook"] = self._gefen_codebook
        return sd

    def load_state_dict(self, state_dict):
        """Restores and then undoes torch's dtype cast of the state tensors, which would turn the
        uint8 codes and low-precision scalars into the parameter dtype (reference :1351-1397)."""
        state_dict = dict(state_dict)
        global_step = state_dict.pop("gefen_global_step", 0)
        codebook = state_dict.pop("gefen_codebook", None)
        saved_state = state_dict.get("state", {}) or {}
        super().load_state_dict(state_dict)
        self._gefen_global_step = global_step
        self._gefen_codebook = codebook
        self._plan = _StepPlan()
        self._plans = {}
        self._steady = None
        id_map = dict(zip(chain.from_iterable(g["params"] for g in state_dict["param_groups"]),
                          chain.from_iterable(g["params"] for g in self.param_groups)))
        for param_id, saved in saved_state.items():
            param = id_map.get(param_id)
            live = self.state.get(param) if param is not None else None
            if live is None:
                continue
            for key, value in saved.items():
                if not torch.is_tensor(value):
                    continue
                cur = live.get(key)
                if torch.is_tensor(cur) and cur.dtype == value.dtype:
                    continue
                device = cur.device if torch.is_tensor(cur) else param.device
                live[key] = value.to(device=device, dtype=value.dtype)

    # ------------------------------------------------------------------ public step
    @torch.no_grad()
    def step(self, closure=None):
        """Calibrates before running the closure, like the reference (:1399-1420)."""
        self._maybe_refresh_gefen_codebook()
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.fused:
            self._step_multi_tensor()
        else:
            for group in self.param_groups:
                for p in group["params"]:
                    if p.grad is not None:
                        self._step_automatic(group, group["name"], p, p.grad)
        self._gefen_global_step += 1
        return loss
