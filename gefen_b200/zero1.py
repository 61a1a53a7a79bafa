"""ZeRO-1 style data parallelism around the Gefen step: every rank keeps the full parameters, owns
the optimizer state of one contiguous segment of a flat layout, and a step is

    reduce-scatter(gradients)  ->  Gefen step on the owned segment  ->  all-gather(parameters).

On NCCL the parameter and gradient buffers of all ranks are symmetric memory: mapped into every
process and, where the machine has NVSwitch multicast, bound to a multicast address as well. The step
kernels then carry both collectives on their own accesses while they compute. With multicast, a
gradient chunk arrives with one `multimem.ld_reduce` (the switch adds the ranks' copies) and an
updated parameter chunk leaves with one `multimem.st` (the switch delivers it to every copy): each
rank pulls 1/N of the gradient bytes and pushes 1/N of the parameter bytes that the unicast
collectives move, and the two directions of the links are busy at the same time inside one kernel.
Without multicast (two or three ranks, where the switch's loop back to the sender costs more than it saves)
the kernels store to every peer copy (plain peer stores), and the gradients reach their owners by
device-to-device copies: every rank pushes the segments it does not own into a receive buffer on their
owners, bucket by bucket on a side stream, and the step kernels sum the local copies in rank order while
they read them, taking bucket k while bucket k + 1 is on the wire. Where the receive buffer ((N-1)/N of one
buffer) does not fit, NCCL reduce-scatters the gradients first. One-element all-reduces order the ranks.

The reference has no communication code at all (its only distributed awareness is unwrapping
DTensor shards, gefen.py:692-706); this module is the exchange step the data-parallel use of the
optimizer needs. Two properties are kept so that N ranks reproduce one rank bit for bit on the state
and parameters of every piece, given the same reduced gradients and periods:
  * segments are cut at ROW boundaries of the 2-D tensors, so every partition block of the
    optimizer lives on exactly one rank whenever the period divides the row length (the periods
    that row-scaled gradients give). The reference picks a tensor's period from the divisors of its
    whole flattened length (partitioning.py:147, :253); a piece scores the divisors of ITS length, a
    smaller candidate set, so a split tensor can come out with another period than one process would
    choose. The largest piece decides, disagreements are kept in `period_mismatches` and a warning
    names them;
  * the codebook is fitted from the histogram of ALL tensors: per-piece int64 histograms are
    gathered, pieces of one tensor are added exactly, and tensors are accumulated in float32 in
    parameter order, which is the single-process arithmetic (reference: gefen.py:331-347).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

ALIGN = 8  # elements; keeps every piece 16-byte aligned for 2-byte dtypes


@dataclass
class Piece:
    tensor: int      # index into the parameter list
    row0: int        # first row of the tensor held by this piece (0 for 1-D tensors)
    rows: int        # number of rows (1 for 1-D tensors)
    cols: int        # elements per row (numel for 1-D tensors)
    rank: int        # owner
    offset: int      # element offset in the flat buffer

    @property
    def numel(self) -> int:
        return self.rows * self.cols


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatLayout:
    """Places tensors, in order, into `world` equal segments of one flat buffer. A tensor that does
    not fit in the rest of a segment is split between rows: its first piece is pushed against the
    end of the segment and the next piece starts the following segment, so the tensor stays one
    contiguous range of the buffer (the model's parameter is a plain view of it)."""

    def __init__(self, shapes: Sequence[Tuple[int, ...]], world: int):
        self.world = world
        self.shapes = [tuple(s) for s in shapes]
        dims = [(s[0], int(math.prod(s[1:]))) if len(s) >= 2 else (1, int(math.prod(s)) if len(s) else 1)
                for s in self.shapes]
        total = sum(r * c for r, c in dims)
        unit = ALIGN
        for r, c in dims:
            if r > 1 and r * c > total // max(world, 1):  # may cover a whole segment: rows must tile it
                unit = unit * c // math.gcd(unit, c)
        seg = _round_up(max(-(-total // world), 1), unit)
        while True:
            pieces = self._fill(dims, seg)
            if pieces is not None:
                break
            seg += unit
        self.segment = seg
        self.total = seg * world
        self.pieces: List[Piece] = pieces
        self.tensor_offset = [min(p.offset for p in pieces if p.tensor == t) for t in range(len(dims))]

    def _fill(self, dims, seg) -> Optional[List[Piece]]:
        """Sequential fill; returns None when `seg` is too small (the caller grows it)."""
        pieces, rank, fill = [], 0, 0
        for t, (rows, cols) in enumerate(dims):
            n = rows * cols
            start = _round_up(fill, ALIGN)
            if start + n <= seg:
                pieces.append(Piece(t, 0, rows, cols, rank, rank * seg + start))
                fill = start + n
                continue
            fit_rows = (seg - start) // cols if rows > 1 and start < seg else 0
            if fit_rows == 0:  # nothing of this tensor fits here: open the next segment
                rank, fill = rank + 1, 0
                if rank >= self.world:
                    return None
                if n <= seg:
                    pieces.append(Piece(t, 0, rows, cols, rank, rank * seg))
                    fill = n
                    continue
                if rows == 1:
                    return None
                fit_rows = seg // cols
                if fit_rows == 0:
                    return None
            # split between rows: the first piece is pushed against the end of this segment, middle
            # pieces fill their segments exactly, the last piece starts its segment
            pieces.append(Piece(t, 0, fit_rows, cols, rank, rank * seg + seg - fit_rows * cols))
            row0, left = fit_rows, rows - fit_rows
            while left > 0:
                rank += 1
                if rank >= self.world:
                    return None
                fit = seg // cols
                if left <= fit:
                    pieces.append(Piece(t, row0, left, cols, rank, rank * seg))
                    fill = left * cols
                    left = 0
                else:
                    if seg % cols != 0:
                        return None
                    pieces.append(Piece(t, row0, fit, cols, rank, rank * seg))
                    row0 += fit
                    left -= fit
        return pieces

    def owned(self, rank: int) -> List[Piece]:
        return [p for p in self.pieces if p.rank == rank]


class WholeTensorLayout:
    """Assigns WHOLE tensors to ranks (largest first, each to the least loaded rank) and places every
    rank's tensors, in parameter order, in its segment of the flat buffer. For optimizers whose update
    of a matrix needs the whole matrix (GefenMuon's Newton-Schulz)."""

    def __init__(self, shapes: Sequence[Tuple[int, ...]], world: int):
        self.world = world
        self.shapes = [tuple(s) for s in shapes]
        dims = [(s[0], int(math.prod(s[1:]))) if len(s) >= 2 else (1, int(math.prod(s)) if len(s) else 1)
                for s in self.shapes]
        load = [0] * world
        owner = [0] * len(dims)
        for t in sorted(range(len(dims)), key=lambda i: (-dims[i][0] * dims[i][1], i)):
            r = min(range(world), key=lambda q: (load[q], q))
            owner[t] = r
            load[r] += _round_up(dims[t][0] * dims[t][1], ALIGN)
        self.segment = _round_up(max(max(load), 1), ALIGN)
        self.total = self.segment * world
        fill = [0] * world
        self.pieces: List[Piece] = []
        for t, (rows, cols) in enumerate(dims):
            r = owner[t]
            self.pieces.append(Piece(t, 0, rows, cols, r, r * self.segment + fill[r]))
            fill[r] += _round_up(rows * cols, ALIGN)
        self.tensor_offset = [p.offset for p in self.pieces]

    def owned(self, rank: int) -> List[Piece]:
        return [p for p in self.pieces if p.rank == rank]


class GpuOps:
    """Device work of the calibration, on the library's kernels."""

    def predict_periods(self, grads: List[torch.Tensor]) -> List[int]:
        from . import partitioning

        launched = [partitioning.launch_period_scores(g, input_is_squared=False) if g.numel() > 1 else (1, [], None, False)
                    for g in grads]
        stats = [s for _, _, s, _ in launched if s is not None]
        host = torch.cat(stats, 0).cpu() if stats else None
        out, cur = [], 0
        for n, cand, s, _ in launched:
            if s is None:
                out.append(1)
            else:
                out.append(partitioning.decide_period(n, cand, host[cur:cur + len(cand)]))
                cur += len(cand)
        return out

    def histograms(self, flats_and_periods, bins: int) -> torch.Tensor:
        from .kernels.exact_histogram_fused import gefen_exact_histogram_cuda

        if not flats_and_periods:
            return torch.zeros((0, bins), dtype=torch.int64)
        rows = torch.zeros((len(flats_and_periods), bins), dtype=torch.int64, device=flats_and_periods[0][0].device)
        for row, (flat, period) in zip(rows, flats_and_periods):
            gefen_exact_histogram_cuda(flat, period, row)
        return rows.cpu()

    def fit_codebook(self, bin_counts: torch.Tensor, num_codebooks: int, device) -> torch.Tensor:
        from . import quantization

        bins = bin_counts.numel()
        edges = torch.linspace(-1.0, 1.0, steps=bins + 1, dtype=torch.float32)
        centers = 0.5 * (edges[:-1] + edges[1:])
        active = bin_counts > 0
        stats = {"active_centers": centers[active], "active_counts": bin_counts[active]}
        return quantization.exact_dp(stats, num_codebooks, True, device=device).to(device)

    def make_optimizer(self, named_pieces, **kwargs):
        from .gefen import Gefen

        return Gefen(named_pieces, **kwargs)


def push_plan(layout, tensor_periods, q: int, n_buckets: int, element_size: int):
    """Buckets of rank q's segment for the pushed reduce-scatter: runs of whole blocks of consecutive pieces,
    about equal in bytes (`host_stream.cut_buckets`). Returns (pieces in address order, the period used for
    each, the cuts, and per bucket the range of elements it covers relative to the start of the segment,
    padded with empty ranges to `n_buckets`). A function of the layout and the periods only, so every rank
    computes the same plan for every other rank."""
    from .host_stream import cut_buckets

    seg = layout.segment
    pieces = sorted(layout.owned(q), key=lambda pc: pc.offset)
    periods = []
    for pc in pieces:
        period = int(tensor_periods[pc.tensor])
        periods.append(period if period > 1 and pc.numel % period == 0 else 1)
    cuts = cut_buckets([pc.numel for pc in pieces], [element_size] * len(pieces), periods, n_buckets) if pieces else []
    ranges = []
    for bucket in cuts:
        lo = min(pieces[i].offset + (0 if whole else b0 * periods[i]) for i, b0, b1, whole in bucket)
        hi = max(pieces[i].offset + (pieces[i].numel if whole else b1 * periods[i]) for i, b0, b1, whole in bucket)
        ranges.append((lo - q * seg, hi - q * seg))
    ranges += [(0, 0)] * (n_buckets - len(ranges))
    return pieces, periods, cuts, ranges


class Zero1Gefen:
    """Gefen over ZeRO-1 sharded optimizer state.

    named_params: list of (name, Parameter) of ONE dtype and device. The parameters and their
    `.grad` are re-pointed into two flat buffers (views, no copies per step). `step()` averages
    the gradients over the ranks of `group` while scattering them, runs the Gefen step on the
    pieces this rank owns and gathers the updated parameters.
    """

    def __init__(self, named_params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, *, group=None,
                 ops=None, average_gradients: bool = True, fused_all_gather: Optional[bool] = None,
                 fused_reduce_scatter: Optional[bool] = None, multicast: Optional[bool] = None, device=None,
                 dtype=None, push_reduce_scatter: Optional[bool] = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.ops = ops if ops is not None else GpuOps()
        self.average = average_gradients
        self.named = [(n, p) for n, p in named_params]
        if not self.named:
            raise ValueError("Zero1Gefen needs at least one parameter")
        # (name, shape) entries instead of (name, Parameter): a model too large to exist twice. The flat
        # buffers are created on `device` with `dtype`, the parameters are made as views of them (see
        # `self.named` afterwards) and the caller fills them.
        self._from_shapes = not torch.is_tensor(self.named[0][1])
        if self._from_shapes:
            if device is None or dtype is None:
                raise ValueError("Zero1Gefen built from shapes needs `device` and `dtype`")
            self.dtype, self.device = dtype, torch.device(device)
            self.named = [(n, tuple(int(x) for x in shape)) for n, shape in self.named]
        else:
            p0 = self.named[0][1]
            self.dtype, self.device = p0.dtype, p0.device
            for n, p in self.named:
                if p.dtype != self.dtype or p.device != self.device:
                    raise ValueError("Zero1Gefen expects one dtype and device per instance, got {} for {}".format(p.dtype, n))
        self.layout = self._make_layout([tuple(p) if self._from_shapes else tuple(p.shape) for _, p in self.named])
        self._token = None
        import os

        # Multicast pays from four ranks on. A multicast store also comes back to the sender through the
        # switch, and a switch-reduced load also pulls the reader's own copy over the links: with two ranks
        # that doubles the bytes per link against plain peer accesses (measured: 7.7 ms against 5.8 ms for
        # 1.5 G bf16 parameters); with N ranks it is (N+1)/N of one buffer per direction for both collectives
        # together, against 2(N-1)/N with peer accesses.
        env_mc = os.environ.get("GEFEN_B200_ZERO1_MULTICAST", "auto")
        want_mc = multicast if multicast is not None else (self.world >= 4 if env_mc == "auto" else env_mc != "0")
        self.flat_param, param_ptrs, param_mc = self._allocate_flat(fused_all_gather, "GEFEN_B200_ZERO1_FUSED_AG",
                                                                    "all_gather")
        # The gradient buffer is symmetric as well unless fused_reduce_scatter=False. Averaging inside the step
        # kernels is the default when the buffer has a multicast address (one switch-reduced load per chunk).
        # Over plain peer loads (fused_reduce_scatter=True or GEFEN_B200_ZERO1_FUSED_RS=1) NVLink's load latency
        # bounds the kernel, more so with more sources per element: that form, exact (fp32 sum in rank order),
        # is taken by default only with two ranks and no room for the pushed form's receive buffer (see below;
        # GEFEN_B200_ZERO1_FUSED_RS=0 keeps NCCL's reduce-scatter there).
        self.flat_grad, grad_ptrs, grad_mc = self._allocate_flat(False if fused_reduce_scatter is False else None,
                                                                 "GEFEN_B200_ZERO1_SYMMETRIC_GRADS", "reduce_scatter")
        if not want_mc:
            param_mc = grad_mc = 0
        env_peer = os.environ.get("GEFEN_B200_ZERO1_FUSED_RS", "auto")
        peer_rs = fused_reduce_scatter if fused_reduce_scatter is not None else env_peer not in ("0", "auto")
        mc_rs = os.environ.get("GEFEN_B200_ZERO1_MULTICAST_RS", "1") != "0"
        # peers in ring order starting after this rank, so that concurrent ranks write to different GPUs
        self._peer_deltas = None if param_ptrs is None else np.array(
            [param_ptrs[(self.rank + k) % self.world] - param_ptrs[self.rank] for k in range(1, self.world)], dtype=np.int64)
        self._param_mc_delta = int(param_mc - param_ptrs[self.rank]) if (param_ptrs is not None and param_mc) else 0
        # gradient buffers in rank order: the same summation order on every rank
        self._grad_mc_delta = int(grad_mc - grad_ptrs[self.rank]) if (grad_ptrs is not None and grad_mc and mc_rs) else 0
        use_grad_srcs = grad_ptrs is not None and (self._grad_mc_delta != 0 or peer_rs)
        self._grad_deltas = np.array([grad_ptrs[r] - grad_ptrs[self.rank] for r in range(self.world)], dtype=np.int64) \
            if use_grad_srcs else None
        # Two ranks (no multicast; three when asked): instead of NCCL's reduce-scatter, every rank pushes the segments it
        # does not own into a receive buffer on their owners with plain device-to-device copies (the copy
        # engines, at the full peer-copy rate), and the step kernels sum the local copies in rank order while
        # they read them. Costs (N-1)/N of one buffer in memory; off where that is too much.
        self._recv = None
        self._push_views = []
        if self._grad_deltas is None and grad_ptrs is not None and fused_reduce_scatter is None:
            self._setup_push(push_reduce_scatter, grad_ptrs)
            # Two ranks without room for the receive buffer (a model that fills the GPUs): averaging by peer
            # loads inside the step kernels still beats NCCL's reduce-scatter in front of them (Llama-32B:
            # 113.7 ms against 118.5 ms per step) and needs no memory.
            if self._recv is None and self.world == 2 and env_peer == "auto" and push_reduce_scatter is None:
                self._grad_deltas = np.array([grad_ptrs[r] - grad_ptrs[self.rank] for r in range(self.world)],
                                             dtype=np.int64)
        with torch.no_grad():
            for t, (n, p) in enumerate(self.named):
                off = self.layout.tensor_offset[t]
                shape = self.layout.shapes[t]
                numel = int(math.prod(shape)) if len(shape) else 1
                view = self.flat_param[off:off + numel].view(shape)
                gview = self.flat_grad[off:off + numel].view(shape)
                if self._from_shapes:
                    p = torch.nn.Parameter(view)
                    self.named[t] = (n, p)
                else:
                    view.copy_(p.data)
                    if p.grad is not None:
                        gview.copy_(p.grad)
                    p.data = view
                p.grad = gview
        seg = self.layout.segment
        self.my_param = self.flat_param[self.rank * seg:(self.rank + 1) * seg]
        self.my_grad = self.flat_grad[self.rank * seg:(self.rank + 1) * seg]
        self.pieces = self.layout.owned(self.rank)
        self.piece_params = []
        named_pieces = []
        for pc in self.pieces:
            shape = (pc.rows, pc.cols) if len(self.named[pc.tensor][1].shape) >= 2 else (pc.cols,)
            if len(self.named[pc.tensor][1].shape) > 2 and pc.rows == self.named[pc.tensor][1].shape[0]:
                shape = tuple(self.named[pc.tensor][1].shape)
            prm = torch.nn.Parameter(self.flat_param[pc.offset:pc.offset + pc.numel].view(shape))
            prm.grad = self.flat_grad[pc.offset:pc.offset + pc.numel].view(shape)
            self.piece_params.append(prm)
            named_pieces.append(("{}#{}".format(self.named[pc.tensor][0], pc.row0), prm))
        self.local = self._make_local(named_pieces, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay) \
            if named_pieces else None
        if self.local is not None and self._peer_deltas is not None:
            self.local._peer_param_deltas = self._peer_deltas
            self.local._param_multicast_delta = self._param_mc_delta
        self.period_mismatches: List[Tuple[str, Dict[int, int]]] = []
        self._events = None
        self._calibrated = False

    def _make_layout(self, shapes):
        return FlatLayout(shapes, self.world)

    def _setup_push(self, requested: Optional[bool], grad_ptrs) -> None:
        """Receive buffer of the pushed reduce-scatter: slot k of rank q holds the copy of q's segment that the
        k-th other rank (rank order) computed. All ranks take the same decision."""
        import os

        env = os.environ.get("GEFEN_B200_ZERO1_PUSH_RS", "auto")
        want = requested if requested is not None else (env != "0")
        seg = self.layout.segment
        nbytes = (self.world - 1) * seg * self.flat_grad.element_size()
        if requested is None and env == "auto":
            total_memory = torch.cuda.get_device_properties(self.device).total_memory
            # (measured and tested with two ranks; three ranks take it only when asked)
            want = self.world == 2 and nbytes * 6 <= total_memory and torch.cuda.mem_get_info(self.device)[0] > nbytes + (8 << 30)
        votes = self._gather_objects(bool(want))
        if not all(votes):
            return
        try:
            import torch.distributed._symmetric_memory as symm_mem

            group = self.group if self.group is not None else dist.group.WORLD
            recv = symm_mem.empty((self.world - 1) * seg, dtype=self.dtype, device=self.device)
            handle = symm_mem.rendezvous(recv, group)
            views = []
            for k in range(1, self.world):   # ring order: concurrent ranks write to different GPUs
                q = (self.rank + k) % self.world
                slot = self.rank if self.rank < q else self.rank - 1
                views.append((q, handle.get_buffer(q, (seg,), self.dtype, slot * seg)))
            own = grad_ptrs[self.rank] + self.rank * seg * recv.element_size()
            deltas = []
            for r in range(self.world):
                slot = r if r < self.rank else r - 1
                deltas.append(0 if r == self.rank else recv.data_ptr() + slot * seg * recv.element_size() - own)
            ok = all(d % 16 == 0 for d in deltas)
        except Exception as exc:
            self.fused_errors["push_reduce_scatter"] = "{}: {}".format(type(exc).__name__, exc)
            ok = False
        if not all(self._gather_objects(bool(ok))):
            self.fused_errors.setdefault("push_reduce_scatter", "another rank could not set up its receive buffer")
            return
        self._symm_handle_push = handle
        self._recv = recv
        self._push_views = views
        self._push_deltas = np.array(deltas, dtype=np.int64)

    def _make_local(self, named_pieces, **kwargs):
        return self.ops.make_optimizer(named_pieces, **kwargs)

    # ------------------------------------------------------------------ flat buffers
    def _allocate_flat(self, requested: Optional[bool], env_name: str, what: str, default: str = "1"):
        """One flat buffer of the layout's size. With NCCL and more than one rank it is symmetric memory
        mapped into every rank, so that the step kernels can do the collective themselves
        (`gefen_b200_multi_tensor_step_peers`): store each updated parameter into all copies
        (no all-gather afterwards), read each gradient from all copies (no reduce-scatter before).
        Returns (buffer, every rank's address of it or None). `requested=False`, or the environment
        variable set to 0, keeps the NCCL collective; so does a failed mapping on any rank (the reason
        is kept in `fused_errors[what]`)."""
        import os

        if not hasattr(self, "fused_errors"):
            self.fused_errors = {}
        want = requested
        if want is None:
            want = os.environ.get(env_name, default) != "0"
        usable = (want and self.world > 1 and self.world - 1 <= 7 and self.device.type == "cuda"
                  and self._backend() == "nccl" and self.dtype != torch.float64)
        if not usable:
            return torch.zeros(self.layout.total, dtype=self.dtype, device=self.device), None, 0
        buf, ptrs, mc = None, None, 0
        try:
            import torch.distributed._symmetric_memory as symm_mem

            group = self.group if self.group is not None else dist.group.WORLD
            buf = symm_mem.empty(self.layout.total, dtype=self.dtype, device=self.device)
            handle = symm_mem.rendezvous(buf, group)
            ptrs = [int(x) for x in handle.buffer_ptrs]
            if ptrs[self.rank] != buf.data_ptr():
                raise RuntimeError("symmetric buffer is not at the address the mapping reports")
            if any((x - ptrs[self.rank]) % 16 for x in ptrs):
                raise RuntimeError("peer buffers are not 16-byte congruent")
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)   # 0: no NVSwitch multicast on this machine
            if mc and (mc - ptrs[self.rank]) % 16:
                mc = 0
            setattr(self, "_symm_handle_" + what, handle)   # keeps the mapping alive
            buf.zero_()
        except Exception as exc:  # mapping is a property of the machine: fall back to the collective
            self.fused_errors[what] = "{}: {}".format(type(exc).__name__, exc)
            buf, ptrs, mc = None, None, 0
        ok = [None] * self.world
        dist.all_gather_object(ok, (ptrs is not None, bool(mc)), group=self.group)
        if not all(o[0] for o in ok):
            self.fused_errors.setdefault(what, "another rank could not map its buffer")
            return torch.zeros(self.layout.total, dtype=self.dtype, device=self.device), None, 0
        if not all(o[1] for o in ok):
            mc = 0
        if self._token is None:
            self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        return buf, ptrs, mc

    @property
    def fused_all_gather_error(self):
        return self.fused_errors.get("all_gather")

    @property
    def reduce_scatter_mode(self) -> str:
        if self.world == 1:
            return "none"
        if self._recv is not None:
            return "device-to-device pushes + sum of the local copies in the step kernels"
        if self._grad_deltas is None:
            return "nccl reduce_scatter"
        return "multimem.ld_reduce in the step kernels" if self._grad_mc_delta else "peer loads in the step kernels"

    @property
    def all_gather_mode(self) -> str:
        if self.world == 1:
            return "none"
        if self._peer_deltas is None:
            return "nccl all_gather"
        return "multimem.st from the step kernels" if self._param_mc_delta else "peer stores from the step kernels"

    # ------------------------------------------------------------------ collectives
    def _backend(self) -> str:
        return dist.get_backend(self.group) if dist.is_initialized() else "none"

    def _rank_barrier(self) -> None:
        """Orders the ranks' streams: a one-element all-reduce completes on a rank only after every
        rank's earlier work on its stream has."""
        dist.all_reduce(self._token, group=self.group)

    def _reduce_scatter(self) -> None:
        if self.world == 1:
            return
        fused = self._grad_deltas is not None and self._calibrated and not getattr(self, "_materialize_gradients", False)
        if self.local is not None:
            # the calibration step needs the averaged gradients in memory (periods, histogram), so it
            # uses the collective; afterwards the step kernels average while they read
            self.local._grad_src_deltas = self._grad_deltas if fused else None
            self.local._grad_multicast_delta = self._grad_mc_delta if fused else 0
            self.local._grad_src_scale = (1.0 / self.world) if self.average else 1.0
        if fused:
            self._rank_barrier()   # every rank's gradients are final, nobody still reads old parameters
            return
        if self._backend() == "nccl":
            op = dist.ReduceOp.AVG if self.average else dist.ReduceOp.SUM
            dist.reduce_scatter_tensor(self.my_grad, self.flat_grad, op=op, group=self.group)
        else:  # gloo has no reduce-scatter: reduce everything, keep the owned segment
            dist.all_reduce(self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
            if self.average:
                self.my_grad.div_(self.world)

    def _all_gather(self) -> None:
        if self.world == 1:
            return
        if self._peer_deltas is not None:
            # the kernels have already written every copy; what is left is the ordering: a rank may
            # use its parameters only after all ranks' launches have finished (a one-element
            # all-reduce on the same stream is that barrier)
            self._rank_barrier()
            return
        # (with fused gradient averaging and this collective, the collective is also what tells a
        # rank that the peers have finished reading its gradients)
        if self._backend() == "nccl":
            dist.all_gather_into_tensor(self.flat_param, self.my_param, group=self.group)
        else:
            seg = self.layout.segment
            parts = [self.flat_param[r * seg:(r + 1) * seg] for r in range(self.world)]
            gathered = [torch.empty_like(self.my_param) for _ in range(self.world)]
            dist.all_gather(gathered, self.my_param.clone(), group=self.group)
            for dst, src in zip(parts, gathered):
                dst.copy_(src)

    def _gather_objects(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.group)
        return out

    # ------------------------------------------------------------------ calibration
    def _calibrate(self) -> None:
        """Periods per piece, one period per tensor, global histogram, one codebook everywhere."""
        from .gefen import HISTOGRAM_BINS, NUM_CODEBOOK_ENTRIES

        grads = [prm.grad.detach() for prm in self.piece_params]
        local_periods = self.ops.predict_periods(grads) if grads else []
        mine = {(pc.tensor, pc.row0): (per, pc.numel) for pc, per in zip(self.pieces, local_periods)}
        everyone: Dict[Tuple[int, int], Tuple[int, int]] = {}
        for d in self._gather_objects(mine):
            everyone.update(d)
        # one period per tensor: the choice of its largest piece (first on ties); pieces normally agree
        chosen: Dict[int, int] = {}
        for t in range(len(self.named)):
            votes = sorted(((numel, -row0, per) for (tt, row0), (per, numel) in everyone.items() if tt == t), reverse=True)
            period = votes[0][2]
            if any(v[2] != period for v in votes):
                self.period_mismatches.append((self.named[t][0], {-v[1]: v[2] for v in votes}))
                if any(v[0] % period for v in votes):
                    period = math.gcd(*[v[2] for v in votes])
            chosen[t] = period
        if self.period_mismatches and self.rank == 0:
            import warnings

            warnings.warn("Zero1Gefen: the pieces of {} tensor(s) voted for different periods ({}); the largest piece "
                          "decided, a single process might choose otherwise".format(
                              len(self.period_mismatches), ", ".join(n for n, _ in self.period_mismatches[:4])))
        flats = [(g.reshape(-1), chosen[pc.tensor]) for pc, g in zip(self.pieces, grads)]
        hist = self.ops.histograms(flats, HISTOGRAM_BINS)
        mine_h = {(pc.tensor, pc.row0): hist[i] for i, pc in enumerate(self.pieces)}
        all_h: Dict[Tuple[int, int], torch.Tensor] = {}
        for d in self._gather_objects(mine_h):
            all_h.update(d)
        bin_counts = torch.zeros(HISTOGRAM_BINS, dtype=torch.float32)
        for t in range(len(self.named)):
            rows = [h for (tt, _), h in sorted(all_h.items()) if tt == t]
            if rows:
                bin_counts.add_(torch.stack(rows).sum(0).to(torch.float32))   # int64 sum is exact
        codebook = self.ops.fit_codebook(bin_counts, NUM_CODEBOOK_ENTRIES, self.device)
        self.codebook = codebook
        if self.local is not None:
            for pc, prm in zip(self.pieces, self.piece_params):
                self.local.state[prm]["automatic_period"] = chosen[pc.tensor]
            self.local._gefen_codebook = codebook.contiguous()
        self.periods = chosen
        self._calibrated = True

    # ------------------------------------------------------------------ step
    def _mark(self):
        if self.device.type != "cuda":
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def _plan_push(self) -> None:
        """Cuts every rank's segment into the buckets of the pushed reduce-scatter (every rank computes all
        ranks' cuts: a pusher must know its receivers' bucket limits). A bucket is a run of whole blocks of
        consecutive pieces, about equal in bytes; `_push_ranges[q][k]` is its range of elements relative to
        the start of q's segment, `_push_steps[k]` what this rank steps once bucket k has arrived."""
        import os

        n_buckets = max(1, int(os.environ.get("GEFEN_B200_ZERO1_PUSH_BUCKETS", "8")))
        esize = self.flat_grad.element_size()
        self._push_ranges, self._push_steps = {}, []
        for q in range(self.world):
            pieces, periods, cuts, ranges = push_plan(self.layout, self.periods, q, n_buckets, esize)
            self._push_ranges[q] = ranges
            if q == self.rank:
                by_offset = {pc.offset: prm for pc, prm in zip(self.pieces, self.piece_params)}
                for bucket in cuts:
                    prms = [(by_offset[pieces[i].offset], b0, b1, whole) for i, b0, b1, whole in bucket]
                    self._push_steps.append((set(id(p) for p, _, _, _ in prms),
                                             {id(p): (b0, b1) for p, b0, b1, whole in prms if not whole},
                                             set(id(p) for p, b0, _, _ in prms if b0 == 0)))
                self._push_steps += [None] * (n_buckets - len(self._push_steps))
        self._push_stream = torch.cuda.Stream(self.device)
        self._push_token = torch.zeros(1, dtype=torch.float32, device=self.device)

    def _step_pushed(self) -> None:
        """The step with the pushed reduce-scatter, bucket by bucket: on a side stream the copy engines push
        bucket k of every segment this rank does not own to its owner, followed by a barrier of the ranks;
        the step kernels (which also store the updated parameters to every rank) take bucket k as soon as it
        is complete, while the pushes of bucket k + 1 are on the wire."""
        if getattr(self, "_push_ranges", None) is None:
            self._plan_push()
        seg = self.layout.segment
        main = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(main)   # gradients are final; the receive buffers' readers (the previous step) are done
        self._push_stream.wait_event(start)
        arrived = []
        with torch.cuda.stream(self._push_stream):
            for k in range(len(self._push_ranges[self.rank])):
                for q, view in self._push_views:
                    lo, hi = self._push_ranges[q][k]
                    if hi > lo:
                        view[lo:hi].copy_(self.flat_grad[q * seg + lo:q * seg + hi], non_blocking=True)
                dist.all_reduce(self._push_token, group=self.group)   # every rank's pushes of bucket k have landed
                e = torch.cuda.Event()
                e.record(self._push_stream)
                arrived.append(e)
        if self.local is not None:
            self.local._maybe_refresh_gefen_codebook()
            self.local._grad_src_deltas = self._push_deltas
            self.local._grad_multicast_delta = 0
            self.local._grad_src_scale = (1.0 / self.world) if self.average else 1.0
        for k, e in enumerate(arrived):
            main.wait_event(e)
            if self.local is not None and self._push_steps[k] is not None:
                only, ranges, advance = self._push_steps[k]
                self.local._step_multi_tensor(only=only, ranges=ranges, advance=advance)
        if self.local is not None:
            self.local._gefen_global_step += 1

    @torch.no_grad()
    def step(self):
        if self._recv is not None and self._calibrated and not getattr(self, "_materialize_gradients", False):
            marks = [self._mark(), self._mark()]
            self._step_pushed()
            marks.append(self._mark())
            self._all_gather()
            marks.append(self._mark())
            self._events = marks
            return
        marks = [self._mark()]
        self._reduce_scatter()
        marks.append(self._mark())
        if not self._calibrated:
            self._calibrate()
        if self.local is not None:
            self.local.step()
        marks.append(self._mark())
        self._all_gather()
        marks.append(self._mark())
        self._events = marks

    def last_breakdown_ms(self):
        """Device time of the last step's three phases (synchronises)."""
        if not self._events or self._events[0] is None:
            return {}
        torch.cuda.synchronize(self.device)
        m = self._events
        launches = 0
        if self.local is not None and getattr(self.local, "_plan", None) is not None:
            launches = sum(len(set(t.get("classes", [1]))) for t in (self.local._plan.tables or []))
        return {"reduce_scatter": m[0].elapsed_time(m[1]), "local_step": m[1].elapsed_time(m[2]),
                "all_gather": m[2].elapsed_time(m[3]), "kernel_launches_per_step": launches}

    def zero_grad(self):
        self.flat_grad.zero_()

    # ------------------------------------------------------------------ N ranks against one process
    def verify_against_single_process(self, steps: int = 2, max_elements: int = 48 << 20) -> Dict[str, object]:
        """Collective; call it between steps of a calibrated optimizer. Checks the invariant of the sharding:
        given the same reduced gradients, the state and parameters of the pieces a rank owns are bit for bit
        what a plain single-process `Gefen` computes. Every rank takes a few of its pieces (up to
        `max_elements` elements), clones their state and parameters into a single-process optimizer, and for
        `steps` steps both sides consume the gradients that NCCL's reduce-scatter left in memory: the sharded
        side through its production step kernels (parameters leaving through multimem.st or peer stores), the
        single-process side through `Gefen.step`. Codes, magnitudes, second moments and parameters must be
        identical. Where the gradients are normally summed by the switch inside the kernel, one more step
        compares that path with a single-process step fed the same switch-summed values written to memory
        (`gefen_b200_multicast_sum`). Finally all ranks must hold the same parameter buffer. Advances the
        optimizer by steps (+1) real steps. Returns the verdict (identical on every rank)."""
        from . import _lib

        if not self._calibrated:
            raise RuntimeError("verify_against_single_process needs a calibrated optimizer: run one step first")
        chosen, total = [], 0
        if self.local is not None:
            for pc, prm in zip(self.pieces, self.piece_params):
                if total + pc.numel <= max_elements:
                    chosen.append((pc, prm))
                    total += pc.numel
            if not chosen:   # nothing small enough: the smallest piece
                pc, prm = min(zip(self.pieces, self.piece_params), key=lambda item: item[0].numel)
                chosen, total = [(pc, prm)], pc.numel
        single, mine = None, []
        if chosen:
            named = []
            for pc, prm in chosen:
                clone = torch.nn.Parameter(prm.detach().clone())
                clone.grad = torch.zeros_like(clone)
                mine.append(clone)
                named.append(("{}#{}".format(self.named[pc.tensor][0], pc.row0), clone))
            single = self._make_single_process(named)
            for (pc, prm), clone in zip(chosen, mine):
                single.state[clone].update({k: (v.detach().clone() if torch.is_tensor(v) else v)
                                            for k, v in self.local.state[prm].items()})
            single._gefen_codebook = self.local._gefen_codebook.clone()
            single._gefen_global_step = self.local._gefen_global_step

        def identical() -> bool:
            ok = True
            for (pc, prm), clone in zip(chosen, mine):
                a, b = self.local.state[prm], single.state[clone]
                ok = ok and torch.equal(prm.detach(), clone.detach())
                for key in ("m_codebook", "m_magnitude", "vmean"):
                    if key in a:
                        ok = ok and torch.equal(a[key], b[key])
            return ok

        verdict = {"tensors": len(chosen), "elements": total, "steps": steps, "bit_identical": True}
        self._materialize_gradients = True
        try:
            for _ in range(steps):
                self._reduce_scatter()                        # NCCL: the averaged gradients are in memory
                for (pc, prm), clone in zip(chosen, mine):
                    clone.grad.copy_(prm.grad)
                if self.local is not None:
                    self.local.step()                         # production kernels, production all-gather
                self._all_gather()
                if single is not None:
                    single.step()
                    verdict["bit_identical"] = verdict["bit_identical"] and identical()
        finally:
            self._materialize_gradients = False
        if self._grad_mc_delta and self._grad_deltas is not None:
            # the production gradient path: summed by the switch inside the kernel
            lib = _lib.load()
            classes_ok = []
            if single is not None:
                scale = (1.0 / self.world) if self.average else 1.0
                for (pc, prm), clone in zip(chosen, mine):
                    src = prm.grad.data_ptr() + self._grad_mc_delta
                    usable = pc.numel % 8 == 0 and prm.grad.data_ptr() % 16 == 0
                    classes_ok.append(usable)
                    if usable:
                        with _lib.device_guard(self.device):
                            _lib.check(lib.gefen_b200_multicast_sum(_lib.ptr(clone.grad), ctypes.c_void_p(src),
                                                                    _lib.dtype_tag(self.dtype), pc.numel, scale,
                                                                    _lib.current_stream(self.device)))
            self.step()
            if single is not None:
                # pieces that the generic kernels handle take the rank-order sum of the peers' copies: leave
                # them out of this comparison (they were covered above)
                keep = [i for i, ok in enumerate(classes_ok) if ok and self._piece_is_staged(chosen[i][1])]
                single.step()
                same = True
                for i in keep:
                    (pc, prm), clone = chosen[i], mine[i]
                    a, b = self.local.state[prm], single.state[clone]
                    same = same and torch.equal(prm.detach(), clone.detach()) and torch.equal(a["m_codebook"], b["m_codebook"]) \
                        and torch.equal(a["m_magnitude"], b["m_magnitude"]) and torch.equal(a["vmean"], b["vmean"])
                verdict["in_kernel_reduce_bit_identical"] = same
                verdict["in_kernel_reduce_tensors"] = len(keep)
        elif self._recv is not None:
            # the production gradient path: pushed copies summed in rank order inside the kernel
            if single is not None:
                scale = (1.0 / self.world) if self.average else 1.0
                seg = self.layout.segment
            self.step()
            if single is not None:
                for (pc, prm), clone in zip(chosen, mine):
                    acc = torch.zeros(pc.numel, dtype=torch.float32, device=self.device)
                    for r in range(self.world):
                        if r == self.rank:
                            acc += self.flat_grad[pc.offset:pc.offset + pc.numel].float()
                        else:
                            slot = r if r < self.rank else r - 1
                            begin = slot * seg + pc.offset - self.rank * seg
                            acc += self._recv[begin:begin + pc.numel].float()
                    clone.grad.copy_((acc * scale).to(self.dtype).view_as(clone.grad))
                single.step()
                verdict["in_kernel_reduce_bit_identical"] = identical()
                verdict["in_kernel_reduce_tensors"] = len(chosen)
        # every rank ends with the same parameters
        # (summed in slices: the int64 copy torch makes of a slice stays small beside a buffer that may fill the GPU)
        bits = torch.int16 if self.flat_param.element_size() == 2 else torch.int32
        as_int = self.flat_param.view(bits)
        check = torch.zeros(1, dtype=torch.int64, device=self.device)
        for begin in range(0, as_int.numel(), 1 << 27):
            check += as_int[begin:begin + (1 << 27)].sum(dtype=torch.int64)
        lo, hi = check.clone(), check.clone()
        if self.world > 1:
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
        verdict["params_identical_across_ranks"] = bool(int(lo) == int(hi))
        flags = torch.tensor([1.0 if verdict["bit_identical"] else 0.0,
                              1.0 if verdict.get("in_kernel_reduce_bit_identical", True) else 0.0,
                              float(verdict["tensors"]), float(verdict["elements"]),
                              float(verdict.get("in_kernel_reduce_tensors", 0))], device=self.device, dtype=torch.float64)
        worst = flags[:2].clone()
        sums = flags[2:].clone()
        if self.world > 1:
            dist.all_reduce(worst, op=dist.ReduceOp.MIN, group=self.group)
            dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=self.group)
        verdict["bit_identical"] = bool(worst[0] > 0)
        if self._grad_mc_delta or self._recv is not None:
            verdict["in_kernel_reduce_bit_identical"] = bool(worst[1] > 0)
            verdict["in_kernel_reduce_tensors"] = int(sums[2])
        verdict["tensors"], verdict["elements"] = int(sums[0]), int(sums[1])
        return verdict

    def _make_single_process(self, named):
        """The plain optimizer that `verify_against_single_process` holds the sharded one against."""
        from .gefen import Gefen

        g0 = self.local.param_groups[0]
        return Gefen(named, lr=g0["lr"], betas=(g0["beta1"], g0["beta2"]), eps=g0["eps"], weight_decay=g0["weight_decay"])

    def _piece_is_staged(self, prm) -> bool:
        """True if the local optimizer steps this piece with the staged (vectorised) kernel."""
        plan = getattr(self.local, "_plan", None)
        if plan is None:
            return False
        params = [p for g in self.local.param_groups for p in g["params"] if p.grad is not None]
        for table in plan.tables or []:
            for entry, cls in zip(table["entries"], table["classes"]):
                if entry < len(params) and params[entry] is prm:
                    return cls >= 1
        return False

    def state_dict(self):
        """This rank's shard of the optimizer state plus the (identical everywhere) codebook."""
        return {"rank": self.rank, "world": self.world, "periods": getattr(self, "periods", None),
                "local": None if self.local is None else self.local.state_dict()}

    def load_state_dict(self, sd):
        if sd["world"] != self.world or sd["rank"] != self.rank:
            raise ValueError("Zero1Gefen state was saved for rank {}/{}".format(sd["rank"], sd["world"]))
        if self.local is not None and sd["local"] is not None:
            self.local.load_state_dict(sd["local"])
            self.codebook = self.local._gefen_codebook
            self._calibrated = self.codebook is not None
        self.periods = sd.get("periods")

    # ------------------------------------------------------------------ world-size independent checkpoint
    def _piece_blocks(self, pc: Piece, period: int) -> Tuple[int, int]:
        """Range of the tensor's partition blocks that lie in piece `pc` (blocks never straddle pieces)."""
        first, last = pc.row0 * pc.cols, (pc.row0 + pc.rows) * pc.cols
        if first % period or last % period:
            raise ValueError("period {} does not tile the piece at row {}".format(period, pc.row0))
        return first // period, last // period

    def full_state_dict(self):
        """Collective. The optimizer state of the WHOLE model on every rank, per tensor and in the layout
        a single process keeps (reference: gefen.py:1039-1062, 1343-1349): the pieces' codes, magnitudes
        and second moments concatenated in row order (CPU tensors). It can be loaded at any other world
        size with `load_full_state_dict`, and `state` has the reference's per-parameter schema."""
        mine = {}
        for pc, prm in zip(self.pieces, self.piece_params):
            st = self.local.state[prm] if self.local is not None else {}
            mine[(pc.tensor, pc.row0)] = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in st.items()}
        everyone = {}
        for d in self._gather_objects(mine):
            everyone.update(d)
        state = {}
        for t in range(len(self.named)):
            parts = [everyone[k] for k in sorted(k for k in everyone if k[0] == t)]
            parts = [p for p in parts if p]
            if not parts:
                continue
            if len(parts) == 1:
                state[t] = dict(parts[0])
                continue
            if any(p.get("automatic_period") == 1 for p in parts):
                raise NotImplementedError("a tensor with period 1 that is split between ranks keeps rank-local "
                                          "magnitude blocks and cannot be consolidated")
            merged = {}
            for key, value in parts[0].items():
                if torch.is_tensor(value) and value.dim() >= 1:
                    merged[key] = torch.cat([p[key] for p in parts], dim=0)
                else:
                    merged[key] = value
            if "m_codebook_shape" in merged:
                merged["m_codebook_shape"] = tuple(merged["m_codebook"].shape)
            state[t] = merged
        codebook = getattr(self, "codebook", None)
        return {"format": "gefen_b200.zero1.full/1", "names": [n for n, _ in self.named],
                "shapes": [tuple(p.shape) for _, p in self.named], "state": state,
                "periods": dict(getattr(self, "periods", None) or {}),
                "gefen_codebook": None if codebook is None else codebook.detach().cpu(),
                "gefen_global_step": max([int(st.get("step", 0)) for st in state.values()] or [0])}

    def load_full_state_dict(self, full) -> None:
        """Takes this rank's share of a `full_state_dict` (saved at any world size)."""
        if [tuple(s) for s in full["shapes"]] != [tuple(p.shape) for _, p in self.named]:
            raise ValueError("the checkpoint was written for different parameter shapes")
        self.periods = {int(k): int(v) for k, v in full["periods"].items()}
        codebook = full["gefen_codebook"]
        self.codebook = None if codebook is None else codebook.to(self.device)
        if self.local is None:
            self._calibrated = self.codebook is not None
            return
        for pc, prm in zip(self.pieces, self.piece_params):
            whole = full["state"].get(pc.tensor)
            target = self.local.state[prm]
            target.clear()
            if not whole:
                continue
            period = int(whole["automatic_period"])
            whole_rows = self.layout.shapes[pc.tensor][0] if len(self.layout.shapes[pc.tensor]) >= 2 else 1
            if pc.rows == whole_rows or len(self.layout.shapes[pc.tensor]) < 2:
                piece_state = dict(whole)
            else:
                if period == 1:
                    raise NotImplementedError("a tensor with period 1 cannot be split between ranks on load")
                b0, b1 = self._piece_blocks(pc, period)
                nb = whole["m_codebook"].shape[0]
                piece_state = {k: (v[b0:b1].clone() if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == nb else v)
                               for k, v in whole.items()}
                if "m_codebook_shape" in piece_state:
                    piece_state["m_codebook_shape"] = tuple(piece_state["m_codebook"].shape)
            for k, v in piece_state.items():
                target[k] = v.to(self.device) if torch.is_tensor(v) else v
        self.local._gefen_codebook = None if self.codebook is None else self.codebook.contiguous()
        if hasattr(self.local, "_gefen_global_step"):
            self.local._gefen_global_step = int(full.get("gefen_global_step", 0))
        if hasattr(self.local, "_plans"):
            self.local._plans = {}
            self.local._steady = None
        self._calibrated = self.codebook is not None


class Zero1GefenMuon(Zero1Gefen):
    """GefenMuon over ZeRO-1 sharded state. Newton-Schulz needs whole matrices, so whole tensors are
    assigned to ranks (`WholeTensorLayout`); the step is NCCL's reduce-scatter of the gradients, then
    GefenMuon on the owned matrices, whose last kernel per matrix (decay + update,
    `gefen_b200_muon_apply`) also stores the new matrix into every peer's parameter buffer: the
    all-gather rides on those stores, under the other matrices' Newton-Schulz products (plain peer
    stores; the multicast form would only add the loop back through the switch here, since nothing flows
    the other way at the same time). N ranks reproduce one rank bit for bit: every matrix is processed
    whole by the same kernels, and the codebook is fitted from the gathered histogram."""

    def __init__(self, named_params, lr=1e-3, weight_decay=0.1, momentum=0.95, nesterov=True,
                 ns_coefficients=(3.4445, -4.7750, 2.0315), eps=1e-7, ns_steps=5, adjust_lr_fn=None, *, group=None,
                 ops=None, average_gradients: bool = True, fused_all_gather: Optional[bool] = None):
        self._muon_kwargs = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                                 ns_coefficients=ns_coefficients, eps=eps, ns_steps=ns_steps, adjust_lr_fn=adjust_lr_fn)
        super().__init__(named_params, lr=lr, eps=eps, weight_decay=weight_decay, group=group, ops=ops,
                         average_gradients=average_gradients, fused_all_gather=fused_all_gather,
                         fused_reduce_scatter=False, multicast=False)

    def _make_layout(self, shapes):
        for s in shapes:
            if len(s) != 2:
                raise ValueError("GefenMuon only supports 2D parameters whereas we found a parameter with size: {}".format(s))
        return WholeTensorLayout(shapes, self.world)

    def _make_single_process(self, named):
        from .gefen_muon import GefenMuon

        return GefenMuon(named, **self._muon_kwargs)

    def _make_local(self, named_pieces, **kwargs):
        if hasattr(self.ops, "make_muon_optimizer"):
            return self.ops.make_muon_optimizer(named_pieces, **self._muon_kwargs)
        from .gefen_muon import GefenMuon

        return GefenMuon(named_pieces, **self._muon_kwargs)
