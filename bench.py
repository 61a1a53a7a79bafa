"""Benchmark of the Gefen optimizer step on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload llama_1_5b]

One JSON line on stdout (rank 0). A "step" is one Gefen optimizer step over the whole parameter
set. N = 1: Llama-style 1.5B, bf16 parameters and gradients, lr 3e-4, weight decay 0.1, synthetic
seeded inputs resident in HBM; N > 1: the same parameter set ZeRO-1 sharded (reduce-scatter of
gradients, local step, all-gather of parameters). `--impl reference` times the CPU oracle port of
the reference step on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from gefen_b200 import workloads  # noqa: E402

PUBLISHED_LLAMA_1_5B_MS = 29.0  # reference README.md:145, hardware not stated
WORKLOADS = {
    "llama_1_5b": dict(shapes=workloads.llama_1_5b, dtype=torch.bfloat16, lr=3e-4, wd=0.1, sigma=1e-3, tau=1.0),
    "gpt2_125m": dict(shapes=workloads.gpt2_125m, dtype=torch.float32, lr=1e-3, wd=0.0, sigma=1e-3, tau=1.0),
    "llama_32b": dict(shapes=workloads.llama_32b, dtype=torch.bfloat16, lr=1.5e-4, wd=0.1, sigma=1e-3, tau=1.0),
    "qwen3_muon": dict(shapes=workloads.qwen3_1_7b_matrices, dtype=torch.bfloat16, lr=0.02, wd=0.1, sigma=1e-3, tau=0.5,
                       muon=True),
}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_model(cfg, device, limit_elems=None):
    """Parameters and one set of gradients on `device`. limit_elems keeps a prefix of whole tensors."""
    shapes = cfg["shapes"]()
    if limit_elems is not None:
        kept, total = [], 0
        for name, shape in shapes[1:]:  # skip the embedding: a layer-shaped sample
            if total + workloads.numel(shape) > limit_elems:
                break
            kept.append((name, shape))
            total += workloads.numel(shape)
        shapes = kept
    params, grads = [], []
    for i, (name, shape) in enumerate(shapes):
        params.append(workloads.init_param(name, shape, i, cfg["dtype"], device))
        grads.append(workloads.make_grad(shape, i, 0, cfg["dtype"], device, cfg["sigma"], cfg["tau"]))
    return shapes, params, grads


# --------------------------------------------------------------------------- CPU arm (oracle port)
def workload_config(args, cfg, world, n_tensors, total_elems):
    """The `config` object of the JSON line: static facts of the workload only, so that the GPU arm and the
    reference arm print the same object (what calibration finds goes into `periods`, beside it)."""
    elem_bytes = 2 if cfg["dtype"] == torch.bfloat16 else 4
    return {"workload": args.workload, "optimizer": "Gefen(fused=True)", "lr": cfg["lr"],
            "weight_decay": cfg["wd"], "betas": [0.9, 0.999], "eps": 1e-8,
            "tensors": n_tensors, "elements": total_elems,
            "parallelism": "zero1-dp{}".format(world) if world > 1 else "single-gpu",
            "l2": "inputs ({:.1f} GB per step) are larger than L2".format(total_elems * (3 * elem_bytes + 2) / 1e9)}


def periods_found(shapes, periods):
    """What the calibration chose: the distinct periods and the elements under each."""
    by_period = period_census(shapes, periods)
    return {"distinct": sorted(set(periods)), "elements_by_period": {str(k): by_period[k] for k in sorted(by_period)}}


def period_census(shapes, per_tensor):
    by_period = {}
    for (_, shape), period in zip(shapes, per_tensor):
        by_period[period] = by_period.get(period, 0) + workloads.numel(shape)
    return by_period


def cpu_port_run(cfg, steps: int, warmup: int, sample_elems, budget_s=None):
    """The CPU oracle's restatement of the reference step on the host cores (C with OpenMP, all
    threads): the oracle's own calibration (period search, histogram, exact-DP codebook), then
    `warmup` untimed and `steps` timed steady-state steps. sample_elems=None: the whole workload;
    otherwise a prefix of whole layer tensors of about that many elements."""
    from oracle.ref_loop import OracleGefen

    device = torch.device("cpu")
    shapes, params, grads = build_model(cfg, device, limit_elems=sample_elems)
    opt = OracleGefen(params, lr=cfg["lr"], betas=(0.9, 0.999), eps=1e-8, weight_decay=cfg["wd"])
    t0 = time.perf_counter()
    opt.calibrate(grads)
    calib_s = time.perf_counter() - t0
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        opt.step(grads)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
            if budget_s is not None and sum(times) + dt > budget_s:   # the next step would overrun the budget
                break
    periods = [st["automatic_period"] for st in opt.state]
    return {"ms": 1e3 * sum(times) / len(times), "shapes": shapes, "periods": periods, "calibration_s": calib_s,
            "elements": sum(workloads.numel(s) for _, s in shapes), "cores": os.cpu_count(), "timed_steps": len(times)}


REFERENCE_ARM_BUDGET_S = 100.0   # a CPU step of the 1.5 B set takes seconds: the arm stops timing after this long


def run_reference_arm(args, cfg, rank, world):
    """`--impl reference`: the whole workload through the CPU port, nothing sampled or scaled. It times the
    K steps it is asked for unless they would take longer than REFERENCE_ARM_BUDGET_S; `steps` of the line
    is the number actually timed (`requested_steps` the number asked for)."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    run = cpu_port_run(cfg, max(1, args.steps), 1, None, budget_s=REFERENCE_ARM_BUDGET_S)
    shapes, periods = run["shapes"], run["periods"]
    elem_bytes = 2 if cfg["dtype"] == torch.bfloat16 else 4
    algo_bytes = workloads.step_bytes(shapes, periods, elem_bytes, elem_bytes)
    ms = run["ms"]
    line = {
        "impl": "reference", "metric": "optimizer_step_ms", "value": ms, "unit": "ms", "n_gpus": args.gpus,
        "steps": run["timed_steps"], "warmup": 1, "requested_steps": args.steps, "requested_warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": ms / PUBLISHED_LLAMA_1_5B_MS if args.workload == "llama_1_5b" else None,
        "dtype": "bf16" if cfg["dtype"] == torch.bfloat16 else "f32", "data": "synthetic",
        "config": workload_config(args, cfg, world, len(shapes), run["elements"]),
        "periods": periods_found(shapes, periods), "algorithmic_bytes_per_step": algo_bytes,
        "timed_steps_note": "a CPU step of this workload takes seconds: {} steady-state steps were timed after one "
                            "untimed step (the arm stops after {:.0f} s of timed steps); nothing is sampled or scaled"
                            .format(run["timed_steps"], REFERENCE_ARM_BUDGET_S),
        "calibration_s": run["calibration_s"],
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": run["cores"], "kind": "port",
                         "sample": "the whole workload ({} elements, {} tensors): the C oracle with OpenMP, its own "
                                   "calibration, steady-state steps".format(run["elements"], len(shapes))},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU arm
def timed(fn, steps: int, stream=None):
    """CUDA-event time of `steps` calls of fn on the current stream, synchronised on both sides."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_sharded_arm(args, cfg, rank, world, local_rank):
    """N > 1: the parameter set ZeRO-1 sharded over the ranks (gefen_b200.Zero1Gefen). The flat buffers are
    created first and the synthetic parameters and gradients are written straight into them, so that a
    model exists once per GPU (the 32 B set: 65 GB of parameters + 65 GB of gradients per rank)."""
    import torch.distributed as dist

    from gefen_b200.zero1 import Zero1Gefen

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    shapes = cfg["shapes"]()
    opt = Zero1Gefen(shapes, lr=cfg["lr"], betas=(0.9, 0.999), eps=1e-8, weight_decay=cfg["wd"], device=device,
                     dtype=cfg["dtype"])
    with torch.no_grad():
        for i, ((name, shape), (_, p)) in enumerate(zip(shapes, opt.named)):
            p.data.copy_(workloads.init_param(name, shape, i, cfg["dtype"], device))
            # every rank its own gradients (seeded by rank), as data-parallel ranks have
            p.grad.copy_(workloads.make_grad(shape, i, rank, cfg["dtype"], device, cfg["sigma"], cfg["tau"]))
    step = opt.step
    calibration_ms = timed(step, 1)
    warm = max(args.warmup - 1, 2)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warm):
        step()
    dist.barrier()
    ms = timed(step, args.steps)
    t = torch.tensor([ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    breakdown = opt.last_breakdown_ms()
    for _ in range(int(400.0 / max(ms, 0.05)) + 1):   # the same load until the clock sampler has seen it
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    dist.barrier()

    per_tensor = [opt.periods[t] for t in range(len(shapes))]
    elem_bytes = opt.flat_param.element_size()
    total_elems = sum(workloads.numel(s) for _, s in shapes)
    algo_bytes = workloads.step_bytes(shapes, per_tensor, elem_bytes, elem_bytes)
    result = {"ms": ms, "calibration_ms": calibration_ms, "clocks": clocks, "algo_bytes": algo_bytes,
              "total_elems": total_elems, "n_tensors": len(shapes), "periods": per_tensor, "shapes": shapes}
    breakdown["all_gather_mode"] = opt.all_gather_mode
    breakdown["reduce_scatter_mode"] = opt.reduce_scatter_mode
    if opt.fused_errors:
        breakdown["fused_errors"] = dict(opt.fused_errors)
    # what each rank moves over NVLink per step, and what the links could do at best: every rank must send
    # (N-1)/N of its gradients and receive (N-1)/N of the parameters; with the switch's multicast the other
    # direction of each collective shrinks to 1/N of the buffer
    flat_bytes = opt.flat_param.numel() * elem_bytes
    frac = (world - 1) / world
    mc_rs = opt.reduce_scatter_mode.startswith("multimem")
    mc_ag = opt.all_gather_mode.startswith("multimem")
    egress = flat_bytes * frac + (flat_bytes / world if mc_ag else flat_bytes * frac)
    ingress = (flat_bytes / world if mc_rs else flat_bytes * frac) + (flat_bytes if mc_ag else flat_bytes * frac)
    breakdown["wire_bytes_per_rank"] = {"egress": int(egress), "ingress": int(ingress)}
    breakdown["link_floor_ms"] = {"at_770_gbs_measured_peer_copy": max(egress, ingress) / 770e6,
                                  "at_900_gbs_nominal": max(egress, ingress) / 900e6}
    breakdown["achieved_link_gbs"] = max(egress, ingress) / ms / 1e6

    # the 1/N part: this rank's share of the step with nothing crossing NVLink (max over ranks)
    local_ms = None
    if opt.local is not None:
        saved = {k: getattr(opt.local, k, None) for k in ("_peer_param_deltas", "_grad_src_deltas", "_param_multicast_delta",
                                                         "_grad_multicast_delta")}
        for k in saved:
            setattr(opt.local, k, None)
        opt.local.step()
        local_ms = timed(opt.local.step, max(2, min(args.steps, 5)))
        for k, v in saved.items():
            setattr(opt.local, k, v)
    lt = torch.tensor([local_ms if local_ms is not None else 0.0], device=device)
    dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    breakdown["local_compute_ms"] = float(lt)
    # the local steps above touched only the owned segments: bring every copy back in line before the check
    opt.step()
    result["breakdown"] = breakdown
    try:
        result["n_vs_1"] = opt.verify_against_single_process(steps=2)
    except torch.OutOfMemoryError as exc:   # the check is an extra: the measured line must survive it
        result["n_vs_1"] = {"error": "out of memory in the check: {}".format(str(exc)[:120])}

    e2e = None
    if not args.no_e2e:
        # end to end at N ranks: every rank's gradients come from its own pinned host buffer and the full
        # updated parameters go back to it (flat buffers, one copy each way per rank and step)
        host_g = host_p = None
        try:
            host_g = torch.empty(opt.flat_grad.shape, dtype=opt.flat_grad.dtype, pin_memory=True)
            host_p = torch.empty(opt.flat_param.shape, dtype=opt.flat_param.dtype, pin_memory=True)
            host_g.copy_(opt.flat_grad)
        except RuntimeError as exc:   # e.g. the host cannot pin the buffers of every rank
            host_g = None
            breakdown["e2e_skipped"] = str(exc)[:200]
        everyone = torch.tensor([1.0 if host_g is not None else 0.0], device=device)
        dist.all_reduce(everyone, op=dist.ReduceOp.MIN)
        if float(everyone) > 0:
            # The read-back of step k runs on its own stream and overlaps the gradients of step k + 1 coming in
            # (PCIe carries both directions at once); step k + 1 starts only when the read-back of step k has
            # finished on this rank, and its opening barrier makes that true for every rank before any rank's
            # kernels store new parameters into the others' buffers.
            main = torch.cuda.current_stream(device)
            out = torch.cuda.Stream(device)
            left = [None]

            def e2e_step():
                opt.flat_grad.copy_(host_g, non_blocking=True)
                if left[0] is not None:
                    main.wait_event(left[0])
                step()
                stepped = torch.cuda.Event()
                stepped.record(main)
                out.wait_event(stepped)
                with torch.cuda.stream(out):
                    host_p.copy_(opt.flat_param, non_blocking=True)
                    left[0] = torch.cuda.Event()
                    left[0].record(out)

            def e2e_steps(k):
                for _ in range(k):
                    e2e_step()
                main.wait_event(left[0])   # the timed region ends when the last parameters are on the host

            e2e_steps(1)
            dist.barrier()
            k = max(2, min(args.steps, 5))
            e2e_ms = timed(lambda: e2e_steps(k), 1) / k
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            nbytes = opt.flat_grad.numel() * opt.flat_grad.element_size()
            e2e = {"value": float(t), "unit": "ms", "h2d_bytes_per_step": nbytes * world,
                   "d2h_bytes_per_step": nbytes * world, "note": "per rank {} bytes each way".format(nbytes),
                   "host_params_match_device": bool(torch.equal(host_p[:1 << 20], opt.flat_param[:1 << 20].cpu()))}
    # for scale: NCCL's own all-reduce of one buffer of this size (the traffic of reduce-scatter + all-gather, nothing
    # computed), in place on the gradient buffer, whose values are not needed any more (last of all for that reason)
    try:
        for _ in range(2):
            dist.all_reduce(opt.flat_grad)
        nccl_ms = timed(lambda: dist.all_reduce(opt.flat_grad), 5)
        t = torch.tensor([nccl_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        breakdown["nccl_all_reduce_of_one_buffer_ms"] = float(t)
    except RuntimeError as exc:
        breakdown["nccl_all_reduce_of_one_buffer_ms"] = None
        breakdown["nccl_all_reduce_error"] = str(exc)[:120]

    return result, e2e


# DRAM bytes (read + write) per algorithmic byte of one launch of the staged step kernel, from an ncu
# capture of a 134 M-element launch of the same kernel (traffic grows in proportion to the elements).
STEP_KERNEL_DRAM_BYTES_PER_ALGORITHMIC_BYTE = {2: 0.967}


def run_gpu_arm(args, cfg, rank, world, local_rank):
    from gefen_b200 import Gefen

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    shapes, params, grads = build_model(cfg, device)
    named = [(name, torch.nn.Parameter(p)) for (name, _), p in zip(shapes, params)]
    for (_, p), g in zip(named, grads):
        p.grad = g
    opt = Gefen(named, lr=cfg["lr"], betas=(0.9, 0.999), eps=1e-8, weight_decay=cfg["wd"])
    step = opt.step

    # first step = calibration (period scan, histogram, exact-DP codebook) + one optimizer step
    calibration_ms = timed(step, 1)
    warm = max(args.warmup - 1, 2)
    sampler = ClockSampler(local_rank)
    sampler.start()   # nvidia-smi needs a moment to start: begin before the warm-up
    for _ in range(warm):
        step()
    ms = timed(step, args.steps)
    # the timed region is a few tens of milliseconds, shorter than the sampling period: keep the same
    # load running (untimed) until the sampler has seen it
    for _ in range(int(400.0 / max(ms, 0.05)) + 1):
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    opt.check()

    per_tensor = [opt.state[p]["automatic_period"] for _, p in named]
    elem_bytes = params[0].element_size()
    total_elems = sum(workloads.numel(s) for _, s in shapes)
    algo_bytes = workloads.step_bytes(shapes, per_tensor, elem_bytes, elem_bytes)
    result = {"ms": ms, "calibration_ms": calibration_ms, "clocks": clocks, "algo_bytes": algo_bytes,
              "total_elems": total_elems, "n_tensors": len(shapes), "periods": per_tensor, "shapes": shapes}

    # ---- roofline of the dominant kernel: the staged vector step over all its tensors, one launch
    from gefen_b200 import _lib

    lib = _lib.load()
    table = next(t for t in opt._plan.tables)
    rows = table["rows"]
    cls = [lib.gefen_b200_step_tensor_class(rows[r:r + 1].ctypes.data, table["tag"]) for r in range(len(rows))]

    def row_bytes(r):
        return int(r["num_blocks"]) * int(r["period"]) * (3 * elem_bytes + 2) + int(r["num_blocks"]) * 4 * elem_bytes

    # (the staged kernel comes in two kinds, one launch each: class 1 = one block per warp pass, class 2 = several
    # blocks of up to 1024 elements per warp pass; the roofline is reported for the one that moves more bytes)
    by_class = {c: sum(row_bytes(rows[r]) for r, k in enumerate(cls) if k == c) for c in (1, 2)}
    top = 1 if by_class[1] >= by_class[2] else 2
    vec_rows = rows[[r for r, c in enumerate(cls) if c == top]].copy()
    vec_bytes = int(sum(row_bytes(r) for r in vec_rows))
    dev_table = torch.empty(vec_rows.nbytes, dtype=torch.uint8, device=device)
    ws = _lib.codebook_workspace(opt._gefen_codebook)

    def vec_only():
        _lib.check(lib.gefen_b200_multi_tensor_step(vec_rows.ctypes.data, _lib.ptr(dev_table), len(vec_rows),
                                                    table["tag"], _lib.ptr(ws), _lib.current_stream(device)))

    for _ in range(3):
        vec_only()
    vec_ms = timed(vec_only, max(args.steps, 5))
    peak, peak_kind = measured_peaks()
    achieved = vec_bytes / vec_ms / 1e6
    ratio = STEP_KERNEL_DRAM_BYTES_PER_ALGORITHMIC_BYTE.get(elem_bytes)
    result["roofline"] = {"bound": "hbm", "kernel": "step_vec_kernel<{}, {}>".format(
                              "bf16" if elem_bytes == 2 else "f32",
                              "one block per warp pass" if top == 1 else "several blocks per warp pass"),
                          "achieved": achieved, "peak": peak, "peak_kind": peak_kind + " copy bandwidth, burst",
                          "unit": "GB/s", "frac": achieved / peak,
                          "traffic": ratio * vec_bytes if ratio is not None else None,
                          "algorithmic_bytes_per_launch": vec_bytes, "launch_ms": vec_ms}
    result["launches_per_step"] = len(set(cls))

    # ---- end to end through the public API with HOST buffers: gradients come from pinned host
    # memory every step and the updated parameters go back to pinned host memory
    # (gefen_b200.HostStreamedGefen: the same step, bucket by bucket, copies overlapped both ways).
    e2e = None
    if not args.no_e2e:
        from gefen_b200.host_stream import HostStreamedGefen

        host_g = [torch.empty(g.shape, dtype=g.dtype, pin_memory=True) for g in grads]
        host_p = [torch.empty(p.shape, dtype=p.dtype, pin_memory=True) for p in params]
        for h, g in zip(host_g, grads):
            h.copy_(g)
        streamed = HostStreamedGefen(opt, host_g, host_p, buckets=args.e2e_buckets)

        def e2e_step():
            streamed.step()

        e2e_step()
        e2e_ms = timed(e2e_step, max(2, min(args.steps, 5)))
        nbytes = sum(g.numel() * g.element_size() for g in grads)
        e2e = {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
               "buckets": len(streamed.buckets or []),
               # after the timed steps the host copies must be the device's parameters, element for element
               "host_params_match_device": all(torch.equal(h, p.detach().cpu()) for h, p in zip(host_p, params))}
        del streamed, host_g, host_p

    # ---- the reference's own CUDA kernels on the same tensors, in the reference's launch order
    if not args.no_reference_cuda:
        result["reference_cuda"] = reference_cuda_step_ms(shapes, params, grads, per_tensor, opt, cfg, max(3, min(args.steps, 5)), ms)
    return result, e2e


def reference_cuda_step_ms(shapes, params, grads, periods, opt, cfg, steps, own_ms):
    """The reference's CUDA kernels (compiled unmodified for sm_100a, the second checker of the tests) stepping
    the whole parameter set the way the reference optimizer launches them: per tensor the second-moment
    kernel, the weight-decay multiply and the fused step kernel (reference: gefen.py:1276-1311; period-1
    tensors through their own kernel, :1299). A measured comparison beside the product's number; it runs
    after the timed region on fresh state and the product's periods and codebook."""
    try:
        from oracle import build_ref

        ext = build_ref.load_module()
    except Exception as exc:   # the checker is optional
        return {"unavailable": "{}: {}".format(type(exc).__name__, str(exc)[:120])}
    if ext is None:
        return {"unavailable": "the reference kernels have not been built on this machine"}
    lr, wd, beta1, beta2, eps = cfg["lr"], cfg["wd"], 0.9, 0.999, 1e-8
    codebook = opt._gefen_codebook
    state = []
    for p, period in zip(params, periods):
        n, dev, dt = p.numel(), p.device, p.dtype
        st = {"codes": torch.zeros(n // period, period, dtype=torch.uint8, device=dev)}
        if period == 1:
            st["divisor"] = opt._period_one_divisor_for_numel(n)
            st["mag"] = torch.zeros(n // st["divisor"], 1, dtype=dt, device=dev)
            st["v"] = torch.zeros(n, 1, dtype=dt, device=dev)
        else:
            st["mag"] = torch.zeros(n // period, 1, dtype=dt, device=dev)
            st["v"] = torch.zeros(n // period, 1, dtype=dt, device=dev)
        state.append(st)
    counter = [0]

    def step():
        counter[0] += 1
        bc1, bc2 = 1 - beta1 ** counter[0], 1 - beta2 ** counter[0]
        for p, g, st, period in zip(params, grads, state, periods):
            flat = g.reshape(-1)
            if period != 1:
                view = flat.view(-1, period)
                ext.automatic_vmean_update_cuda(st["v"], view, beta2)
                if wd > 0.0:
                    p.mul_(1 - lr * wd)
                ext.automatic_gefen_fused_update_from_vmean_cuda(p, view, st["codes"], st["mag"], st["v"], codebook, False,
                                                                 beta1, lr, bc1, bc2, eps)
            else:
                if wd > 0.0:
                    p.mul_(1 - lr * wd)
                ext.automatic_gefen_period1_update_cuda(p, flat, st["codes"], st["mag"], st["v"], codebook, st["divisor"],
                                                        beta1, beta2, lr, bc1, bc2, eps)

    with torch.no_grad():
        for _ in range(2):
            step()
        # the reference launches on the legacy default stream: time with events on that stream
        ms = timed(step, steps)
    launches = sum(3 if period != 1 else 2 for period in periods) if wd > 0.0 else sum(2 if period != 1 else 1 for period in periods)
    return {"value": ms, "unit": "ms", "ratio_to_this_library": ms / own_ms, "kernel_launches_per_step": launches,
            "what": "the reference's own CUDA kernels compiled for sm_100a, its per-tensor launch order, same tensors"}


def ns_flops(shape, steps=5):
    m, n = min(shape), max(shape)
    return steps * (4 * m * m * n + 2 * m ** 3)


def run_muon_sharded_arm(args, cfg, rank, world, local_rank):
    """GefenMuon with whole matrices assigned to the ranks (Zero1GefenMuon): reduce-scatter of the
    gradients, GefenMuon on the owned matrices, all-gather of the parameters."""
    import torch.distributed as dist

    from gefen_b200 import newton_schulz as ns
    from gefen_b200.zero1 import Zero1GefenMuon

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    shapes, params, grads = build_model(cfg, device)
    named = [(name, torch.nn.Parameter(p)) for (name, _), p in zip(shapes, params)]
    for (_, p), g in zip(named, grads):
        p.grad = g
    opt = Zero1GefenMuon(named, lr=cfg["lr"], weight_decay=cfg["wd"], momentum=0.95, ns_steps=5)
    calibration_ms = timed(opt.step, 1)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup - 1, 2)):
        opt.step()
    dist.barrier()
    ms = timed(opt.step, args.steps)
    t = torch.tensor([ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    breakdown = opt.last_breakdown_ms()
    for _ in range(int(400.0 / max(float(t), 0.05)) + 1):   # same load until the clock sampler has seen it
        opt.step()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ns.check_status(device)
    n_vs_1 = opt.verify_against_single_process(steps=2, max_elements=40 << 20)
    if rank != 0:
        return
    elems = sum(workloads.numel(s) for _, s in shapes)
    owned = len(opt.pieces)
    print(json.dumps({
        "metric": "optimizer_step_ms", "value": float(t), "unit": "ms", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(t), "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "optimizer": "GefenMuon(momentum=0.95, ns_steps=5)", "lr": cfg["lr"],
                   "weight_decay": cfg["wd"], "matrices": len(shapes), "elements": elems,
                   "parallelism": "zero1-dp{} (whole matrices per rank)".format(world)},
        "calibration_first_step_ms": calibration_ms, "clocks": clocks, "breakdown_ms": breakdown, "n_vs_1": n_vs_1,
        "gpu_launches": args.steps * (owned * 15 + 8),
    }))


def torch_newton_schulz(grad, coefficients=(3.4445, -4.7750, 2.0315), steps=5, eps=1e-7):
    """The reference's Newton-Schulz chain on torch's (cuBLAS) GEMMs (reference: gefen_muon.py:16-51): the
    library path this library's tcgen05 kernels are compared with. Benchmark-side only."""
    a, b, c = coefficients
    x = grad.bfloat16()
    transposed = x.size(0) > x.size(1)
    if transposed:
        x = x.T
    x = x / x.norm().clamp(min=eps)
    for _ in range(steps):
        gram = x @ x.T
        gram_update = torch.addmm(gram, gram, gram, beta=b, alpha=c)
        x = torch.addmm(x, gram_update, x, beta=a)
    return x.T if transposed else x


def measure_muon(cfg, steps: int, warmup: int):
    """GefenMuon on the Qwen3-1.7B-shaped matrices, one GPU: the whole step, then Newton-Schulz alone on this
    library's tcgen05 GEMMs and on torch's (cuBLAS) GEMMs for the same inputs."""
    from gefen_b200 import GefenMuon
    from gefen_b200 import newton_schulz as ns

    device = torch.device("cuda", torch.cuda.current_device())
    shapes, params, grads = build_model(cfg, device)
    named = [(name, torch.nn.Parameter(p)) for (name, _), p in zip(shapes, params)]
    for (_, p), g in zip(named, grads):
        p.grad = g
    opt = GefenMuon(named, lr=cfg["lr"], weight_decay=cfg["wd"], momentum=0.95, ns_steps=5)
    calibration_ms = timed(opt.step, 1)
    for _ in range(max(warmup - 1, 2)):
        opt.step()
    sampler = ClockSampler(device.index)
    sampler.start()
    ms = timed(opt.step, steps)
    clocks = sampler.stop()
    opt.check()
    total_flops = sum(ns_flops(s) for _, s in shapes)
    coeffs = (3.4445, -4.7750, 2.0315)

    def ns_ours():   # the optimizer's own path: the chains of two matrices side by side
        ns.orthogonalize_all([(g, coeffs, 5, 1e-7) for g in grads], lambda i, ortho: None)

    def ns_torch():
        for g in grads:
            torch_newton_schulz(g, coeffs, 5, 1e-7)

    results = {}
    for name, fn in (("tcgen05", ns_ours), ("torch", ns_torch)):
        fn()
        results[name] = timed(fn, max(2, min(steps, 5)))
    ns.check_status(device)
    peak_file = ROOT / "MEASURED_PEAKS.json"
    peak = json.loads(peak_file.read_text())["bf16_tflops_sustained"] if peak_file.exists() else 1400.0
    achieved = total_flops / results["tcgen05"] / 1e9
    elems = sum(workloads.numel(s) for _, s in shapes)
    roofline = {"bound": "tensor", "kernel": "ns_gemm_tn_kernel", "achieved": achieved, "peak": peak,
                "peak_kind": "measured cuBLAS bf16, sustained", "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": None, "algorithmic_flops_per_step": total_flops,
                "newton_schulz_ms": results["tcgen05"],
                "newton_schulz_ms_torch_cublas": results["torch"],
                "torch_cublas_tflops": total_flops / results["torch"] / 1e9}
    summary = {"workload": "qwen3_muon", "matrices": len(shapes), "elements": elems, "step_ms": ms,
               "newton_schulz_ms": results["tcgen05"], "newton_schulz_tflops": achieved,
               "frac_of_bf16_tflops_sustained": achieved / peak,
               "torch_cublas_chain_ms": results["torch"], "calibration_first_step_ms": calibration_ms}
    return {"ms": ms, "calibration_ms": calibration_ms, "clocks": clocks, "roofline": roofline, "summary": summary,
            "shapes": shapes, "elements": elems}


def run_muon_arm(args, cfg):
    m = measure_muon(cfg, args.steps, args.warmup)
    line = {
        "metric": "optimizer_step_ms", "value": m["ms"], "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": m["ms"], "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": args.workload, "optimizer": "GefenMuon(momentum=0.95, ns_steps=5)", "lr": cfg["lr"],
                   "weight_decay": cfg["wd"], "matrices": len(m["shapes"]), "elements": m["elements"]},
        "calibration_first_step_ms": m["calibration_ms"], "clocks": m["clocks"],
        "roofline": m["roofline"],
        "gpu_launches": args.steps * (len(m["shapes"]) * 15 + 8),
    }
    print(json.dumps(line))


def run_flat_sweep(args):
    """Flat-tensor sweep: one fp32 parameter tensor and gradient of 2^20 ... 2^30 elements, gradients N(0,1) times
    a log-normal scale per 4096-element run. Per size: one fused step (steady state) and every pass of the
    calibration on its own (period scan of all candidate periods, exact histogram, exact-DP codebook fit, one
    Lloyd-Max accumulation), each as ms and as GB/s of its algorithmic bytes (step: 14 B per element; a
    calibration pass: one 4-byte read per element) against the measured copy bandwidth."""
    from gefen_b200 import Gefen, partitioning, quantization
    from gefen_b200.kernels.exact_histogram_fused import gefen_exact_histogram_cuda
    from gefen_b200.kernels.lloyd_max_fused import gefen_lloyd_accumulate_cuda

    device = torch.device("cuda", 0)
    peak, peak_kind = measured_peaks()
    rows = []
    for log2n in (20, 24, 28, 30):
        if log2n > args.sweep_max_log2:
            continue
        n = 1 << log2n
        gen = torch.Generator(device=device).manual_seed(log2n)
        g = torch.randn(n // 4096, 4096, generator=gen, device=device)
        g.mul_(torch.exp(torch.randn(n // 4096, 1, generator=gen, device=device)))
        g = g.reshape(-1)
        p = torch.nn.Parameter(torch.randn(n, generator=gen, device=device) * 0.02)
        p.grad = g
        opt = Gefen([p], lr=1e-3)
        first_ms = timed(opt.step, 1)
        period = opt.state[p]["automatic_period"]
        for _ in range(3):
            opt.step()
        k = max(3, min(args.steps, 20 if log2n <= 24 else 5))
        step_ms = timed(opt.step, k)
        opt.check()
        step_bytes = 14 * n + (n // period) * 16

        def scan():
            return partitioning.find_period_by_block_variance(g, print_results=False, backend="cuda_kernel",
                                                              input_is_squared=False)

        scan()
        scan_ms = timed(scan, 3)
        counts = torch.zeros(4096, dtype=torch.int64, device=device)
        gefen_exact_histogram_cuda(g, period, counts)
        hist_ms = timed(lambda: gefen_exact_histogram_cuda(g, period, counts), 5)
        counts.zero_()
        gefen_exact_histogram_cuda(g, period, counts)
        host = counts.cpu().to(torch.float32)
        edges = torch.linspace(-1.0, 1.0, steps=4097, dtype=torch.float32)
        centers = 0.5 * (edges[:-1] + edges[1:])
        active = host > 0
        stats = {"active_centers": centers[active], "active_counts": host[active]}
        quantization.exact_dp(stats, 256, True, device=device)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        quantization.exact_dp(stats, 256, True, device=device)
        dp_ms = 1e3 * (time.perf_counter() - t0)
        cb = opt._gefen_codebook
        sums = torch.zeros(256, device=device)
        cnts = torch.zeros(256, dtype=torch.int64, device=device)
        gefen_lloyd_accumulate_cuda(g, cb, period, sums, cnts)
        lloyd_ms = timed(lambda: gefen_lloyd_accumulate_cuda(g, cb, period, sums, cnts), 5)
        read_bytes = 4 * n

        def gbs(nbytes, ms):
            return nbytes / ms / 1e6

        rows.append({"log2_elements": log2n, "period": period, "first_step_ms_with_calibration": first_ms,
                     "step_ms": step_ms, "step_gbs": gbs(step_bytes, step_ms), "step_frac": gbs(step_bytes, step_ms) / peak,
                     "period_scan_ms": scan_ms, "period_scan_gbs": gbs(read_bytes, scan_ms),
                     "histogram_ms": hist_ms, "histogram_gbs": gbs(read_bytes, hist_ms), "histogram_frac": gbs(read_bytes, hist_ms) / peak,
                     "exact_dp_ms": dp_ms, "active_bins": int(active.sum()),
                     "lloyd_accumulate_ms": lloyd_ms, "lloyd_accumulate_gbs": gbs(read_bytes, lloyd_ms),
                     "lloyd_accumulate_frac": gbs(read_bytes, lloyd_ms) / peak})
        del opt, p, g
        torch.cuda.empty_cache()
    print(json.dumps({"metric": "flat_sweep", "unit": "ms and GB/s", "n_gpus": 1, "dtype": "f32", "data": "synthetic",
                      "peak_gbs": peak, "peak_kind": peak_kind + " copy bandwidth",
                      "config": {"workload": "flat_sweep", "optimizer": "Gefen(fused=True)", "lr": 1e-3,
                                 "note": "L2 is flushed by the inputs themselves from 2^24 elements on; the 2^20 point "
                                         "(14 MB per step) runs out of L2"},
                      "sweep": rows}))


def run_microbench(spec: str, steps: int, warmup: int):
    """Single-tensor step kernel on seeded random state, e.g. bf16:2048:65536 = dtype:period:blocks.
    Small enough for profiler captures; prints one JSON line."""
    from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_fused_update_from_vmean_cuda

    if spec.split(":")[0] in ("gemm", "gram", "hist", "scan", "ns", "dp", "lloyd", "vmean", "muonmom"):
        return run_microbench_other(spec, steps, warmup)
    name, period, blocks = spec.split(":")
    period, blocks = int(period), int(blocks)
    dtype = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[name]
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    inner = torch.sort(torch.tanh(torch.randn(254, generator=gen, device=dev) * 0.6)).values
    cb = torch.cat([torch.tensor([-1.0], device=dev), inner, torch.tensor([1.0], device=dev)]).float().contiguous()
    g = (torch.randn(blocks, period, generator=gen, device=dev) * 1e-3).to(dtype)
    p = (torch.randn(blocks, period, generator=gen, device=dev) * 0.02).to(dtype)
    codes = torch.randint(0, 256, (blocks, period), dtype=torch.uint8, generator=gen, device=dev)
    mag = (torch.rand(blocks, 1, generator=gen, device=dev) * 2e-3).to(dtype)
    v = (torch.rand(blocks, 1, generator=gen, device=dev) * 1e-6 + 1e-9).to(dtype)
    args = (0.9, 3e-4, 1 - 0.9 ** 3, 1 - 0.999 ** 3, 1e-8)

    def once():
        automatic_gefen_fused_update_from_vmean_cuda(p, g, codes, mag, v, cb, False, *args)

    for _ in range(max(warmup, 3)):
        once()
    ms = timed(once, steps)
    bytes_per_launch = blocks * period * (3 * p.element_size() + 2) + blocks * 4 * p.element_size()
    peak, kind = measured_peaks()
    print(json.dumps({"microbench": spec, "ms_per_launch": ms, "algorithmic_bytes": bytes_per_launch,
                      "achieved_gbs": bytes_per_launch / ms / 1e6, "frac_of_{}_peak".format(kind): bytes_per_launch / ms / 1e6 / peak}))


def run_microbench_other(spec: str, steps: int, warmup: int):
    """gemm:M:N:K (tcgen05 GEMM, K-major operands), hist:dtype:rows:cols (exact histogram, period = cols),
    scan:dtype:rows:cols (all candidate periods of one tensor)."""
    parts = spec.split(":")
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    out = {"microbench": spec}
    if parts[0] == "ns":
        from gefen_b200 import newton_schulz as ns

        rows, cols = int(parts[1]), int(parts[2])
        g = (torch.randn(rows, cols, generator=gen, device=dev) * 1e-3).bfloat16()
        coeffs = (3.4445, -4.7750, 2.0315)
        res = {}
        for mode, fn in (("tcgen05", lambda: ns.zeropower_via_newtonschulz(g, coeffs, 5, 1e-7)),
                         ("torch", lambda: torch_newton_schulz(g, coeffs, 5, 1e-7))):
            for _ in range(max(warmup, 3)):
                fn()
            res[mode] = timed(fn, steps)
        ns.check_status(dev)
        flops = ns_flops((rows, cols))
        out.update({"ms": res["tcgen05"], "tflops": flops / res["tcgen05"] / 1e9, "torch_ms": res["torch"],
                    "torch_tflops": flops / res["torch"] / 1e9})
        print(json.dumps(out))
        return
    if parts[0] in ("vmean", "muonmom"):
        # vmean:dtype:blocks:period - the stand-alone second-moment kernel (one read of the gradient);
        # muonmom:dtype:blocks:period - GefenMuon's 8-bit momentum step (codes in and out, gradient in, the
        # dequantised momentum out: 2 + 2 s bytes per element)
        from gefen_b200.kernels.automatic_gefen_fused import automatic_gefen_muon_momentum_cuda
        from gefen_b200.kernels.automatic_vmean import automatic_vmean_update_cuda

        dtype = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[parts[1]]
        blocks, period = int(parts[2]), int(parts[3])
        g = (torch.randn(blocks, period, generator=gen, device=dev) * 1e-3).to(dtype)
        esize = g.element_size()
        if parts[0] == "vmean":
            v = (torch.rand(blocks, 1, generator=gen, device=dev) * 1e-6 + 1e-9).to(dtype)
            fn = lambda: automatic_vmean_update_cuda(v, g, 0.999)   # noqa: E731
            nbytes = blocks * period * esize + blocks * 2 * esize
        else:
            inner = torch.sort(torch.tanh(torch.randn(254, generator=gen, device=dev) * 0.6)).values
            cb = torch.cat([torch.tensor([-1.0], device=dev), inner, torch.tensor([1.0], device=dev)]).float().contiguous()
            codes = torch.randint(0, 256, (blocks, period), dtype=torch.uint8, generator=gen, device=dev)
            mag = (torch.rand(blocks, 1, generator=gen, device=dev) * 2e-3).to(dtype)
            upd = torch.empty_like(g)
            fn = lambda: automatic_gefen_muon_momentum_cuda(g, codes, mag, cb, upd, False, 0.95)   # noqa: E731
            nbytes = blocks * period * (2 + 2 * esize) + blocks * 2 * esize
        for _ in range(max(warmup, 3)):
            fn()
        ms = timed(fn, steps)
        peak, kind = measured_peaks()
        out.update({"ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ms / 1e6,
                    "frac_of_{}_peak".format(kind): nbytes / ms / 1e6 / peak})
        print(json.dumps(out))
        return
    if parts[0] == "dp":
        # dp:active_bins:entries - the exact-DP codebook fit on a synthetic bell-shaped histogram
        from gefen_b200 import quantization

        active, k = int(parts[1]), int(parts[2])
        centers = torch.linspace(-1.0, 1.0, active)
        counts = (torch.exp(-0.5 * (centers / 0.3) ** 2) * 1e6 + 1.0).float()
        stats = {"active_centers": centers, "active_counts": counts}
        quantization.exact_dp(stats, k, True, device=dev)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            quantization.exact_dp(stats, k, True, device=dev)
        out.update({"ms": 1e3 * (time.perf_counter() - t0) / steps, "active_bins": active, "entries": k})
        print(json.dumps(out))
        return
    if parts[0] == "lloyd":
        # lloyd:dtype:rows:cols - one Lloyd-Max accumulation pass (period = cols, capped as for hist)
        from gefen_b200.kernels.lloyd_max_fused import gefen_lloyd_accumulate_cuda

        dtype = {"bf16": torch.bfloat16, "f32": torch.float32}[parts[1]]
        rows, cols = int(parts[2]), int(parts[3])
        flat = workloads.make_grad((rows, cols), 0, 0, dtype, dev).reshape(-1)
        period = cols if cols <= 1024 else 2048
        inner = torch.sort(torch.tanh(torch.randn(254, generator=gen, device=dev) * 0.6)).values
        cb = torch.cat([torch.tensor([-1.0], device=dev), inner, torch.tensor([1.0], device=dev)]).float().contiguous()
        sums = torch.zeros(256, device=dev)
        counts = torch.zeros(256, dtype=torch.int64, device=dev)
        for _ in range(max(warmup, 3)):
            gefen_lloyd_accumulate_cuda(flat, cb, period, sums, counts)
        ms = timed(lambda: gefen_lloyd_accumulate_cuda(flat, cb, period, sums, counts), steps)
        peak, kind = measured_peaks()
        gbs = flat.numel() * flat.element_size() / ms / 1e6
        out.update({"ms": ms, "period": period, "achieved_gbs": gbs, "frac_of_{}_peak".format(kind): gbs / peak})
        print(json.dumps(out))
        return
    if parts[0] == "gram":
        # gram:M:K - the two symmetric products of a Newton-Schulz step: G = X X^T and b G + c G G
        from gefen_b200.newton_schulz import check_status, gemm_tn

        M, K = (int(x) for x in parts[1:])
        x = (torch.randn(M, K, generator=gen, device=dev) / K ** 0.5).bfloat16()
        g = torch.empty(M, M, dtype=torch.bfloat16, device=dev)
        poly = torch.empty(M, M, dtype=torch.bfloat16, device=dev)
        for _ in range(max(warmup, 3)):
            gemm_tn(x, x, out=g, symmetric=True)
            gemm_tn(g, g, c=g, alpha=2.0315, beta=-4.775, out=poly, symmetric=True)
        ms1 = timed(lambda: gemm_tn(x, x, out=g, symmetric=True), steps)
        ms2 = timed(lambda: gemm_tn(g, g, c=g, alpha=2.0315, beta=-4.775, out=poly, symmetric=True), steps)
        check_status(dev)
        out.update({"gram_ms": ms1, "gram_tflops": 2.0 * M * M * K / ms1 / 1e9, "poly_ms": ms2,
                    "poly_tflops": 2.0 * M * M * M / ms2 / 1e9})
        print(json.dumps(out))
        return
    if parts[0] == "gemm":
        from gefen_b200.newton_schulz import check_status, gemm_tn

        M, N, K = (int(x) for x in parts[1:])
        a = torch.randn(M, K, generator=gen, device=dev).bfloat16()
        b = torch.randn(N, K, generator=gen, device=dev).bfloat16()
        d = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        for _ in range(max(warmup, 3)):
            gemm_tn(a, b, out=d)
        ms = timed(lambda: gemm_tn(a, b, out=d), steps)
        check_status(dev)
        for _ in range(3):
            torch.mm(a, b.T)
        ref = timed(lambda: torch.mm(a, b.T), steps)
        out.update({"ms": ms, "tflops": 2.0 * M * N * K / ms / 1e9, "torch_matmul_ms": ref,
                    "torch_matmul_tflops": 2.0 * M * N * K / ref / 1e9})
    else:
        dtype = {"bf16": torch.bfloat16, "f32": torch.float32}[parts[1]]
        rows, cols = int(parts[2]), int(parts[3])
        g = workloads.make_grad((rows, cols), 0, 0, dtype, dev)
        flat = g.reshape(-1)
        if parts[0] == "hist":
            from gefen_b200.kernels.exact_histogram_fused import gefen_exact_histogram_cuda

            counts = torch.zeros(4096, dtype=torch.int64, device=dev)
            period = cols if cols <= 1024 else 2048
            for _ in range(max(warmup, 3)):
                gefen_exact_histogram_cuda(flat, period, counts)
            ms = timed(lambda: gefen_exact_histogram_cuda(flat, period, counts), steps)
            peak, kind = measured_peaks()
            gbs = flat.numel() * flat.element_size() / ms / 1e6
            out.update({"ms": ms, "period": period, "achieved_gbs": gbs, "frac_of_{}_peak".format(kind): gbs / peak})
        else:
            from gefen_b200 import partitioning

            def scan():
                return partitioning.find_period_by_block_variance(flat, print_results=False, backend="cuda_kernel",
                                                                  input_is_squared=False)

            for _ in range(max(warmup, 2)):
                period = scan()
            ms = timed(scan, steps)
            cands = partitioning.decision_periods(partitioning.candidate_periods(flat.numel()))
            out.update({"ms": ms, "period": period, "candidates": len(cands),
                        "achieved_gbs_one_read": flat.numel() * flat.element_size() / ms / 1e6})
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="gefen_b200", choices=["gefen_b200", "reference"])
    ap.add_argument("--workload", default="llama_1_5b", choices=sorted(WORKLOADS) + ["flat_sweep"])
    ap.add_argument("--cpu-sample-elems", type=int, default=62_000_000,
                    help="size of the CPU baseline's sample of the workload, in elements")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-buckets", type=int, default=32)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip timing the reference's CUDA kernels")
    ap.add_argument("--no-muon", action="store_true", help="skip the GefenMuon summary of the default line")
    ap.add_argument("--sweep-max-log2", type=int, default=30, help="flat_sweep: largest tensor, log2 of its elements")
    ap.add_argument("--microbench", default=None, help="dtype:period:blocks, single-tensor step kernel only")
    args = ap.parse_args()
    if args.microbench:
        run_microbench(args.microbench, args.steps, args.warmup)
        return
    if args.workload == "flat_sweep":
        run_flat_sweep(args)
        return
    cfg = WORKLOADS[args.workload]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, cfg, rank, world)
        return

    if cfg.get("muon"):
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device")
        if world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            try:
                run_muon_sharded_arm(args, cfg, rank, world, local_rank)
            finally:
                dist.destroy_process_group()
            return
        run_muon_arm(args, cfg)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: gefen_b200 has no CPU path (use --impl reference for the "
                         "CPU oracle port)")
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        result, e2e = run_sharded_arm(args, cfg, rank, world, local_rank)
    else:
        result, e2e = run_gpu_arm(args, cfg, rank, world, local_rank)
    if rank == 0:
        peak, peak_kind = measured_peaks()
        ms = result["ms"]
        eff_gbs = result["algo_bytes"] / ms / 1e6
        shapes, periods = result["shapes"], result["periods"]
        line = {
            "metric": "optimizer_step_ms", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": ms / PUBLISHED_LLAMA_1_5B_MS if args.workload == "llama_1_5b" else None,
            "vs_baseline_note": "reference README: Gefen step 29 ms for Llama 3 1.5B, hardware not stated",
            "dtype": "bf16" if cfg["dtype"] == torch.bfloat16 else "f32", "data": "synthetic",
            "config": workload_config(args, cfg, world, result["n_tensors"], result["total_elems"]),
            "periods": periods_found(shapes, periods),
            "effective_hbm_gbs": eff_gbs, "effective_hbm_frac_of_{}".format(peak_kind): eff_gbs * (1 if world == 1 else 1.0 / world) / peak,
            "algorithmic_bytes_per_step": result["algo_bytes"],
            "calibration_first_step_ms": result["calibration_ms"],
            "clocks": result["clocks"],
        }
        if "roofline" in result:
            line["roofline"] = result["roofline"]
            line["gpu_launches"] = result["launches_per_step"] * args.steps
        if "breakdown" in result:
            line["breakdown_ms"] = result["breakdown"]
            line["gpu_launches"] = result["breakdown"].get("kernel_launches_per_step", 0) * args.steps
            # N > 1: the step kernels carry both collectives and the links bound them. achieved = the bytes a rank
            # must move over NVLink per step (the larger direction) / the step time; peak = the measured rate of a
            # peer copy on this pool (one direction; nominal 900 GB/s)
            wire = result["breakdown"].get("wire_bytes_per_rank")
            if wire:
                line["roofline"] = {"bound": "nvlink", "kernel": "step kernels with both collectives on their accesses",
                                    "achieved": result["breakdown"]["achieved_link_gbs"], "peak": 770.0,
                                    "peak_kind": "measured peer copy, one direction", "unit": "GB/s",
                                    "frac": result["breakdown"]["achieved_link_gbs"] / 770.0, "traffic": None,
                                    "algorithmic_bytes_per_launch": max(wire["egress"], wire["ingress"])}
        if "n_vs_1" in result:
            line["n_vs_1"] = result["n_vs_1"]
        if "reference_cuda" in result:
            line["reference_cuda"] = result["reference_cuda"]
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.no_muon and args.workload == "llama_1_5b":
            # GefenMuon on the Qwen3-1.7B-shaped matrices, measured after everything above (its own tensors)
            torch.cuda.empty_cache()
            try:
                line["muon"] = measure_muon(WORKLOADS["qwen3_muon"], max(2, min(args.steps, 5)), 3)["summary"]
            except Exception as exc:   # the summary is an extra: never lose the headline line to it
                line["muon"] = {"unavailable": "{}: {}".format(type(exc).__name__, str(exc)[:160])}
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            run = cpu_port_run(cfg, 2, 1, args.cpu_sample_elems)
            scaled = run["ms"] * result["total_elems"] / run["elements"]
            line["cpu_baseline"] = {
                "value": scaled, "unit": "ms", "cores": run["cores"], "kind": "port",
                "sample": "{} of {} elements (the tensors of the first transformer layers, whole tensors): the C "
                          "oracle with OpenMP, its own calibration, {} steady-state steps at {:.0f} ms each, scaled "
                          "by element count to the whole workload (`--impl reference` runs the whole workload)"
                          .format(run["elements"], result["total_elems"], run["timed_steps"], run["ms"])}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
