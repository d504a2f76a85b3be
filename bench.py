"""Benchmark of the kernel-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--path auto|fma|tc]

Workload at the default settings: the spectral-mixture configuration (16 components sharing
x and rhs, m = n = 65536 sorted U[0, 500], l ~ LogUniform[0.5, 5], f ~ U[0, 2], cutoff 4 l,
rhs 65536 x 16; seeded synthetic inputs, ``kernel_matmul_b200/workloads.py``).  One step is one
pass of the hot path over that batch: the forward product ``K . rhs`` and the hyper-parameter
gradients ``matmul_bwd`` of all 16 components.  The metric is kernel entries x rhs columns per
second: a step processes ``2 * E * k`` units (E visited entries, once forward and once in the
gradient).

Printed keys (one JSON line, rank 0):
  value      whole-job units/s with inputs resident in HBM, CUDA-event time per step summed over
             K steps, L2 flushed between steps, max over ranks;
  e2e        the same metric through ``kernel_matmul_b200.host.matmul_and_grad_from_host`` with
             HOST (pinned) buffers: every step copies x, rhs, params and out_grad to the device,
             builds the band on the device, runs forward + gradient and copies out and grad back
             (copies on two extra streams, overlapping the kernels);
  roofline   the dominant kernel against the pipe that bounds it, measured live with the library's
             calibration kernels: the SFU rate for the tensor-core kernels (the contraction runs as
             tcgen05.mma; generating kappa costs 2-3 SFU operations per entry), the FP32 FFMA rate
             for the FMA-pipe kernels (FMA-equivalent TFLOP/s = 2 x FP32-pipe instructions);
  cpu_baseline  the dense PyTorch formulation (materialise K, mask by ranges, matmul, autograd)
             in fp32 on all host cores, on a bounded sample of the same workload.

With N > 1 (torchrun) every rank runs its own batch of 16 components with the same seeded
parameters (the same work per GPU at every N): independent work, no data-path collective, weak
scaling.

``--impl reference`` times only the CPU dense formulation (the reference has no CPU kernel of
its own for this path; the dense formulation is what its tests define as the expected result).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "kernel_entries_x_rhs_cols_per_s"
UNIT = "entry-cols/s"

# Algorithmic per-entry instruction budget of the FMA path (FP32-pipe instructions, SFU ops):
# generation + contraction.  Forward: k FFMA per entry; gradient: k FFMA for the coefficient
# <left_i, right_j> plus one FFMA per parameter.
GEN_FWD = {"rbf": (3, 1), "spectral": (5, 2), "locally_periodic": (6, 2)}
GEN_BWD = {"rbf": (4, 1), "spectral": (8, 3), "locally_periodic": (11, 3)}
NPARAMS = {"rbf": 2, "spectral": 3, "locally_periodic": 4}
# The tensor-core kernels contract on tcgen05.mma and factor the sine / cosine of a phase
# difference into per-row and per-column values, so an entry costs ONE SFU operation (ex2) and
# these FP32-pipe instructions (per entry; the kernels issue them packed, two entries each):
#   forward   tau, its envelope exponent, cos(W tau) = c_i c_j + s_i s_j, the product, + 2 for the
#             fp16 hi / lo split;
#   gradient  the same plus sin(W tau), the coefficient and one accumulation per parameter.
TC_FWD = {"rbf": (5, 1), "spectral": (8, 1), "locally_periodic": (9, 1)}
TC_BWD = {"rbf": (6, 1), "spectral": (13, 1), "locally_periodic": (15, 1)}


def fp32_instr_fwd(kt: str, k: int) -> int:
    return GEN_FWD[kt][0] + k


def fp32_instr_bwd(kt: str, k: int) -> int:
    return GEN_BWD[kt][0] + k + NPARAMS[kt]


# ------------------------------------------------------------------------------------ helpers


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons of one GPU while the timed region
    runs: a thread reading NVML every 10 ms (read-only queries; short timed regions still get
    samples, which a freshly spawned nvidia-smi would miss)."""

    REASONS = {  # NVML clocks-event-reason bits
        0x0000000000000008: "hw_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000004: "sw_power_cap",
    }

    def __init__(self, device_index: int):
        self.samples, self.max_mhz, self.reasons = [], None, set()
        self.stop_flag = threading.Event()
        self.thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except TypeError:
                handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def run():
                while not self.stop_flag.is_set():
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        bits = int(reasons_fn(handle))
                        for bit, name in self.REASONS.items():
                            if bits & bit:
                                self.reasons.add(name)
                    except Exception:  # noqa: BLE001 - a failed read is a missing sample
                        pass
                    self.stop_flag.wait(0.01)

            self.thread = threading.Thread(target=run, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001 - no NVML: report empty clocks
            self.thread = None

    def stop(self) -> dict:
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        sm = list(self.samples)
        busy = [v for v in sm if v > 0.5 * max(sm)] if sm else []
        return {
            "sm_mhz": statistics.median(busy) if busy else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(sm),
        }


def device_delay() -> None:
    """Keep the GPU busy for ~1 ms (touching no memory) so that the launches of the timed region
    are already queued when its first event is reached: the events then measure device time, not
    the host's enqueue latency (which the end-to-end figure covers)."""
    torch.cuda._sleep(2_000_000)


def cuda_ms(fn, stream=None) -> float:
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


# ----------------------------------------------------------------------------------- workload


def make_workload(name: str, rank: int):
    from kernel_matmul_b200 import workloads

    if name == "spectral_mixture":
        w = workloads.spectral_mixture()
    elif name == "spectral_mixture_small":
        w = workloads.spectral_mixture(n=8192, components=4, k=16, span=62.5)
    else:
        raise SystemExit(f"unknown workload {name}")
    return w


# -------------------------------------------------------------------------------- CPU baseline


def cpu_dense_sample(w, seconds: float = 12.0, max_seconds: float = 30.0) -> dict:
    """Dense formulation (oracle/dense_reference.py) in fp32 on all host cores: forward slab
    product + autograd gradient for row-block slabs of the workload, drawn round-robin over the
    components, until ``seconds`` of work are done.  Returns units/s."""
    from oracle import dense_reference as D
    from oracle import oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = w.x
    n = w.n
    k = w.rhs.shape[-1]
    B = w.params.shape[0]
    R = -(-n // 128)
    bands = [O.make_ranges(c, x) for c in w.cutoffs]
    units = 0
    entries = 0
    slabs = 0
    t0 = time.perf_counter()
    group = 8  # row blocks per slab
    order = [(b, r0) for p in range(16) for r0 in range(p * group, R, group * 16) for b in range(B)]
    for b, r0 in order:
        start, end = bands[b if len(bands) > 1 else 0]
        r1 = min(r0 + group, R)
        c0 = int(start[r0:r1].min())
        c1 = min(int(end[r0:r1].max()), n)
        rows = slice(r0 * 128, min(r1 * 128, n))
        p = w.params[b].clone().requires_grad_(True)
        K = D.kernel_matrix(w.kernel_type, x[rows], x[c0:c1], p)
        mask = D.band_mask(start[r0:r1] - c0, end[r0:r1] - c0, K.shape[0], c1 - c0)
        Km = torch.where(mask, K, torch.zeros((), dtype=K.dtype))
        out = Km @ w.rhs[c0:c1]
        out.backward(gradient=w.extra["out_grad"][b, rows])
        e = int(mask.sum())
        entries += e
        units += 2 * e * k
        slabs += 1
        el = time.perf_counter() - t0
        if el >= seconds or el >= max_seconds:
            break
    el = time.perf_counter() - t0
    return {
        "value": units / el,
        "unit": UNIT,
        "cores": cores,
        "kind": "port",
        "sample": f"{slabs} slabs of {group} row blocks ({entries} entries, fwd + autograd bwd, fp32) in {el:.1f} s",
        "seconds": el,
    }


# --------------------------------------------------------------------------------------- main


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    w = make_workload(args.workload, 0)
    per_step = max(2.0, min(10.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_dense_sample(w, seconds=per_step / 4, max_seconds=per_step)
    vals, secs = [], []
    base = None
    for _ in range(args.steps):
        base = cpu_dense_sample(w, seconds=per_step, max_seconds=2 * per_step)
        vals.append(base["value"])
        secs.append(base["seconds"])
    value = statistics.mean(vals)
    base["value"] = value
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(secs),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "what": "dense PyTorch formulation on host cores, bounded sample per step"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_cuda_timing(w, dev, xb, rhs, params, start, end, og) -> dict | None:
    """Times the reference's own CUDA kernels (compiled unmodified into oracle/_ref) on the same
    inputs, when those modules are present.  Informational: the generic-SIMT bar on this GPU."""
    import importlib.util

    out = {}
    try:
        k = rhs.shape[-1]
        for op, modname in (("fwd", f"km_ref_matmul_{w.kernel_type}_k{k}"), ("bwd", f"km_ref_matmul_bwd_{w.kernel_type}")):
            path = os.path.join(ROOT, "oracle", "_ref", modname, modname + ".so")
            if not os.path.exists(path):
                return None
            spec = importlib.util.spec_from_file_location(modname, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            fn = (lambda m=mod: m.call(xb, xb, rhs, params, start, end)) if op == "fwd" else (
                lambda m=mod: m.call(xb, xb, rhs, params, start, end, og))
            fn()
            torch.cuda.synchronize()
            # the reference launches on the legacy default stream: time with full device syncs
            ts = []
            for _ in range(3):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn()
                torch.cuda.synchronize()
                ts.append(1e3 * (time.perf_counter() - t0))
            out[f"{op}_ms"] = min(ts)
        return out
    except Exception as exc:  # noqa: BLE001 - informational only
        return {"error": str(exc)[:200]}


def run_ours(args, rank: int, world: int, local: int) -> None:
    import kernel_matmul_b200 as km  # raises if libkm_b200.so is missing: no fallback
    from kernel_matmul_b200 import ops, ranges, workloads
    from kernel_matmul_b200._lib import check, lib
    import ctypes

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    w = make_workload(args.workload, rank)
    kt = w.kernel_type
    n, k = w.n, w.rhs.shape[-1]
    B = w.params.shape[0]

    # ---- resident inputs
    x = w.x.to(dev)
    xb = x.expand(B, -1)
    rhs = w.rhs.to(dev).expand(B, -1, -1)
    params = w.params.to(dev)
    og = w.extra["out_grad"].to(dev)
    start, end = workloads.band(w, x)
    E = int(ops.count_entries(n, n, start, end))
    units_per_step = 2 * E * k

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB of L2

    path = args.path

    def step():
        out = ops.matmul(kt, xb, xb, rhs, params, start, end, path=path)
        g = ops.matmul_bwd(kt, xb, xb, rhs, params, start, end, og, path=path)
        return out, g

    for _ in range(max(args.warmup, 3)):
        out_w, g_w = step()
    torch.cuda.synchronize()
    # which kernels the ops chose (tensor cores for this width and size, else the FMA pipe);
    # a tensor-core kernel reports a bounded wait that gave up through its status word
    tc_fwd, tc_bwd = hasattr(out_w, "_km_workspace"), hasattr(g_w, "_km_workspace")
    if ops.tc_status(out_w) != 0 or ops.tc_status(g_w) != 0:
        raise RuntimeError("a tensor-core kernel reported a failed wait")

    # ---- live FP32 and SFU peaks (calibration kernels of the library)
    flops = ctypes.c_double()
    sfu_ops = ctypes.c_double()
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def probe():
        check(lib.km_probe_fp32_peak(20000, None, ctypes.byref(flops), stream))

    def probe_sfu():
        check(lib.km_probe_sfu_peak(20000, None, ctypes.byref(sfu_ops), stream))

    probe()
    fp32_peak = max(flops.value / (cuda_ms(probe) * 1e-3) for _ in range(3)) / 1e12
    probe_sfu()
    sfu_peak = max(sfu_ops.value / (cuda_ms(probe_sfu) * 1e-3) for _ in range(3)) / 1e12

    # ---- timed region
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    wall0 = time.perf_counter()
    step_ms, fwd_ms, bwd_ms = [], [], []
    for _ in range(args.steps):
        flush.fill_(1)
        device_delay()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        ops.matmul(kt, xb, xb, rhs, params, start, end, path=path)
        e1.record()
        ops.matmul_bwd(kt, xb, xb, rhs, params, start, end, og, path=path)
        e2.record()
        e2.synchronize()
        fwd_ms.append(e0.elapsed_time(e1))
        bwd_ms.append(e1.elapsed_time(e2))
        step_ms.append(e0.elapsed_time(e2))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - wall0
    total_ms = sum(step_ms)

    # ---- end to end with host buffers (pinned), copies inside the timed region
    hx = w.x.pin_memory()
    hrhs = w.rhs.contiguous().pin_memory()
    hp = w.params.contiguous().pin_memory()
    hog = w.extra["out_grad"].contiguous().pin_memory()
    hout = torch.empty(B, n, k).pin_memory()
    hgrad = torch.empty(B, w.params.shape[-1]).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (hx, hrhs, hp, hog))
    d2h = sum(t.numel() * t.element_size() for t in (hout, hgrad))

    from kernel_matmul_b200 import host

    host_streams = host.HostStreams(dev)

    def e2e_step():
        # copies in, band construction, product, gradient and copies out, overlapped on three streams
        host.matmul_and_grad_from_host(kt, hx, hrhs, hp, hog, lambda dx: workloads.band(w, dx), hout, hgrad,
                                       host_streams, path=path)

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = []
    for _ in range(args.steps):
        flush.fill_(1)
        e2e_ms.append(cuda_ms(e2e_step))
    clocks = sampler.stop()
    e2e_total = sum(e2e_ms)

    # ---- max over ranks
    if world > 1:
        t = torch.tensor([total_ms, e2e_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_total = float(t[0]), float(t[1])
        u = torch.tensor([float(units_per_step)], device=dev, dtype=torch.float64)
        dist.all_reduce(u, op=dist.ReduceOp.SUM)
        units_all = float(u[0])
    else:
        units_all = float(units_per_step)

    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = units_all / (ms_per_step * 1e-3)
        e2e_value = units_all / (e2e_total / args.steps * 1e-3)
        fwd = statistics.mean(fwd_ms)
        bwd = statistics.mean(bwd_ms)
        # Per-entry budgets.  FMA-pipe kernels: generation + k FMAs (+ P in the gradient).
        # Tensor-core kernels: the contraction runs as tcgen05.mma, the threads only generate
        # (forward: + 2 operations for the hi / lo split; gradient: + one FMA per parameter).
        fwd_name = "matmul_tc_kernel" if tc_fwd else "matmul_fma_kernel"
        bwd_name = "grad_tc_kernel" if tc_bwd else "grad_band_kernel"
        kernels = {
            fwd_name: {"ms": fwd, "sfu_per_entry": TC_FWD[kt][1] if tc_fwd else GEN_FWD[kt][1],
                       "contraction": "tcgen05.mma kind::f16 (fp16 hi/lo split)" if tc_fwd else "fma.rn.f32x2",
                       "fp32_instr_per_entry": TC_FWD[kt][0] if tc_fwd else fp32_instr_fwd(kt, k)},
            bwd_name: {"ms": bwd, "sfu_per_entry": TC_BWD[kt][1] if tc_bwd else GEN_BWD[kt][1],
                       "contraction": "tcgen05.mma kind::tf32 (3xTF32)" if tc_bwd else "fma.rn.f32x2",
                       "fp32_instr_per_entry": TC_BWD[kt][0] if tc_bwd else fp32_instr_bwd(kt, k)},
        }
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "dram_traffic.json")
        dom = max(kernels, key=lambda kname: kernels[kname]["ms"])
        if os.path.exists(tpath):
            traffic = json.load(open(tpath)).get(args.workload, {}).get(dom)
        for kname, kd in kernels.items():
            kd["achieved_tflops"] = 2.0 * E * kd["fp32_instr_per_entry"] / (kd["ms"] * 1e-3) / 1e12
            kd["frac_fp32"] = kd["achieved_tflops"] / fp32_peak
            kd["achieved_sfu_tops"] = E * kd["sfu_per_entry"] / (kd["ms"] * 1e-3) / 1e12
            kd["frac_sfu"] = kd["achieved_sfu_tops"] / sfu_peak
        d = kernels[dom]
        dom_tc = (dom == fwd_name and tc_fwd) or (dom == bwd_name and tc_bwd)
        if dom_tc and d["frac_sfu"] > d["frac_fp32"]:
            roof = {"bound": "sfu", "kernel": dom, "achieved": d["achieved_sfu_tops"], "peak": sfu_peak,
                    "unit": "Tops/s (special-function operations)", "frac": d["frac_sfu"], "traffic": traffic,
                    "peak_source": "measured live: km_probe_sfu_peak (ex2.approx issue rate of all SMs); achieved = "
                                   "algorithmic SFU operations per launch / CUDA-event time.  The contraction runs on "
                                   "the tensor cores (a few % of their peak at this width); what bounds the kernel is "
                                   "generating the kernel entries"}
        else:
            roof = {"bound": "fp32", "kernel": dom, "achieved": d["achieved_tflops"], "peak": fp32_peak,
                    "unit": "TFLOP/s", "frac": d["frac_fp32"], "traffic": traffic,
                    "peak_source": "measured live: km_probe_fp32_peak (FFMA issue rate of all SMs); achieved = 2 x "
                                   "algorithmic FP32-pipe instructions per launch / CUDA-event time"
                                   + (".  The contraction runs on the tensor cores (a few % of their peak at this "
                                      "width); what bounds the kernel is generating the kernel entries" if dom_tc else "")}
        peaks = {}
        ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(ppath):
            peaks = json.load(open(ppath))
        hbm_bytes = 4 * (n * k + B * n * k * 2 + n + 2 * B * (n // 128))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": w.name, "ops": "matmul fwd + matmul_bwd", "path": path, "entries_per_rank": E, "rhs_cols": k,
                "units_per_step": units_all, "l2": "flushed between steps (256 MB write)",
                "per_rank": "own batch of 16 components (same seeded parameters on every rank), no collective",
            },
            "roofline": {
                **roof,
                "fp32_peak_tflops": fp32_peak, "sfu_peak_tops": sfu_peak,
                "hbm": {"algorithmic_bytes_per_step": hbm_bytes,
                        "frac_of_measured_hbm": (hbm_bytes / (ms_per_step * 1e-3)) / (peaks.get("hbm_gbs", 6650.0) * 1e9)},
                "kernels": kernels,
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_total / args.steps},
            # forward: product kernel (+ column-maximum and image pre-passes on the tensor-core path);
            # gradient: band kernel + finish kernel (+ image pre-pass on the tensor-core path)
            "gpu_launches": ((3 if tc_fwd else 1) + (3 if tc_bwd else 2)) * args.steps,
            "clocks": clocks,
            "wall_s": wall,
        }
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_dense_sample(w)
        ref_cuda = reference_cuda_timing(w, dev, xb, rhs, params, start, end, og)
        if ref_cuda is not None:
            line["reference_cuda_kernels_same_gpu"] = ref_cuda
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_cg(args, rank: int, world: int, local: int) -> None:
    """Config-5 style workload: (K + sigma^2 I) V = Y by CG, K the sum of 64 spectral components
    (shared band), rows sharded over the ranks, one NCCL all-gather per iteration.  One step =
    one CG iteration (sharded product + all-gather + replicated vector updates); total work is
    fixed, so scaling is strong."""
    import ctypes

    import kernel_matmul_b200  # noqa: F401
    from kernel_matmul_b200 import ops, workloads
    from kernel_matmul_b200._lib import check, lib
    from kernel_matmul_b200.cg import CGSolver, ShardedOperator, conjugate_gradient

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    w = workloads.cg_sum_kernel() if args.workload == "cg_sum" else workloads.cg_sum_kernel(n=1 << 17, components=8, span=625.0)
    kt, n, k, B = w.kernel_type, w.n, w.rhs.shape[-1], w.params.shape[0]
    x = w.x.to(dev)
    params = w.params.to(dev)
    y = w.rhs.to(dev)
    start, end = workloads.band(w, x)
    E = int(ops.count_entries(n, n, start, end))  # over all components
    units = float(E) * k
    op = ShardedOperator.from_kernel(kt, x, params, start[0], end[0], w.extra["sigma2"])

    flops = ctypes.c_double()
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def probe():
        check(lib.km_probe_fp32_peak(20000, None, ctypes.byref(flops), stream))

    probe()
    fp32_peak = max(flops.value / (cuda_ms(probe) * 1e-3) for _ in range(3)) / 1e12
    sm_clock = fp32_peak * 1e12 / (148 * 128 * 2)

    # a running solve: a few iterations are warm-up, then K timed iterations
    solver = CGSolver(op, y)
    for _ in range(max(args.warmup, 3)):
        solver.step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        solver.step()
    t1.record()
    t1.synchronize()
    total_ms = t0.elapsed_time(t1)
    # the product alone (this rank's rows, no collective)
    apply_ms = statistics.mean(cuda_ms(lambda: op.apply_rows(solver.p)) for _ in range(3))
    clocks = sampler.stop()

    # end to end: host y in, solution out, full solve of `iters` iterations
    iters = int(w.extra["iterations"]) if args.workload == "cg_sum" and world > 1 else min(int(w.extra["iterations"]), 10)
    hy = w.rhs.contiguous().pin_memory()
    hx = w.x.pin_memory()
    hp = w.params.contiguous().pin_memory()
    hsol = torch.empty(n, k).pin_memory()

    def solve_e2e():
        dx = hx.to(dev, non_blocking=True)
        dp = hp.to(dev, non_blocking=True)
        dy = hy.to(dev, non_blocking=True)
        st, en = workloads.band(w, dx)
        o = ShardedOperator.from_kernel(kt, dx, dp, st[0], en[0], w.extra["sigma2"])
        res = conjugate_gradient(o, dy, iterations=iters)
        hsol.copy_(res.solution, non_blocking=True)

    e2e_ms = cuda_ms(solve_e2e)
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms, apply_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, apply_ms = (float(v) for v in t)
    if rank == 0:
        ms_per_step = total_ms / args.steps
        # All components share inputs, band and lengthscale, so the batch sum runs on the tensor
        # cores (matmul_sum_tc_kernel): sum_b s_b cos(w_b tau) = <phi(x_i), psi(x_j)> with 2B-vectors
        # of per-point phases.  Per UNIQUE (row, column) entry: one envelope exponential + 2B / 128
        # SFU operations for the column's phase vector (shared by the 128 rows of the block), three
        # fp16 MMAs of 2B multiply-adds, and k + ~6 FP32 operations.
        e_unique = E / B / world  # row windows are equal
        t_apply = apply_ms * 1e-3
        tensor_flops = e_unique * 3 * 2 * (2 * B)
        sfu_ops = e_unique * (1 + 2 * B / 128)
        fp32_ops = e_unique * (k + 6)
        peaks = {}
        ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(ppath):
            peaks = json.load(open(ppath))
        f16_peak = peaks.get("bf16_tflops", 1590.0)
        sfu_peak = 148 * 16 * sm_clock
        frac_tensor = tensor_flops / t_apply / 1e12 / f16_peak
        frac_sfu = sfu_ops / t_apply / sfu_peak
        frac_fp32 = 2.0 * fp32_ops / t_apply / 1e12 / fp32_peak
        line = {
            "metric": METRIC, "value": units / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w.name, "ops": "CG iteration: batch-summed banded product, vector updates and inner products sharded by rows; all-gather of the search direction and of per-row-block partial inner products",
                       "entries_per_matvec": E, "rhs_cols": k, "components": B, "sigma2": w.extra["sigma2"],
                       "l2": "operands (134 MB vectors) exceed L2", "collective": "3 all_gather_into_tensor per iteration (search direction 134 MB, two arrays of partial inner products 1 MB)" if world > 1 else "none"},
            "roofline": {
                "bound": "tensor", "kernel": "matmul_sum_tc_kernel",
                "achieved": tensor_flops / t_apply / 1e12, "peak": f16_peak, "unit": "TFLOP/s", "frac": frac_tensor,
                "traffic": None, "frac_sfu": frac_sfu, "frac_fp32": frac_fp32, "product_ms": apply_ms,
                "peak_source": "MEASURED_PEAKS.json bf16_tflops (burst; kind::f16 MMAs); tensor, SFU and FP32 bounds of this "
                               "kernel lie within 25 % of each other (5.4 / 5.0 / 4.4 ms at config 5 on one GPU); SFU peak = "
                               "148 SMs x 16 ops/clk x SM clock implied by the live FFMA probe.  The metric counts "
                               "component entries (B per unique entry), as the reference would evaluate them",
            },
            "e2e": {"value": units * iters / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": (hy.numel() + hx.numel() + hp.numel()) * 4 // iters,
                    "d2h_bytes_per_step": hsol.numel() * 4 // iters, "solve_ms": e2e_ms, "iterations": iters},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_single_op(args, local: int) -> None:
    """The other benchmark configurations, one op each, on one GPU (inputs resident in HBM, CUDA
    events, L2 flushed between steps).  Workloads:
      rbf_small                  config 1: RBF forward, n = 4096, k = 1 (launch-latency bound)
      locally_periodic_bilinear  config 3: bilinear_derivative, batch 4, n = 262144, k = 32
      rbf_unbanded               config 4: unbanded RBF forward, n = 131072, k = 128 (tensor cores)
      rbf_unbanded_index         config 4: 2^24 random (row, col) gathers
    """
    import ctypes

    import kernel_matmul_b200  # noqa: F401
    from kernel_matmul_b200 import ops, ranges, workloads
    from kernel_matmul_b200._lib import check, lib

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    name = args.workload
    peaks = {}
    ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(ppath):
        peaks = json.load(open(ppath))
    flops = ctypes.c_double()
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def probe():
        check(lib.km_probe_fp32_peak(20000, None, ctypes.byref(flops), stream))

    probe()
    fp32_peak = max(flops.value / (cuda_ms(probe) * 1e-3) for _ in range(3)) / 1e12
    sfu_ops = ctypes.c_double()

    def probe_sfu():
        check(lib.km_probe_sfu_peak(20000, None, ctypes.byref(sfu_ops), stream))

    probe_sfu()
    sfu_peak = max(sfu_ops.value / (cuda_ms(probe_sfu) * 1e-3) for _ in range(3)) / 1e12

    if name == "rbf_small":
        w = workloads.rbf_small()
        x = w.x.to(dev)
        start, end = workloads.band(w, x)
        rhs, params = w.rhs.to(dev), w.params.to(dev)
        E, k, kt = int(ops.count_entries(w.n, w.n, start, end)), 1, "rbf"
        fn = lambda: ops.matmul(kt, x, x, rhs, params, start, end)  # noqa: E731
        model = {"bound": "launch latency", "fp32_instr": fp32_instr_fwd(kt, k), "sfu": GEN_FWD[kt][1]}
        units, kernel = E * k, "matmul_fma_cluster_kernel"
    elif name == "locally_periodic_bilinear":
        w = workloads.locally_periodic_bilinear()
        B = w.params.shape[0]
        x = w.x.to(dev)
        start, end = workloads.band(w, x)
        xb = x.expand(B, -1)
        lhs, rhs, params = w.extra["lhs"].to(dev), w.rhs.to(dev), w.params.to(dev)
        kt, k = "locally_periodic", w.rhs.shape[-1]
        E = int(ops.count_entries(w.n, w.n, start, end))
        fn = lambda: ops.bilinear_derivative(kt, xb, xb, lhs, rhs, params, start, end)  # noqa: E731
        # tensor-core gradient (k <= 32): threads only evaluate the factors of d kappa / d p
        model = {"bound": "fp32", "fp32_instr": TC_BWD[kt][0], "sfu": TC_BWD[kt][1]}
        units, kernel = E * k, "grad_tc_kernel"
    elif name == "rbf_unbanded":
        w = workloads.rbf_unbanded(lookups=16)
        x = w.x.to(dev)
        start, end = ranges.make_ranges(None, x)
        rhs, params = w.rhs.to(dev), w.params.to(dev)
        kt, k, E = "rbf", w.rhs.shape[-1], w.n * w.n
        fn = lambda: ops.matmul(kt, x, x, rhs, params, start, end)  # noqa: E731
        # three fp16 MMAs (hi*lo, lo*hi, hi*hi) per product
        model = {"bound": "tensor", "tensor_flops": 3 * 2.0 * E * k, "fp32_instr": TC_FWD[kt][0], "sfu": TC_FWD[kt][1]}
        units, kernel = E * k, "matmul_tc_kernel"
    elif name == "rbf_unbanded_index":
        w = workloads.rbf_unbanded()
        x = w.x.to(dev)
        start, end = ranges.make_ranges(None, x)
        params = w.params.to(dev)
        row, col = w.extra["row"].to(dev), w.extra["col"].to(dev)
        L = row.numel()
        fn = lambda: ops.index("rbf", x, x, params, start, end, (), row, col)  # noqa: E731
        model = {"bound": "hbm", "bytes": 12 * L}
        units, kernel, E, k, kt = L, "index_kernel", L, 1, "rbf"
    else:
        raise SystemExit(f"unknown workload {name}")

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        fn()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    ms = []
    for _ in range(args.steps):
        flush.fill_(1)
        device_delay()
        ms.append(cuda_ms(fn))
    clocks = sampler.stop()
    t = statistics.mean(ms) * 1e-3
    roof = {"bound": model["bound"], "kernel": kernel, "traffic": None}
    if model["bound"] == "tensor":
        # peak: the measured dense bf16 rate (kind::f16 MMAs run at the same rate)
        f16_peak = peaks.get("bf16_tflops", 1590.0)
        roof.update(achieved=model["tensor_flops"] / t / 1e12, peak=f16_peak, unit="TFLOP/s",
                    peak_source="MEASURED_PEAKS.json bf16_tflops (burst); achieved counts the 3 fp16 MMAs per product",
                    frac_sfu=E * model["sfu"] / t / 1e12 / sfu_peak)
    elif model["bound"] == "hbm":
        roof.update(achieved=model["bytes"] / t / 1e9, peak=peaks.get("hbm_gbs", 6650.0), unit="GB/s",
                    peak_source="MEASURED_PEAKS.json hbm_gbs; algorithmic bytes = row + col + out per lookup")
    elif model["bound"] == "sfu":
        roof.update(achieved=E * model["sfu"] / t / 1e12, peak=sfu_peak, unit="Tops/s (special-function operations)",
                    peak_source="live SFU probe (km_probe_sfu_peak); the coefficients run as tcgen05.mma",
                    frac_fp32=2.0 * E * model["fp32_instr"] / t / 1e12 / fp32_peak)
    else:
        roof.update(achieved=2.0 * E * model["fp32_instr"] / t / 1e12, peak=fp32_peak, unit="TFLOP/s",
                    peak_source="live FFMA probe", frac_sfu=E * model["sfu"] / t / 1e12 / sfu_peak)
    roof["frac"] = roof["achieved"] / roof["peak"]
    print(json.dumps({
        "metric": METRIC if name != "rbf_unbanded_index" else "gathered_kernel_entries_per_s",
        "value": units / t, "unit": UNIT if name != "rbf_unbanded_index" else "entries/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name if name != "rbf_unbanded_index" else w.name + "_index", "entries": E, "rhs_cols": k,
                   "l2": "flushed between steps (256 MB write)"},
        "roofline": roof, "gpu_launches": args.steps, "clocks": clocks,
    }), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="spectral_mixture")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--path", default="auto", choices=["auto", "fma", "tc"],
                    help="default workload: kernels of the ops (auto: what the ops choose; fma: FMA-pipe kernels; "
                         "tc: tensor-core kernels)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        if args.workload != "spectral_mixture" and args.workload != "spectral_mixture_small":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "CPU leg implemented for the default workload only"}))
            return
        run_reference(args, rank, world)
    elif args.workload.startswith("cg_sum"):
        run_cg(args, rank, world, local)
    elif args.workload in ("rbf_small", "locally_periodic_bilinear", "rbf_unbanded", "rbf_unbanded_index"):
        if rank == 0:
            run_single_op(args, local)
    else:
        run_ours(args, rank, world, local)


if __name__ == "__main__":
    main()
