"""Benchmark of the kernel-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--exchange auto|halo|allgather] [--path auto|fma|tc] [--no-cpu] [--no-secondary]

Default workload (every N): the conjugate-gradient solve ``(K + sigma^2 I) V = Y`` with K the sum
of 64 spectral components that share inputs, band and lengthscale (n = 2^22 sorted U[0, 20000],
l = 1.5, f ~ U[0, 1] with f_0 = 0, cutoff 6, sigma^2 = 0.01, Y 2^22 x 8; seeded synthetic inputs,
``kernel_matmul_b200/workloads.py``).  One step is one CG iteration: the banded product
``sum_b K_b p`` (all 64 components inside one kernel), the inner products and the vector updates.
With N > 1 (torchrun) the rows are sharded over the ranks -- total work is fixed, ``scaling`` is
"strong" -- and an iteration contains two NCCL all-gathers (``--exchange halo``, the default
for a banded operator: the neighbours' halo rows of q and the partial inner products;
``--exchange allgather``: all of q, 134 MB).  The metric is kernel entries x rhs columns per
second: a matvec visits E component entries, a step processes ``E * k`` units.

Printed keys (one JSON line, rank 0):
  value      whole-job units/s with operands resident in HBM: the sum of the CUDA-event times of
             K iterations (L2 flushed between them), max over ranks;
  e2e        the same metric for whole solves (``iterations`` steps) through
             ``kernel_matmul_b200.host.cg_solve_from_host`` with HOST (pinned) buffers: every rank
             copies x, params and its rows of Y to the device, builds the band, iterates, and copies
             its rows of the solution back;
  roofline   the dominant kernel (``matmul_sum_ph_kernel``: the batch sum with the operator's phase
             vectors written once per solve by a pre-pass; ``KM_SUM_PHASES=0`` selects
             ``matmul_sum_tc_kernel``, which evaluates them in every product) against the measured dense bf16 rate
             (its three fp16 MMAs per 16 phase values are what bounds it), its time taken with CUDA
             events around the product inside the timed iterations;
  cpu_baseline  the dense PyTorch formulation (materialise every K_b, mask by ranges, matmul, sum)
             in fp32 on all host cores, on a seeded sample of row blocks of the same product,
             extrapolated linearly in entries;
  secondary  (N = 1) the other benchmark configurations, each timed the same way: forward +
             ``matmul_bwd`` of the 16-component spectral mixture with their roofline fractions,
             the locally periodic ``bilinear_derivative``, the unbanded k = 128 product, the 2^24
             gathers, the small RBF product; and the reference's own CUDA kernels (best of its
             autotune candidates, compiled unmodified) on the same GPU where they can run.

``--impl reference`` times only the CPU dense formulation of the chosen workload (the reference
has no CPU kernel of its own for this path; the dense formulation is what its tests define as
the expected result).  Under torchrun rank 0 alone runs it.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "kernel_entries_x_rhs_cols_per_s"
UNIT = "entry-cols/s"
DEFAULT_WORKLOAD = "cg_sum"
ALIGN_ITERATIONS = 2  # untimed CG iterations between the barrier and the timed ones (see run_cg)

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


_T0 = time.perf_counter()
TRACE = bool(os.environ.get("KM_BENCH_TRACE"))


def trace(msg: str) -> None:
    """Progress lines on stderr (``--trace`` or KM_BENCH_TRACE=1): where a slow run spends its time."""
    if TRACE:
        print(f"[bench {time.perf_counter() - _T0:7.2f} s] {msg}", file=sys.stderr, flush=True)


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def load_workloads():
    """The workload generators, loaded by path: they need PyTorch only, and the reference arm must
    not import the package (which maps the product's library)."""
    spec = importlib.util.spec_from_file_location("km_b200_workloads", os.path.join(ROOT, "kernel_matmul_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return json.load(open(path)) if os.path.exists(path) else {}


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


def cuda_ms(fn) -> float:
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


def live_peaks(dev) -> tuple[float, float]:
    """(FP32 FFMA TFLOP/s, SFU Tops/s) measured with the library's calibration kernels."""
    import ctypes

    from kernel_matmul_b200._lib import check, lib

    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    flops, sfu_ops = ctypes.c_double(), ctypes.c_double()

    def probe():
        check(lib.km_probe_fp32_peak(20000, None, ctypes.byref(flops), stream))

    def probe_sfu():
        check(lib.km_probe_sfu_peak(20000, None, ctypes.byref(sfu_ops), stream))

    probe()
    fp32_peak = max(flops.value / (cuda_ms(probe) * 1e-3) for _ in range(3)) / 1e12
    probe_sfu()
    sfu_peak = max(sfu_ops.value / (cuda_ms(probe_sfu) * 1e-3) for _ in range(3)) / 1e12
    return fp32_peak, sfu_peak


def dram_traffic(workload: str, kernel: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch, copied by hand from the ncu captures
    summarised under profiles/ into profiles/dram_traffic.json."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    return json.load(open(path)).get(workload, {}).get(kernel)


# ----------------------------------------------------------------------------------- workloads


def make_workload(W, name: str):
    if name == "cg_sum":
        return W.cg_sum_kernel()
    if name == "cg_sum_small":
        return W.cg_sum_kernel(n=1 << 17, components=8, span=625.0)
    if name == "spectral_mixture":
        return W.spectral_mixture()
    if name == "spectral_mixture_small":
        return W.spectral_mixture(n=8192, components=4, k=16, span=62.5)
    raise SystemExit(f"unknown workload {name}")


def config_of(w, entries: int) -> dict:
    """The ``config`` key: the same in both arms."""
    k = w.rhs.shape[-1]
    B = w.params.shape[0] if w.params.dim() > 1 else 1
    if w.name.startswith("cg_sum"):
        return {"workload": w.name, "ops": "CG iteration: batch-summed banded product + inner products + vector updates",
                "n": w.n, "components": B, "rhs_cols": k, "entries_per_matvec": entries, "units_per_step": float(entries) * k,
                "sigma2": w.extra["sigma2"], "iterations_per_solve": int(w.extra["iterations"])}
    return {"workload": w.name, "ops": "matmul fwd + matmul_bwd", "n": w.n, "components": B, "rhs_cols": k,
            "entries_per_pass": entries, "units_per_step": 2.0 * entries * k}


# -------------------------------------------------------------------------------- CPU baselines


def cpu_dense_sample_mixture(w, seconds: float = 12.0, max_seconds: float = 30.0) -> dict:
    """Dense formulation (oracle/dense_reference.py) in fp32 on all host cores: forward slab
    product + autograd gradient for row-block slabs of the spectral-mixture workload, drawn
    round-robin over the components, until ``seconds`` of work are done.  Returns units/s."""
    from oracle import dense_reference as D
    from oracle import oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, n, k, B = w.x, w.n, w.rhs.shape[-1], w.params.shape[0]
    R = -(-n // 128)
    bands = [O.make_ranges(c, x) for c in w.cutoffs]
    units = entries = slabs = 0
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
        "value": units / el, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"{slabs} slabs of {group} row blocks ({entries} entries, fwd + autograd bwd, fp32) in {el:.1f} s",
        "seconds": el,
    }


def cpu_dense_sample_cg(w, seconds: float = 12.0, min_blocks: int = 64, max_seconds: float = 40.0) -> dict:
    """Dense formulation of the CG workload's product in fp32 on all host cores: for a seeded random
    sample of row blocks, every component's K_b is materialised over the block's band, masked and
    multiplied with the right-hand side, and the results are added (what the reference's
    SumKernel operator does, kernel_matmul/gpytorch/sum.py:16-24).  At least ``min_blocks`` row blocks
    and ``seconds`` of work; the rate is per entry, so it extrapolates linearly to the full product
    (7.4e11 entries would take most of an hour).  The vector updates of the iteration (~1 % of the
    product's memory traffic) are not part of the sample."""
    from oracle import dense_reference as D
    from oracle import oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, n, k, B = w.x, w.n, w.rhs.shape[-1], w.params.shape[0]
    R = -(-n // 128)
    start, end = O.make_ranges(w.cutoffs[0], x)
    g = torch.Generator().manual_seed(0)
    order = torch.randperm(R, generator=g).tolist()
    entries = blocks = 0
    t0 = time.perf_counter()
    with torch.no_grad():
        for r in order:
            c0, c1 = int(start[r]), min(int(end[r]), n)
            rows = slice(r * 128, min((r + 1) * 128, n))
            acc = torch.zeros(rows.stop - rows.start, k)
            xr, xc, rhs = x[rows], x[c0:c1], w.rhs[c0:c1]
            for b in range(B):
                acc += D.kernel_matrix(w.kernel_type, xr, xc, w.params[b]) @ rhs
            entries += B * (rows.stop - rows.start) * (c1 - c0)
            blocks += 1
            el = time.perf_counter() - t0
            if (blocks >= min_blocks and el >= seconds) or el >= max_seconds:
                break
    el = time.perf_counter() - t0
    return {
        "value": entries * k / el, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"{blocks} random row blocks x {B} components ({entries} entries, fp32 dense product per component, "
                  f"summed) in {el:.1f} s; extrapolated linearly in entries",
        "seconds": el,
    }


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    W = load_workloads()
    from oracle import oracle as O

    w = make_workload(W, args.workload)
    cg = w.name.startswith("cg_sum")
    sample = cpu_dense_sample_cg if cg else cpu_dense_sample_mixture
    entries = sum(O.count_entries(w.n, w.n, *O.make_ranges(c, w.x)) for c in w.cutoffs)
    if cg:
        entries *= w.params.shape[0]
    per_step = max(2.0, min(10.0, 60.0 / max(1, args.steps + args.warmup)))
    extra = {"min_blocks": 4} if cg else {}
    for _ in range(args.warmup):
        sample(w, seconds=per_step / 4, max_seconds=per_step, **extra)
    vals, secs, base = [], [], None
    extra = {"min_blocks": 8} if cg else {}
    for _ in range(args.steps):
        base = sample(w, seconds=per_step, max_seconds=3 * per_step, **extra)
        vals.append(base["value"])
        secs.append(base["seconds"])
    value = statistics.mean(vals)
    base["value"] = value
    base["sample"] = f"per step: {base['sample']}; {args.steps} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(secs),
        "higher_is_better": True, "scaling": "strong" if cg else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_of(w, entries),
        "what": "dense PyTorch formulation on host cores, bounded sample per step",
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------- the reference's CUDA kernels, same GPU


def reference_cuda_timing(kind: str, kernel_type: str, k: int, call_args: tuple, reps: int = 3) -> dict | None:
    """Times the reference's own CUDA kernels (compiled unmodified into oracle/_ref by
    oracle/build_ref.py) on the same inputs: every autotune candidate that was built for this op,
    kernel type and width (kernel_matmul/configurations.py:94-118), the fastest one reported.
    The reference launches on the legacy default stream, so each call is timed between device
    synchronisations.  None when no module was built.  Every module is compiled for ONE leading
    batch dim (KM_BATCH_DIM = 1): the arguments must have exactly one."""
    import glob

    base = os.path.join(ROOT, "oracle", "_ref")
    stem = f"km_ref_matmul_{kernel_type}_k{k}" if kind == "matmul" else f"km_ref_{kind}_{kernel_type}"
    best, tried, errors = None, 0, []
    if call_args[0].dim() != 2:
        return {"error": "reference modules take exactly one leading batch dim"}
    for d in sorted(glob.glob(os.path.join(base, stem + "*"))):
        name = os.path.basename(d)
        if name != stem and not name.startswith(stem + "_"):
            continue  # e.g. ..._k1 must not pick up ..._k16
        so = os.path.join(d, name + ".so")
        if not os.path.exists(so):
            continue
        try:
            spec = importlib.util.spec_from_file_location(name, so)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.call(*call_args)
            torch.cuda.synchronize()
            ts = []
            for _ in range(reps):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                mod.call(*call_args)
                torch.cuda.synchronize()
                ts.append(1e3 * (time.perf_counter() - t0))
            tried += 1
            trace(f"reference module {name}: {min(ts):.3f} ms")
            if best is None or min(ts) < best[0]:
                best = (min(ts), name)
        except Exception as exc:  # noqa: BLE001 - informational only
            errors.append(f"{name}: {str(exc)[:120]}")
    if best is None:
        return {"error": "; ".join(errors)[:400]} if errors else None
    return {"ms": best[0], "module": best[1], "candidates_timed": tried}


# ------------------------------------------------------------------------ spectral mixture (config 2)


def measure_mixture(w, dev, steps: int, path: str, fp32_peak: float, sfu_peak: float, with_e2e: bool, with_ref: bool) -> dict:
    """Forward product + matmul_bwd of the spectral mixture: resident inputs, CUDA events, L2 flushed
    between steps.  Returns times, roofline fractions per kernel and (optionally) the end-to-end
    figure from host buffers and the reference's CUDA kernels on the same GPU."""
    from kernel_matmul_b200 import host, ops, workloads

    kt = w.kernel_type
    n, k, B = w.n, w.rhs.shape[-1], w.params.shape[0]
    x = w.x.to(dev)
    xb = x.expand(B, -1)
    rhs = w.rhs.to(dev).expand(B, -1, -1)
    params = w.params.to(dev)
    og = w.extra["out_grad"].to(dev)
    start, end = workloads.band(w, x)
    E = int(ops.count_entries(n, n, start, end))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for _ in range(3):
        out_w = ops.matmul(kt, xb, xb, rhs, params, start, end, path=path)
        g_w = ops.matmul_bwd(kt, xb, xb, rhs, params, start, end, og, path=path)
    ops.check(dev)
    tc_fwd, tc_bwd = ops.used_tensor_cores(out_w), ops.used_tensor_cores(g_w)
    fwd_ms, bwd_ms, step_ms = [], [], []
    for _ in range(steps):
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
    ops.check(dev)
    fwd, bwd = statistics.mean(fwd_ms), statistics.mean(bwd_ms)
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
    for kname, kd in kernels.items():
        kd["achieved_tflops"] = 2.0 * E * kd["fp32_instr_per_entry"] / (kd["ms"] * 1e-3) / 1e12
        kd["frac_fp32"] = kd["achieved_tflops"] / fp32_peak
        kd["achieved_sfu_tops"] = E * kd["sfu_per_entry"] / (kd["ms"] * 1e-3) / 1e12
        kd["frac_sfu"] = kd["achieved_sfu_tops"] / sfu_peak
        kd["traffic"] = dram_traffic("spectral_mixture", kname) if w.n == 65536 else None
    ms_per_step = statistics.mean(step_ms)
    res = {
        "config": config_of(w, E), "path": path, "ms_per_step": ms_per_step, "value": 2.0 * E * k / (ms_per_step * 1e-3),
        "unit": UNIT, "steps": steps, "l2": "flushed between steps (256 MB write)", "kernels": kernels,
        "fp32_peak_tflops": fp32_peak, "sfu_peak_tops": sfu_peak,
        "bound": "fp32 (FFMA issue rate measured live; the contraction runs on the tensor cores at a few % of their peak, "
                 "what bounds the kernels is generating the kernel entries)",
        "gpu_launches_per_step": (3 if tc_fwd else 1) + (3 if tc_bwd else 2),
    }
    if with_e2e:
        hx, hrhs = w.x.pin_memory(), w.rhs.contiguous().pin_memory()
        hp, hog = w.params.contiguous().pin_memory(), w.extra["out_grad"].contiguous().pin_memory()
        hout, hgrad = torch.empty(B, n, k).pin_memory(), torch.empty(B, w.params.shape[-1]).pin_memory()
        streams = host.HostStreams(dev)

        def e2e_step():
            host.matmul_and_grad_from_host(kt, hx, hrhs, hp, hog, lambda dx: workloads.band(w, dx), hout, hgrad, streams, path=path)

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        e2e_ms = []
        for _ in range(steps):
            flush.fill_(1)
            e2e_ms.append(cuda_ms(e2e_step))
        res["e2e"] = {"value": 2.0 * E * k / (statistics.mean(e2e_ms) * 1e-3), "unit": UNIT,
                      "h2d_bytes_per_step": sum(t.numel() * 4 for t in (hx, hrhs, hp, hog)),
                      "d2h_bytes_per_step": sum(t.numel() * 4 for t in (hout, hgrad)), "ms_per_step": statistics.mean(e2e_ms)}
    if with_ref:
        ref_f = reference_cuda_timing("matmul", kt, k, (xb, xb, rhs, params, start, end))
        ref_b = reference_cuda_timing("matmul_bwd", kt, k, (xb, xb, rhs, params, start, end, og))
        if ref_f or ref_b:
            res["reference_cuda_kernels_same_gpu"] = {"matmul": ref_f, "matmul_bwd": ref_b}
    return res


# ------------------------------------------------------------------------------ single ops (configs 1, 3, 4)


def measure_single_op(name: str, dev, steps: int, fp32_peak: float, sfu_peak: float, with_ref: bool = True) -> dict:
    """The other benchmark configurations, one op each, on one GPU (inputs resident in HBM, CUDA
    events, L2 flushed between steps).  Workloads:
      rbf_small                  RBF forward, n = 4096, k = 1 (launch-latency bound)
      locally_periodic_bilinear  bilinear_derivative, batch 4, n = 262144, k = 32
      rbf_unbanded               unbanded RBF forward, n = 131072, k = 128 (tensor cores)
      rbf_unbanded_index         2^24 random (row, col) gathers
    """
    from kernel_matmul_b200 import ops, ranges, workloads

    peaks = measured_peaks()
    ref = None
    if name == "rbf_small":
        w = workloads.rbf_small()
        x = w.x.to(dev)
        start, end = workloads.band(w, x)
        rhs, params = w.rhs.to(dev), w.params.to(dev)
        E, k, kt = int(ops.count_entries(w.n, w.n, start, end)), 1, "rbf"
        fn = lambda: ops.matmul(kt, x, x, rhs, params, start, end)  # noqa: E731
        model = {"bound": "launch latency", "fp32_instr": fp32_instr_fwd(kt, k), "sfu": GEN_FWD[kt][1]}
        units, kernel = E * k, "matmul_fma_cluster_kernel"
        if with_ref:  # (the reference modules are built for one leading batch dim)
            ref = reference_cuda_timing("matmul", kt, k, tuple(t.unsqueeze(0) for t in (x, x, rhs, params, start, end)))
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
        model = {"bound": "fp32", "fp32_instr": TC_BWD[kt][0], "sfu": TC_BWD[kt][1]}
        units, kernel = E * k, "grad_tc_kernel"
        if with_ref:
            ref = reference_cuda_timing("bilinear_derivative", kt, k, (xb, xb, lhs, rhs, params.contiguous(), start, end), reps=1)
    elif name == "rbf_unbanded":
        w = workloads.rbf_unbanded(lookups=16)
        x = w.x.to(dev)
        start, end = ranges.make_ranges(None, x)
        rhs, params = w.rhs.to(dev), w.params.to(dev)
        kt, k, E = "rbf", w.rhs.shape[-1], w.n * w.n
        fn = lambda: ops.matmul(kt, x, x, rhs, params, start, end)  # noqa: E731
        model = {"bound": "tensor", "tensor_flops": 3 * 2.0 * E * k, "fp32_instr": TC_FWD[kt][0], "sfu": TC_FWD[kt][1]}
        units, kernel = E * k, "matmul_tc_kernel"
        if with_ref:
            ref = reference_cuda_timing("matmul", kt, k, tuple(t.unsqueeze(0) for t in (x, x, rhs, params, start, end)), reps=1)
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
    for _ in range(3):
        fn()
    ops.check(dev)
    ms = []
    for _ in range(steps):
        flush.fill_(1)
        device_delay()
        ms.append(cuda_ms(fn))
    ops.check(dev)
    t = statistics.mean(ms) * 1e-3
    roof = {"bound": model["bound"], "kernel": kernel, "traffic": dram_traffic(name, kernel)}
    if model["bound"] == "tensor":
        f16_peak = peaks.get("bf16_tflops", 1590.0)
        roof.update(achieved=model["tensor_flops"] / t / 1e12, peak=f16_peak, unit="TFLOP/s",
                    peak_source="MEASURED_PEAKS.json bf16_tflops (burst); achieved counts the 3 fp16 MMAs per product",
                    frac_sfu=E * model["sfu"] / t / 1e12 / sfu_peak)
    elif model["bound"] == "hbm":
        roof.update(achieved=model["bytes"] / t / 1e9, peak=peaks.get("hbm_gbs", 6650.0), unit="GB/s",
                    peak_source="MEASURED_PEAKS.json hbm_gbs; algorithmic bytes = row + col + out per lookup")
    else:
        roof.update(achieved=2.0 * E * model["fp32_instr"] / t / 1e12, peak=fp32_peak, unit="TFLOP/s",
                    peak_source="live FFMA probe", frac_sfu=E * model["sfu"] / t / 1e12 / sfu_peak)
    roof["frac"] = roof["achieved"] / roof["peak"]
    res = {
        "metric": METRIC if name != "rbf_unbanded_index" else "gathered_kernel_entries_per_s",
        "value": units / t, "unit": UNIT if name != "rbf_unbanded_index" else "entries/s", "steps": steps,
        "ms_per_step": t * 1e3,
        "config": {"workload": w.name if name != "rbf_unbanded_index" else w.name + "_index", "entries": E, "rhs_cols": k,
                   "l2": "flushed between steps (256 MB write)"},
        "roofline": roof,
    }
    if ref is not None:
        res["reference_cuda_kernels_same_gpu"] = ref
    del flush
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------ CG (config 5)


def run_cg(args, rank: int, world: int, local: int) -> None:
    import kernel_matmul_b200  # noqa: F401  (raises if libkm_b200.so is missing: no fallback)
    from kernel_matmul_b200 import host, ops, workloads
    from kernel_matmul_b200.cg import CGSolver, ShardedOperator

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    w = make_workload(workloads, args.workload)
    kt, n, k, B = w.kernel_type, w.n, w.rhs.shape[-1], w.params.shape[0]
    x = w.x.to(dev)
    params = w.params.to(dev)
    y = w.rhs.to(dev)
    start, end = workloads.band(w, x)
    E = int(ops.count_entries(n, n, start, end))  # over all components
    units = float(E) * k
    op = ShardedOperator.from_kernel(kt, x, params, start[0], end[0], w.extra["sigma2"], mode=args.exchange)
    trace(f"operator ready: mode {op.mode}, rows [{op.row0}, {op.row1}), kept current [{op.lo}, {op.hi})")
    fp32_peak, sfu_peak = live_peaks(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    trace("peaks probed")

    # a running solve: the first iterations are warm-up, then K timed iterations
    warm = max(args.warmup, 3)
    solver = CGSolver(op, y, max_iterations=warm + ALIGN_ITERATIONS + args.steps + 16)
    matvec = op.matvec_rows
    product_events = []

    def timed_matvec(v, b, c, out):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        matvec(v, b, c, out)
        e1.record()
        product_events.append((e0, e1))

    for _ in range(warm):
        solver.step()
    solver.check_finite()
    torch.cuda.synchronize()
    trace("warm-up iterations done")
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    op.matvec_rows = timed_matvec
    sampler = ClockSampler(local)
    wall0 = time.perf_counter()
    step_events = []
    # ~2 ms of device-side delay first: the launches of the first iterations are then already queued
    # when their events are reached (the events measure device time; the host's enqueue latency is
    # part of the end-to-end figure).  The ranks leave the barrier a few milliseconds apart, and the
    # rank that is first would count its wait for the last one inside its first all-gather: two
    # more untimed iterations, enqueued back to back with the timed ones, bring the ranks into
    # step on the device before the first event pair.
    device_delay()
    device_delay()
    for _ in range(ALIGN_ITERATIONS):
        flush.fill_(1)
        solver.step()
    for _ in range(args.steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        solver.step()
        e1.record()
        step_events.append((e0, e1))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop()
    trace("timed iterations done")
    op.matvec_rows = matvec
    total_ms = sum(a.elapsed_time(b) for a, b in step_events)
    trace("iteration times (ms): " + " ".join(f"{a.elapsed_time(b):.3f}" for a, b in step_events))
    product_ms = statistics.mean(a.elapsed_time(b) for a, b in product_events) if product_events else 0.0
    # where an iteration's time goes: a few more iterations with an event at every phase boundary
    phases: dict[str, list] = {}
    marks: list = []

    def mark(name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))

    solver.mark = mark
    device_delay()
    for _ in range(5):
        flush.fill_(1)
        solver.step()
    solver.mark = None
    torch.cuda.synchronize()
    for (name, ev), (nxt, ev2) in zip(marks, marks[1:]):
        if name != "end":
            phases.setdefault(name, []).append(ev.elapsed_time(ev2))
    breakdown = {name: statistics.mean(v) for name, v in phases.items()}
    solver.check_finite()
    residual = float(solver.residual_norms()[-1].max())
    del solver

    # end to end: whole solves from host buffers (x, params, this rank's rows of Y in; its rows of V out)
    iters = int(w.extra["iterations"])
    hy, hx, hp = w.rhs.contiguous().pin_memory(), w.x.pin_memory(), w.params.contiguous().pin_memory()
    hsol = torch.empty(n, k).pin_memory()

    def solve_e2e():
        return host.cg_solve_from_host(kt, hx, hp, hy, w.cutoffs[0], w.extra["sigma2"], iters, hsol, dev, mode=args.exchange)

    e2e_ms, e2e_residual = float("nan"), None
    if not args.no_e2e:
        solve_e2e()  # warm-up (allocator, NCCL buffers)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e2e_runs = []
        for _ in range(2):
            box = []
            e2e_runs.append(cuda_ms(lambda: box.append(solve_e2e()[0])))
            # (a solve's buffers -- 4.3 GB of phase images among them -- are released before the next
            # one starts, as a caller's would be: with the previous solver still alive the second
            # solve sometimes spent 100-300 ms in the allocator)
            e2e_solver = box.pop()
            e2e_solver.check_finite()
            e2e_residual = float(e2e_solver.residual_norms()[-1].max())
            del e2e_solver
        trace("end-to-end solves (ms): " + " ".join(f"{v:.1f}" for v in e2e_runs))
        e2e_ms = statistics.mean(e2e_runs)
        del box
    trace("end-to-end solves done")
    h2d = (hx.numel() + hp.numel() + (op.hi - op.lo) * k) * 4
    d2h = op.rows * k * 4

    stats = torch.tensor([total_ms, e2e_ms, product_ms, float(h2d), float(d2h)], device=dev, dtype=torch.float64)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, product_ms = float(mx[0]), float(mx[1]), float(mx[2])
        h2d, d2h = float(sm[3]), float(sm[4])

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = total_ms / args.steps
        # All components share inputs, band and lengthscale, so the batch sum runs on the tensor
        # cores: sum_b s_b cos(w_b tau) = <phi(x_i), psi(x_j)> with 2B-vectors of per-point phases
        # (matmul_sum_ph_kernel copies them from images a pre-pass wrote once per operator;
        # matmul_sum_tc_kernel evaluates psi itself: 2B / 128 more SFU operations per entry).  Per
        # UNIQUE (row, column) entry: three fp16 MMAs of 2B multiply-adds, one envelope exponential
        # and k + ~6 FP32 operations.  Row windows are equal, so a rank's launch does 1 / N of it.
        e_unique = E / B / world
        t_prod = product_ms * 1e-3
        tensor_flops = e_unique * 3 * 2 * (2 * B)
        f16_peak = peaks.get("bf16_tflops", 1590.0)
        phase_ws = getattr(op, "phase_workspace", None)
        kernel_name = "matmul_sum_ph_kernel" if phase_ws is not None else "matmul_sum_tc_kernel"
        traffic = dram_traffic("cg_sum", kernel_name) if args.workload == "cg_sum" else None
        roofline = {
            "bound": "tensor", "kernel": kernel_name, "achieved": tensor_flops / t_prod / 1e12, "peak": f16_peak,
            "unit": "TFLOP/s", "frac": tensor_flops / t_prod / 1e12 / f16_peak,
            "traffic": traffic / world if traffic else None,
            "traffic_source": "profiles/dram_traffic.json: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of "
                              f"the full single-GPU launch (profiles/{kernel_name}_cg_sum.md), copied by hand; divided "
                              "by the number of ranks (traffic grows with the rows of a launch)",
            "product_ms": product_ms, "algorithmic_tensor_flops_per_launch": tensor_flops,
            "frac_of_sustained_bf16": tensor_flops / t_prod / 1e12 / peaks.get("bf16_tflops_sustained", 1400.0),
            # SFU operations per unique entry: the envelope, plus (without precomputed phase vectors) the
            # column's phase vector shared by the 128 rows of the block
            "frac_sfu": e_unique * (1 + (0 if phase_ws is not None else 2 * B / 128)) / t_prod / 1e12 / sfu_peak,
            "frac_fp32": 2.0 * e_unique * (k + 6) / t_prod / 1e12 / fp32_peak,
            "fp32_peak_tflops": fp32_peak, "sfu_peak_tops": sfu_peak,
            "peak_source": ("MEASURED_PEAKS.json bf16_tflops (burst; kind::f16 MMAs run at the bf16 rate)" if peaks else
                            "fallback 1590 TFLOP/s (MEASURED_PEAKS.json absent)") +
                           "; product_ms = mean CUDA-event time around the product inside the timed iterations (it also "
                           "covers the FMA-pipe companion launch whose CTAs leave at once); SFU and FP32 fractions against "
                           "the library's live calibration kernels.  The metric counts component entries (B per unique "
                           "entry), as the reference would evaluate them",
        }
        line = {
            "metric": METRIC, "value": units / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(w, E),
            "exchange": op.mode,
            "phase_vectors": ("written once per operator by a pre-pass (%.2f GB workspace per rank; inside the end-to-end "
                              "figure, outside the timed iterations)" % (phase_ws.numel() / 1e9)) if phase_ws is not None
                             else "evaluated inside every product (KM_SUM_PHASES=0)",
            "collective": {"single": "none (one rank)",
                           "halo": f"2 NCCL all_gather_into_tensor per iteration: [{op.halo_above} + {op.halo_below} halo rows "
                                   f"of q + segment sums of p.q] and [segment sums of r.r]",
                           "allgather": "3 NCCL all_gather_into_tensor per iteration: q (all rows, n x k fp32) and two sets "
                                        "of segment sums"}[op.mode],
            "l2": "flushed between iterations (256 MB write, outside the event pairs)",
            "timed_region": f"barrier + synchronize, {ALIGN_ITERATIONS} untimed iterations that bring the ranks into step on the "
                            f"device, {args.steps} iterations each inside its own CUDA-event pair (their sum, max over ranks), "
                            "synchronize + barrier",
            "roofline": roofline,
            "e2e": None if args.no_e2e else {"value": units * iters / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d / iters,
                    "d2h_bytes_per_step": d2h / iters, "solve_ms": e2e_ms, "iterations": iters,
                    "relative_residual": e2e_residual,
                    "what": "host.cg_solve_from_host: pinned host x, params, Y rows in; band, operator set-up, "
                            f"{iters} iterations; solution rows out"},
            # per iteration: product (tensor-core kernel + FMA-pipe companion), q/dots, 2 x segment sums, 2 x update
            "gpu_launches": 7 * args.steps,
            "iteration_breakdown_ms": breakdown,
            "relative_residual_after_timed_region": residual,
            "clocks": clocks, "wall_s": wall,
        }
    if rank == 0 and not args.no_secondary and world == 1:
        sec = {}
        del flush, y
        torch.cuda.empty_cache()
        # the reference's own product kernel on ONE component of this operator (B = 1 keeps its int32
        # offsets below 2^31; the 64-component call overflows them and is not run): x 64 for the sum
        one = reference_cuda_timing("matmul", kt, k, (x[None], x[None], w.rhs.to(dev)[None], params[1:2], start[:1].contiguous(),
                                                      end[:1].contiguous()), reps=1)
        if one is not None:
            line["reference_cuda_kernels_same_gpu"] = {
                "matmul_one_component": one,
                "note": f"one of {B} components; the reference evaluates the sum as {B} such products plus a reduction",
                "matvec_ms_extrapolated": one["ms"] * B if "ms" in one else None}
        sec["spectral_mixture"] = measure_mixture(workloads.spectral_mixture(), dev, min(args.steps, 10), args.path, fp32_peak,
                                                  sfu_peak, with_e2e=True, with_ref=True)
        trace("secondary: spectral mixture done")
        for name in ("rbf_unbanded", "locally_periodic_bilinear", "rbf_unbanded_index", "rbf_small"):
            sec[name] = measure_single_op(name, dev, min(args.steps, 5), fp32_peak, sfu_peak)
            trace(f"secondary: {name} done")
        line["secondary"] = sec
    if rank == 0:
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_dense_sample_cg(w)
            trace("CPU baseline done")
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_mixture(args, rank: int, world: int, local: int) -> None:
    """``--workload spectral_mixture``: forward + matmul_bwd of 16 spectral components; with N > 1
    every rank runs its own copy (independent work, no collective, weak scaling)."""
    import kernel_matmul_b200  # noqa: F401
    from kernel_matmul_b200 import workloads

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    w = make_workload(workloads, args.workload)
    fp32_peak, sfu_peak = live_peaks(dev)
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    res = measure_mixture(w, dev, args.steps, args.path, fp32_peak, sfu_peak, with_e2e=True, with_ref=(rank == 0))
    clocks = sampler.stop()
    ms, e2e_ms = res["ms_per_step"], res["e2e"]["ms_per_step"]
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        units = res["config"]["units_per_step"] * world
        kernels = res["kernels"]
        dom = max(kernels, key=lambda kn: kernels[kn]["ms"])
        d = kernels[dom]
        line = {
            "metric": METRIC, "value": units / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": res["config"], "path": args.path, "l2": res["l2"],
            "per_rank": "own batch of components (same seeded parameters on every rank), no collective",
            "roofline": {"bound": "fp32", "kernel": dom, "achieved": d["achieved_tflops"], "peak": fp32_peak, "unit": "TFLOP/s",
                         "frac": d["frac_fp32"], "traffic": d["traffic"], "traffic_source": "profiles/dram_traffic.json",
                         "peak_source": "measured live: km_probe_fp32_peak (FFMA issue rate of all SMs)",
                         "fp32_peak_tflops": fp32_peak, "sfu_peak_tops": sfu_peak, "kernels": kernels},
            "e2e": {**res["e2e"], "value": units / (e2e_ms * 1e-3), "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": res["e2e"]["h2d_bytes_per_step"] * world,
                    "d2h_bytes_per_step": res["e2e"]["d2h_bytes_per_step"] * world},
            "gpu_launches": res["gpu_launches_per_step"] * args.steps, "clocks": clocks,
        }
        if "reference_cuda_kernels_same_gpu" in res:
            line["reference_cuda_kernels_same_gpu"] = res["reference_cuda_kernels_same_gpu"]
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_dense_sample_mixture(w)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_single(args, local: int) -> None:
    import kernel_matmul_b200  # noqa: F401

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    fp32_peak, sfu_peak = live_peaks(dev)
    sampler = ClockSampler(local)
    res = measure_single_op(args.workload, dev, args.steps, fp32_peak, sfu_peak)
    res.update({"n_gpus": 1, "warmup": 3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "gpu_launches": args.steps, "clocks": sampler.stop()})
    print(json.dumps(res), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--exchange", default="auto", choices=["auto", "halo", "allgather"],
                    help="CG workloads: what the ranks exchange per iteration (auto: halo rows for a banded operator)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-secondary", action="store_true", help="skip the other configurations (N = 1)")
    ap.add_argument("--no-e2e", action="store_true",
                    help="CG workloads: skip the end-to-end solves (profiling runs; the e2e key is then not a measurement)")
    ap.add_argument("--path", default="auto", choices=["auto", "fma", "tc"],
                    help="spectral-mixture workload: kernels of the ops (auto: what the ops choose; fma: FMA-pipe "
                         "kernels; tc: tensor-core kernels)")
    ap.add_argument("--trace", action="store_true", help="progress lines on stderr")
    args = ap.parse_args()
    global TRACE
    TRACE = TRACE or args.trace
    rank, world, local = dist_env()
    if args.impl == "reference":
        if not (args.workload.startswith("cg_sum") or args.workload.startswith("spectral_mixture")):
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "CPU leg implemented for the CG and spectral-mixture workloads"}))
            return
        run_reference(args, rank, world)
    elif args.workload.startswith("cg_sum"):
        run_cg(args, rank, world, local)
    elif args.workload in ("rbf_small", "locally_periodic_bilinear", "rbf_unbanded", "rbf_unbanded_index"):
        if rank == 0:
            run_single(args, local)
    else:
        run_mixture(args, rank, world, local)


if __name__ == "__main__":
    main()
