#!/usr/bin/env python
"""Benchmark of the matmul+ReLU / FMHA kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --case <name> [--iters I]        # one small case, for profiler captures

One JSON line on stdout (rank 0).  The workload of `value` is the same at every N so that the
per-N values form a strong-scaling curve: the large bf16 matmul+ReLU (M=N=K=32768, inputs
N(0, 0.02) in bf16, fp32 accumulate, bf16 output), A and C sharded by row blocks over the ranks,
every finished C tile delivered to all ranks' copies of C by the GEMM epilogue itself (fused
all-gather: one multicast store through the NVSwitch, or unicast peer stores), completion by
per-rank flags and a bounded device-side wait; one step = one full C on every rank.
The configuration the metric string leads with, the fp32-contract 4096x1024x2048 matmul+ReLU,
has its own first-class block `c1` at N=1 (device-timed, end to end from host buffers, CPU
baseline on the full nest, parity against the CPU nest); the remaining configurations ride in
`others` (N=1: the fp32 square sweep, both FMHA configs, the un-fused attention graph, Softmax,
Transpose; N>1: the bf16 causal FMHA sharded by batch*head).

`--impl reference` times the CPU restatement of the reference's loop nest (the reference has
no executable CPU or GPU path of its own in this environment) on all host threads.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture each) of ONE launch of
# the dominant kernel on a case small enough to capture; scaled to the bench's launch by the tiles
# (x k-blocks) processed.  None = not captured.
DRAM_BYTES_GEMM_BF16 = {"shape": (16384, 16384, 16384), "bytes": 8.8297e9 + 0.5368e9}   # read + written
DRAM_BYTES_GEMM_BF16_8192 = {"shape": (8192, 8192, 8192), "bytes": 1.141e9}
DRAM_BYTES_C1 = 60.6e6          # 3xTF32 GEMM 4096x2048x1024 incl. the residual arrays it reads

METRIC = "TFLOP/s & % tensor roofline: matmul+ReLU 4096x1024x2048, FMHA; 1/2/4/8 GPU"
LARGE = 32768


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained")}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def host_threads() -> int:
    """Host threads this process may use.  (Launchers such as torch.distributed.run export
    OMP_NUM_THREADS=1 to their children; the CPU legs therefore pass an explicit count.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 50):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.proc = None
        self.path = f"/tmp/kcg_clocks_{os.getpid()}_{time.monotonic_ns()}.csv"

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.gpu_index)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def stop(self):
        empty = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return empty
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, power, reasons = [], [], [], set()
        for line in Path(self.path).read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clk, clk_max, pw = float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            sm.append(clk)
            mx.append(clk_max)
            power.append(pw)
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if not sm:
            return empty
        # "under load": samples whose power is above half of the highest seen
        hi = max(power)
        loaded = [c for c, p in zip(sm, power) if p >= 0.5 * hi] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": hi}


def with_clocks(entry: dict, clocks: dict) -> dict:
    """Attach a clock sample to a result; `ms_x_mhz` (time x median SM MHz under load) compares
    runs taken at different clocks."""
    entry["clocks"] = clocks
    if clocks.get("sm_mhz") and entry.get("ms") is not None:
        entry["ms_x_mhz"] = entry["ms"] * clocks["sm_mhz"]
    return entry


# ------------------------------------------------------------------------------------------------
# CPU legs: the restatement of the reference's nest on the host cores
# ------------------------------------------------------------------------------------------------
def _bf16_round(x):
    import numpy as np

    u = x.view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def cpu_sample_inputs(rows: int, cols: int, k: int):
    import numpy as np

    rng = np.random.default_rng(40)
    a = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal((k, cols)) * 0.02).astype(np.float32)
    return _bf16_round(a), _bf16_round(b)      # bf16 values (the workload's input type) held as floats


def cpu_time_sample(rows: int, cols: int, k: int, threads: int) -> float:
    from oracle import oracle

    a, b = cpu_sample_inputs(rows, cols, k)
    t0 = time.perf_counter()
    oracle.matmul_relu(a, b, threads=threads if threads > 1 else 1)
    return time.perf_counter() - t0


def cpu_baseline(target_s: float = 10.0):
    """TFLOP/s of the reference nest on the host cores, on a bounded sample of the large GEMM:
    `rows` rows x 2048 columns of C at the full K = 32768."""
    from oracle import oracle

    oracle.build()
    threads = host_threads()
    cols, k = 2048, LARGE
    rows = max(1, threads // 16)
    t = cpu_time_sample(rows, cols, k, threads)
    if t < target_s / 2:
        rows = max(rows, int(rows * target_s / max(t, 1e-3)))
        rows = min(rows, 4096)
        t = cpu_time_sample(rows, cols, k, threads)
    flops = 2.0 * rows * cols * k
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{rows} rows x {cols} cols of C at K={k} (bf16-rounded inputs, fp32 nest), {t:.1f} s"}


def cpu_baseline_c1(a_np, b_np):
    """The whole 4096x1024x2048 nest + ReLU on all host threads; returns (record, C)."""
    from oracle import oracle

    threads = host_threads()
    t0 = time.perf_counter()
    c = oracle.matmul_relu(a_np, b_np, threads=threads if threads > 1 else 1)
    t = time.perf_counter() - t0
    m, k = a_np.shape
    n = b_np.shape[1]
    return {"value": 2.0 * m * n * k / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"the full {m}x{k}x{n} fp32 nest + ReLU, {t:.1f} s"}, c


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    oracle.build()
    threads = host_threads()
    cols, k = 2048, LARGE
    rows = max(1, threads // 16)
    t = cpu_time_sample(rows, cols, k, threads)  # calibration (also a warm-up of the thread pool)
    per_step_target = 4.0
    rows = max(1, min(4096, int(rows * per_step_target / max(t, 1e-3))))
    for _ in range(args.warmup):
        cpu_time_sample(rows, cols, k, threads)
    times = [cpu_time_sample(rows, cols, k, threads) for _ in range(args.steps)]
    total = sum(times)
    flops = 2.0 * rows * cols * k * args.steps
    value = flops / total / 1e12
    sample = f"each step = {rows} rows x {cols} cols of C at K={k}; fp32 loop nest of src/Frontend/Operators.cc:140-173 + ReLU"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "parity": "partial: the CPU nest is pinned only by this repository's own float64 fixtures (the reference holds no vectors)",
        "note": "the reference has no CPU executor and cannot be built here (needs LLVM/MLIR 15); this is the "
                "C restatement of its loop nest on all host threads",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# timing helpers
# ------------------------------------------------------------------------------------------------
def workload_config(n):
    """The workload, in the same words for both arms (what a run did beyond that goes into `run`)."""
    return {"workload": "large bf16 matmul+ReLU M=N=K=32768 (bf16 in N(0,0.02), fp32 accumulate, bf16 out), "
                        "A/C sharded by row blocks, C all-gathered by the GEMM epilogue's own stores",
            "M": LARGE, "N": LARGE, "K": LARGE, "parallelism": f"row-block x{n}",
            "cache": "inputs (2 GiB per operand) are larger than L2 (126 MB); no flush needed"}


def time_steps(fn, steps, warmup, torch, dist=None, drain=None, preheat_s=0.0):
    """W warm-ups (more, until `preheat_s` seconds have run), then K steps between
    barrier+synchronize, CUDA events on the current stream; `drain` (if any) runs inside the timed
    region after the last step.  Returns max-over-ranks milliseconds for the K steps."""
    t0 = time.perf_counter()
    for _ in range(warmup):
        fn()
    while preheat_s > 0:
        torch.cuda.synchronize()
        more = torch.tensor([1.0 if time.perf_counter() - t0 < preheat_s else 0.0], device="cuda")
        if dist is not None:
            dist.all_reduce(more, op=dist.ReduceOp.MIN)      # all ranks leave the warm-up together
        if more.item() == 0.0:
            break
        for _ in range(4):
            fn()
    if drain is not None:
        drain()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    if drain is not None:
        drain()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def time_flushed(fn, iters, torch, flush_buf):
    """Per-launch time (median) with an L2 flush (a write larger than L2) between timed launches."""
    times = []
    for _ in range(iters):
        flush_buf.zero_()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]   # median: single launches of tens of microseconds see outliers


def measure_tf32_peak(torch, dev):
    """cuBLAS TF32 8192^3, best of 10 (the denominator of the 3xTF32 roofline is this / 3)."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    a = torch.randn((8192, 8192), device=dev)
    b = torch.randn((8192, 8192), device=dev)
    for _ in range(3):
        a @ b
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(10):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        a @ b
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    torch.backends.cuda.matmul.allow_tf32 = old
    return 2.0 * 8192 ** 3 / best / 1e9


def settle(torch, seconds=1.0):
    """Idle pause before a short measurement.  After seconds of power-capped work the SM clocks
    stay low for a while (measured: the 80 us fuse_matmul_relu launch takes 120 us right after a
    4 s GEMM loop and 80 us again after a 1 s pause); the burst peaks these kernels are compared
    with were measured on an idle GPU, so they are timed from the same state."""
    torch.cuda.synchronize()
    time.sleep(seconds)


def uniform(torch, dev, shape, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.rand(shape, generator=g, device=dev) * 2 - 1


# ------------------------------------------------------------------------------------------------
# config 1: fuse_matmul_relu fp32 4096x1024x2048, first class
# ------------------------------------------------------------------------------------------------
def c1_block(torch, dev, ops, x3_peak, tf32_peak, flush_buf, gpu_index, with_cpu=True):
    import numpy as np

    M, K, N = 4096, 1024, 2048
    a, b = uniform(torch, dev, (M, K), 0), uniform(torch, dev, (K, N), 1)
    c = torch.empty((M, N), device=dev)
    fn = lambda: ops.matmul_relu(a, b, out=c)
    for _ in range(3):
        fn()
    settle(torch)
    smp = ClockSampler(gpu_index).start()
    ms_cold = time_flushed(fn, 20, torch, flush_buf)
    ms_warm = time_steps(fn, 20, 3, torch) / 20
    clocks = smp.stop()
    fl = 2.0 * M * N * K
    algo_bytes = 4.0 * (M * K + K * N + M * N)
    blk = {"workload": "fuse_matmul_relu fp32 4096x1024x2048: C = ReLU(A.B), uniform[-1,1], 3xTF32 on tcgen05 "
                       "(the residual pass is inside the timed region)",
           "value": fl / ms_cold / 1e9, "unit": "TFLOP/s", "ms": ms_cold, "dtype": "f32 (3xTF32 split, fp32 accumulate)",
           "value_warm_l2": fl / ms_warm / 1e9, "ms_warm_l2": ms_warm,
           "timing": "CUDA events; L2 flushed (256 MiB write) between launches, median of 20; warm = 20 back to back; 1 s idle before",
           "roofline": {"bound": "tensor", "achieved": fl / ms_cold / 1e9, "peak": x3_peak, "unit": "TFLOP/s",
                        "frac": fl / ms_cold / 1e9 / x3_peak, "traffic": DRAM_BYTES_C1, "algorithmic_bytes": algo_bytes,
                        "peak_def": f"cuBLAS TF32 8192^3 measured live ({tf32_peak:.0f}) / 3"}}
    with_clocks(blk, clocks)
    # end to end from host buffers: pinned A, B in, C out, every step, through kcg_gemm_host_staged
    a_h, b_h = a.cpu().pin_memory(), b.cpu().pin_memory()
    c_h = torch.empty((M, N), dtype=torch.float32).pin_memory()
    a_d, b_d, c_d = torch.empty_like(a), torch.empty_like(b), torch.empty_like(c)
    e2e_fn = lambda: ops.matmul_host(a_h, b_h, c_h, a_d, b_d, c_d, relu=True)
    e2e_ms = time_steps(e2e_fn, 10, 3, torch) / 10
    blk["e2e"] = {"value": fl / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                  "h2d_bytes_per_step": 4 * (M * K + K * N), "d2h_bytes_per_step": 4 * M * N,
                  "note": "pinned host A, B -> device, GEMM, C -> host, every step (kcg_gemm_host_staged); PCIe-bound: "
                          "56 MiB per step against 80 us of math"}
    # parity against the CPU nest (the checker), and the CPU baseline on the whole nest
    a_np, b_np = a_h.numpy(), b_h.numpy()
    got = c_h.numpy()
    if with_cpu:
        try:
            rec, want = cpu_baseline_c1(a_np, b_np)
            blk["cpu_baseline"] = rec
            blk["parity"] = {"max_rel_err": float(np.abs(got - want).max() / np.abs(want).max()), "bar": 1e-4,
                             "against": "the full fp32 nest + ReLU on the CPU, same input bits", "pinned": False}
        except Exception as ex:
            blk["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}
        # the same nests as the operator API's own Frontend builds them, lowered to scalar LLVM IR and
        # JIT-compiled for the host: "the repo's own affine module lowered to CPU"
        try:
            from oracle import module_jit

            threads = host_threads()
            mod = module_jit.LoweredModule("matmul_relu", (M, N, K))
            t0 = time.perf_counter()
            c_mod = mod.run(a_np, b_np, threads=threads)
            t = time.perf_counter() - t0
            blk["cpu_baseline_module"] = {
                "value": fl / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "module",
                "sample": f"the Frontend's Matmul + Relu module for {M}x{K}x{N}, lowered to LLVM IR, JIT-compiled, rows over host threads, {t:.1f} s",
                "equals_port_bitwise": bool(np.array_equal(c_mod, want)),
                "max_rel_err_of_gpu_result": float(np.abs(got - c_mod).max() / np.abs(c_mod).max())}
        except Exception as ex:
            blk["cpu_baseline_module"] = {"value": None, "kind": "module", "sample": f"unavailable: {ex}"}
    return blk


# ------------------------------------------------------------------------------------------------
# the other configurations (1 GPU)
# ------------------------------------------------------------------------------------------------
def fmha_long(torch, dev, peaks, ops, bh_lo, bh_hi, gpu_index, dist=None, steps=5):
    """bf16 causal B8 H32 S8192 D128, the (batch*head) range [bh_lo, bh_hi) on this rank."""
    n = bh_hi - bh_lo
    g = torch.Generator(device=dev)
    qkv = []
    for seed in (30, 31, 32):
        g.manual_seed(seed * 1000 + bh_lo)
        qkv.append(torch.randn((1, n, 8192, 128), generator=g, device=dev).bfloat16())
    o = torch.empty_like(qkv[0])
    scale = 128 ** -0.5
    fn = lambda: ops.fmha(qkv[0], qkv[1], qkv[2], scale=scale, causal=True, out=o)
    # three batches of `steps` launches, each after a second of idle time (the peak this is
    # compared with is a burst figure); the median batch is reported and all three are listed, so
    # a clock dip on a shared, power-capped box shows as such
    for _ in range(3):
        fn()
    batches = []
    smp = ClockSampler(gpu_index).start() if gpu_index is not None else None
    for _ in range(3):
        settle(torch)
        batches.append(time_steps(fn, steps, 0, torch, dist) / steps)
    clocks = smp.stop() if smp else None
    batches.sort()
    ms = batches[1]
    fl = 2.0 * 256 * 8192 * 8192 * 128  # whole job: causal = half of 4*B*H*S^2*D
    world = dist.get_world_size() if dist is not None else 1
    peak = peaks["bf16_tflops"] * world
    ent = {"workload": f"FMHA bf16 causal B8 H32 S8192 D128, batch*head sharded x{world}, no collective",
           "tflops": fl / ms / 1e9, "ms": ms, "ms_batches": batches,
           "roofline": {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": peak, "unit": "TFLOP/s",
                        "frac": fl / ms / 1e9 / peak, "peak_def": f"bf16 burst x{world}"}}
    if clocks is not None:
        with_clocks(ent, clocks)
    return ent


def others_single_gpu(torch, dev, peaks, ops, tf32_peak, flush_buf, gpu_index):
    """The remaining configurations of the metric, 1 GPU, CUDA-event timed, L2 flushed between
    launches where the working set fits L2; one second of idle time before each (see settle);
    every entry carries its own clock sample."""
    res = []
    x3_peak = tf32_peak / 3.0

    def timed(entry_fn):
        settle(torch)
        smp = ClockSampler(gpu_index).start()
        ent = entry_fn()
        return with_clocks(ent, smp.stop())

    # fp32 square sweep
    for i, n in enumerate((1024, 2048, 4096, 8192)):
        a, b = uniform(torch, dev, (n, n), 10 + i), uniform(torch, dev, (n, n), 10 + i + 100)
        c = torch.empty((n, n), device=dev)
        fn = lambda: ops.matmul_relu(a, b, out=c)
        for _ in range(3):
            fn()

        def one():
            ms = time_flushed(fn, 10, torch, flush_buf)
            fl = 2.0 * n ** 3
            return {"workload": f"fp32 matmul+ReLU {n}^3 (3xTF32)", "tflops": fl / ms / 1e9, "ms": ms,
                    "roofline": {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": x3_peak, "unit": "TFLOP/s",
                                 "frac": fl / ms / 1e9 / x3_peak}}
        res.append(timed(one))
    del a, b, c
    # FMHA fp32 in/out non-causal B4 H16 S1024 D64
    g = torch.Generator(device=dev)
    qkv = []
    for seed in (20, 21, 22):
        g.manual_seed(seed)
        qkv.append(torch.randn((4, 16, 1024, 64), generator=g, device=dev))
    o = torch.empty_like(qkv[0])
    fn = lambda: ops.fmha(qkv[0], qkv[1], qkv[2], scale=0.125, out=o)
    for _ in range(3):
        fn()
    fl3 = 4.0 * 4 * 16 * 1024 * 1024 * 64

    def fused():
        ms = time_flushed(fn, 20, torch, flush_buf)
        return {"workload": "FMHA fp32-in/out non-causal B4 H16 S1024 D64 (both contractions TF32 on the fp32 tiles, no conversion pass)",
                "tflops": fl3 / ms / 1e9, "ms": ms, "tolerance": "5e-3 (TF32 internals)",
                "roofline": {"bound": "tensor", "achieved": fl3 / ms / 1e9, "peak": tf32_peak, "unit": "TFLOP/s",
                             "frac": fl3 / ms / 1e9 / tf32_peak, "peak_def": "cuBLAS TF32 8192^3 measured live"}}
    res.append(timed(fused))
    # the same attention as the reference's un-fused three-operator graph: BatchedMatmul(Q, K^T) ->
    # Softmax -> BatchedMatmul(P, V) through the standalone kernels (scale folded into Q)
    qs = qkv[0] * 0.125

    def graph():
        s = ops.batched_matmul(qs, qkv[1], b_col_major=True, precision="tf32")
        ops.softmax(s, inplace=True)
        return ops.batched_matmul(s, qkv[2], precision="tf32")
    for _ in range(2):
        graph()

    def unfused():
        ms = time_steps(graph, 5, 3, torch) / 5
        return {"workload": "the same attention un-fused: batched matmul (64 x 1024x1024x64, TF32) -> Softmax -> batched matmul "
                            "(64 x 1024x64x1024), standalone kernels, S materialised (256 MiB)",
                "tflops": fl3 / ms / 1e9, "ms": ms}
    res.append(timed(unfused))
    # standalone Softmax (HBM-bound): 65536 rows x 1024 fp32 in place
    s = torch.randn((65536, 1024), device=dev) * 3
    for _ in range(2):
        ops.softmax(s, inplace=True)

    def soft():
        ms = time_steps(lambda: ops.softmax(s, inplace=True), 10, 3, torch) / 10
        nbytes = 2.0 * s.numel() * 4
        return {"workload": "Softmax 65536 x 1024 fp32 in place (read once, write once)", "gbs": nbytes / ms / 1e6, "ms": ms,
                "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"]}}
    res.append(timed(soft))
    del s, qs
    res.append(fmha_long(torch, dev, peaks, ops, 0, 256, gpu_index))
    del qkv, o
    # Transpose (HBM-bound): 8192 x 8192 fp32, 256 MiB in + 256 MiB out, larger than L2
    x = torch.randn((8192, 8192), device=dev)
    for _ in range(3):
        y = ops.transpose(x)

    def tr():
        ms = time_steps(lambda: ops.transpose(x), 10, 3, torch, None) / 10
        nbytes = 2.0 * x.numel() * 4
        return {"workload": "Transpose 8192x8192 fp32 (read once, write once)", "gbs": nbytes / ms / 1e6, "ms": ms,
                "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"]}}
    res.append(timed(tr))
    del x, y
    return res


# ------------------------------------------------------------------------------------------------
# small cases for profiler captures:  python bench.py --case <name>
# ------------------------------------------------------------------------------------------------
def run_case(args):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    from kernelcodegen_b200 import build, ops

    build.build()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)

    def gemm_bf16(size, copies=0):
        a = (torch.randn((size, size), device=dev) * 0.02).bfloat16()
        b = (torch.randn((size, size), device=dev) * 0.02).bfloat16()
        c = torch.empty((size, size), device=dev, dtype=torch.bfloat16)
        extra = [torch.empty_like(c) for _ in range(copies)]
        return (lambda: ops.matmul_relu(a, b, out=c, peers=[t.data_ptr() for t in extra])), 2.0 * size ** 3, "flop"

    def gemm_f32(m, n, k):
        a, b = uniform(torch, dev, (m, k), 0), uniform(torch, dev, (k, n), 1)
        c = torch.empty((m, n), device=dev)
        return (lambda: ops.matmul_relu(a, b, out=c)), 2.0 * m * n * k, "flop"

    def fmha(bq, h, s, d, causal, dtype):
        q, k, v = (torch.randn((bq, h, s, d), device=dev).to(dtype) for _ in range(3))
        o = torch.empty_like(q)
        fl = (2.0 if causal else 4.0) * bq * h * s * s * d
        return (lambda: ops.fmha(q, k, v, scale=1.0 / math.sqrt(d), causal=causal, out=o)), fl, "flop"

    def transpose():
        x = torch.randn((8192, 8192), device=dev)
        return (lambda: ops.transpose(x)), 2.0 * x.numel() * 4, "byte"

    def softmax():
        x = torch.randn((65536, 1024), device=dev)
        return (lambda: ops.softmax(x, inplace=True)), 2.0 * x.numel() * 4, "byte"

    def batched():
        a, b = torch.randn((64, 1024, 64), device=dev), torch.randn((64, 1024, 64), device=dev)
        return (lambda: ops.batched_matmul(a, b, b_col_major=True, precision="tf32")), 2.0 * 64 * 1024 * 1024 * 64, "flop"

    cases = {
        "gemm_bf16_8192": lambda: gemm_bf16(8192),
        "gemm_bf16_16384": lambda: gemm_bf16(16384),
        "gemm_bf16_8192_7copies": lambda: gemm_bf16(8192, 7),
        "gemm_3xtf32_c1": lambda: gemm_f32(4096, 2048, 1024),
        "gemm_3xtf32_1024": lambda: gemm_f32(1024, 1024, 1024),
        "gemm_3xtf32_8192": lambda: gemm_f32(8192, 8192, 8192),
        "fmha_causal_b2h16": lambda: fmha(2, 16, 8192, 128, True, torch.bfloat16),
        "fmha_causal_b1h32": lambda: fmha(1, 32, 8192, 128, True, torch.bfloat16),
        "fmha_fp32": lambda: fmha(4, 16, 1024, 64, False, torch.float32),
        "transpose_fp32": transpose,
        "softmax_fp32": softmax,
        "batched_qk_tf32": batched,
    }
    if args.case not in cases:
        raise SystemExit(f"unknown case {args.case}; one of {sorted(cases)}")
    fn, work, unit = cases[args.case]()
    ms = time_steps(fn, args.iters, 2, torch) / args.iters
    rate = {"tflops": work / ms / 1e9} if unit == "flop" else {"gbs": work / ms / 1e6}
    print(json.dumps({"case": args.case, "ms": ms, **rate, "iters": args.iters, "device_status": ops.last_device_status()}),
          flush=True)


# ------------------------------------------------------------------------------------------------
# the reference's own sweep:  python bench.py --sweep [--sweep-log FILE]
# ------------------------------------------------------------------------------------------------
def run_sweep(args):
    """The demo shape and the 20 square sizes of the reference's harness (test/test.cc:16, 37), in
    the format of its performance/output.log, with sampled rows of every result held to the CPU
    nest.  One JSON line per size on stdout; the log text goes to --sweep-log."""
    import numpy as np
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    from kernelcodegen_b200 import build, harness, ops
    from oracle import oracle

    build.build()
    dev = torch.device("cuda:0")
    log = open(args.sweep_log, "w") if args.sweep_log else sys.stderr
    shapes = [(4096, 2048, 1024)] + [(s, s, s) for s in harness.SWEEP]
    for m, n, k in shapes:
        rec = harness.run_case(m, n, k, check=False, out=log)
        # parity: the same seeded inputs the harness used, a few rows against the fp32 nest
        g = torch.Generator(device=dev).manual_seed(m * 31 + n * 17 + k)
        a = torch.rand((m, k), generator=g, device=dev) * 2 - 1
        b = torch.rand((k, n), generator=g, device=dev) * 2 - 1
        c = ops.matmul(a, b)
        nrows = 8 if k <= 4096 else 3
        rows = sorted({0, m - 1, *np.random.default_rng(m).integers(0, m, nrows).tolist()})
        want = oracle.matmul_rows(a[rows].cpu().numpy(), b.cpu().numpy(), list(range(len(rows))))
        got = c[rows].cpu().numpy()
        rec["rel_err_vs_cpu_nest"] = float(np.abs(got - want).max() / np.abs(want).max())
        # the same rows accumulated in float64 tell the two apart: how far the fp32 nest itself and the
        # kernel are from the exact product
        exact = oracle.matmul_rows(a[rows].cpu().numpy(), b.cpu().numpy(), list(range(len(rows))), f64=True)
        rec["rel_err_vs_f64"] = float(np.abs(got - exact).max() / np.abs(exact).max())
        rec["cpu_nest_vs_f64"] = float(np.abs(want - exact).max() / np.abs(exact).max())
        rec["rows_checked"] = len(rows)
        rec["tflops"] = 2.0 * m * n * k / rec["mine_ms"] / 1e9
        rec["cublas_sgemm_ratio"] = rec["cublas_nn_ms"] / rec["mine_ms"]
        print(json.dumps(rec), flush=True)
        del a, b, c
    if log is not sys.stderr:
        log.close()


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    # Keep stdout for the one JSON line: anything a library prints to fd 1 (NCCL's version
    # banner, for instance) goes to stderr instead.
    json_fd = os.dup(1)
    os.dup2(2, 1)
    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod

    from kernelcodegen_b200 import build, capi, ops, peer, sharding

    if rank == 0:
        build.build()
    if dist is not None:
        dist.barrier()
    lib = capi.load()
    peaks, peak_src = load_peaks()

    M = N = K = LARGE
    chunk = 2048
    g = torch.Generator(device=dev)
    g.manual_seed(41)
    b = torch.empty((K, N), dtype=torch.bfloat16, device=dev)
    for r0 in range(0, K, chunk):
        b[r0:r0 + chunk] = (torch.randn((chunk, N), generator=g, device=dev) * 0.02).bfloat16()

    def make_a(r_lo, r_hi):
        """Rows [r_lo, r_hi) of A: every aligned 2048-row chunk has its own seed and is generated whole,
        so a rank makes only the chunks its shard touches and the bits do not depend on how the rows
        are dealt out."""
        out = torch.empty((r_hi - r_lo, K), dtype=torch.bfloat16, device=dev)
        for r0 in range(r_lo - r_lo % chunk, r_hi, chunk):
            g.manual_seed(40 * 100003 + r0)
            blk = (torch.randn((chunk, K), generator=g, device=dev) * 0.02).bfloat16()
            s0, s1 = max(r0, r_lo), min(r0 + chunk, r_hi)
            out[s0 - r_lo:s1 - r_lo] = blk[s0 - r0:s1 - r0]
        return out

    # Row blocks: equal by default.  The GPUs of one node run this power-capped GEMM at rates a few
    # per cent apart, and a step ends when the slowest rank ends; with --weighted-rows each rank
    # first times the product on an equal block (no stores to peers), and the rows are then dealt
    # out in proportion to the measured rates, in blocks of 128 rows.
    blocks = [sharding.row_block(M, r, world) for r in range(world)]
    rank_rates = None
    if world > 1 and args.weighted_rows:
        e_lo, e_hi = blocks[rank]
        a_eq = make_a(e_lo, e_hi)
        c_eq = torch.empty((e_hi - e_lo, N), dtype=torch.bfloat16, device=dev)
        cal = lambda: ops.matmul_relu(a_eq, b, out=c_eq)
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < args.preheat_s:     # to the steady power-capped clocks first
            for _ in range(4):
                cal()
            torch.cuda.synchronize()
        cal_ms = time_steps(cal, 6, 1, torch) / 6
        rate = torch.tensor([2.0 * (e_hi - e_lo) * N * K / cal_ms / 1e9], device=dev, dtype=torch.float64)
        rates = [torch.zeros_like(rate) for _ in range(world)]
        dist.all_gather(rates, rate)
        rank_rates = [float(r.item()) for r in rates]
        blocks = sharding.weighted_row_blocks(M, rank_rates)
        del a_eq, c_eq
    lo, hi = blocks[rank]
    rows = hi - lo
    a = make_a(lo, hi)

    # Every rank holds TWO full copies of C (steps alternate between them), so that the flags of
    # step i can be checked while step i+1 already runs (completion "deferred"); "strict" waits for
    # all ranks' flags inside every step.
    completion = args.completion if world > 1 else None
    n_buf = 2 if completion == "deferred" else 1
    cmats = [peer.PeerMatrix(M, N, torch.bfloat16, dev, backend=args.peer_backend) for _ in range(n_buf)] if world > 1 else []
    if world > 1:
        c_fulls = [cm.tensor for cm in cmats]
        multicast = bool(cmats[0].mc_ptr) and not args.no_multicast
        store = ("one multimem.st per 16 bytes through the NVSwitch multicast mapping of C" if multicast
                 else f"unicast peer stores to {world - 1} peers")
    else:
        c_fulls = [torch.empty((M, N), dtype=torch.bfloat16, device=dev)]
        multicast, store = False, None
    counter = {"i": 0}

    def step():
        i = counter["i"]
        counter["i"] = i + 1
        if world == 1:
            ops.matmul_relu(a, b, out=c_fulls[0])
            return
        cm = cmats[i % n_buf]
        ops.matmul_relu(a, b, out=cm.tensor[lo:hi], **cm.store_args(lo, i // n_buf + 1, multicast=multicast))
        if completion == "strict":
            cm.wait(i // n_buf + 1)         # all ranks' row blocks of step i are in this copy
        elif i >= 1:
            prev = cmats[(i - 1) % n_buf]
            prev.wait((i - 1) // n_buf + 1)  # step i-1 is complete everywhere while step i runs

    def drain():
        i = counter["i"]
        if world > 1 and completion == "deferred" and i >= 1:
            cmats[(i - 1) % n_buf].wait((i - 1) // n_buf + 1)

    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    launches0 = lib.kcg_launch_count()
    steps_before = counter["i"]
    ms_total = time_steps(step, args.steps, args.warmup, torch, dist, drain=drain, preheat_s=args.preheat_s)
    clocks = sampler.stop() if sampler else None
    steps_run = counter["i"] - steps_before
    launches = lib.kcg_launch_count() - launches0
    # launches counted over warm-up + timed steps on this rank; keep the timed share
    launches_timed = launches * args.steps // max(1, steps_run)
    if dist is not None:
        t = torch.tensor([launches_timed], device=dev, dtype=torch.int64)
        dist.all_reduce(t)
        launches_timed = int(t.item())
    wait_status = capi.status_str(lib.kcg_peer_wait_status())
    status = 0 if wait_status == "KCG_OK" else wait_status
    ms_step = ms_total / args.steps
    flops = 2.0 * M * N * K
    value = flops / ms_step / 1e9

    # all-gather check (outside the timed region): sampled rows of the NEXT rank's block, as they
    # arrived in THIS rank's copy of C, against the CPU nest in float64 on the same input bits
    # (first 2048 columns), and the whole arrived block against this rank's own recomputation
    allgather_check = None
    if dist is not None:
        from oracle import oracle

        nxt = (rank + 1) % world
        plo, phi = blocks[nxt]
        a_peer = torch.cat([make_a(plo, plo + 256), make_a(phi - 128, phi)])     # first 256 rows and the last 128
        peer_rows = list(range(plo, plo + 256)) + list(range(phi - 128, phi))
        last = cmats[(counter["i"] - 1) % n_buf].tensor
        pick = [0, 1, 127, 128, 255, 256 + 127]                                  # indices into a_peer
        want64 = oracle.matmul_rows(a_peer[pick].float().cpu().numpy(), b[:, :2048].float().cpu().numpy(),
                                    list(range(len(pick))), f64=True)
        want64 = np.maximum(want64, 0.0)
        got = last[[peer_rows[i] for i in pick]][:, :2048].float().cpu().numpy()
        err = float(np.abs(got - want64).max() / np.abs(want64).max())
        mine = ops.matmul_relu(a_peer[:256].contiguous(), b, cta_group=1, tile_n=256)   # same kernel, same order of sums per tile
        same = bool(torch.equal(last[plo:plo + 256], mine))
        t = torch.tensor([err, 0.0 if same else 1.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        allgather_check = {"rows_vs_cpu_nest_f64_per_rank": len(pick), "cols": 2048, "max_rel_err": float(t[0].item()),
                           "bar": 2e-2, "peer_block_equals_local_recomputation_256_rows": bool(t[1].item() == 0.0)}
        del a_peer, mine

    # which kernel the library runs for this rank's block, from its own geometry query
    import ctypes

    gd = capi.GemmDesc()
    gd.M, gd.N, gd.K = rows, N, K
    gd.lda, gd.ldb, gd.ldc = K, N, N
    gd.dtype_in = gd.dtype_out = capi.KCG_BF16
    gd.precision = capi.KCG_PREC_BF16
    geo = (ctypes.c_int32 * 6)()
    lib.kcg_gemm_launch_geometry(ctypes.byref(gd), geo)
    kernel_name = (f"{'gemm_pair_kernel' if geo[2] == 2 else 'gemm_kernel'}<bf16, tile {geo[3]}x{geo[4]}x64> (tcgen05/TMEM), "
                   f"grid {geo[0]} x {geo[1]} threads, {geo[5]} tiles, one launch per step per GPU")
    peak_sust = peaks["bf16_tflops_sustained"]
    per_gpu = value / world
    if DRAM_BYTES_GEMM_BF16["bytes"] is not None:
        src = DRAM_BYTES_GEMM_BF16
    else:
        src = DRAM_BYTES_GEMM_BF16_8192
    sm_, sn_, sk_ = src["shape"]
    traffic = src["bytes"] * (rows / sm_) * (N / sn_) * (K / sk_)
    algo_bytes = 2.0 * (rows * K + K * N + rows * N)
    roofline = {"bound": "tensor", "achieved": per_gpu, "peak": peak_sust, "unit": "TFLOP/s",
                "frac": per_gpu / peak_sust, "traffic": traffic, "algorithmic_bytes": algo_bytes,
                "traffic_def": f"ncu dram bytes of one {sm_}^3 launch x tiles x k-blocks of this launch",
                "kernel": kernel_name,
                "peak_def": f"cuBLAS bf16 sustained, {peak_src} (burst {peaks['bf16_tflops']:.0f}: frac {per_gpu / peaks['bf16_tflops']:.3f})",
                "per_gpu": True, "flop_per_launch": 2.0 * rows * N * K,
                "from": "the timed steps (value / n_gpus)"}
    if clocks and clocks.get("sm_mhz"):
        roofline["ms_x_mhz"] = ms_step * clocks["sm_mhz"]

    extra = {}
    if dist is not None and not args.no_others:
        # for comparison: the launch alone (no completion wait), and the other completion protocol
        def gemm_only():
            cm = cmats[0]
            ops.matmul_relu(a, b, out=cm.tensor[lo:hi], **cm.store_args(lo, 0, multicast=multicast))
        kn = max(3, args.steps // 2)
        extra["kernel_ms_no_wait"] = time_steps(gemm_only, kn, 1, torch, dist) / kn
        # every rank's own time for its block with the stores (no waiting on anybody), rank order
        mine_ms = torch.tensor([time_steps(gemm_only, kn, 1, torch) / kn], device=dev, dtype=torch.float64)
        all_ms = [torch.zeros_like(mine_ms) for _ in range(world)]
        dist.all_gather(all_ms, mine_ms)
        extra["rank_ms_with_stores"] = [float(x.item()) for x in all_ms]
        # the literal alternative: GEMM into the local block, then an NCCL all-gather of the blocks
        blk = torch.empty((rows, N), dtype=torch.bfloat16, device=dev)
        full = cmats[0].tensor

        def nccl_step():
            ops.matmul_relu(a, b, out=blk)
            dist.all_gather_into_tensor(full, blk)
        if len({h - l for l, h in blocks}) == 1:      # the collective wants equal blocks
            extra["ms_per_step_gemm_then_nccl_allgather"] = time_steps(nccl_step, kn, 1, torch, dist) / kn
        del blk
    c_local = c_fulls[0][lo:hi]
    peers = cmats[0].peer_row_ptrs(lo) if cmats else []
    sync_token = torch.zeros(1, device=dev)

    # end to end through the public API with host buffers: H2D of this rank's A block and of B,
    # launch, D2H of this rank's C block, every step.  With several ranks each one copies only its
    # 1/N row block of B over its own PCIe link and the blocks are all-gathered over NVLink.
    a_host = torch.empty((rows, K), dtype=torch.bfloat16).pin_memory()
    a_host.copy_(a)
    share_b = dist is not None and K % world == 0
    klo, khi = sharding.row_block(K, rank, world) if share_b else (0, K)
    b_host = torch.empty((khi - klo, N), dtype=torch.bfloat16).pin_memory()   # this rank's row block of B (all of B at N = 1)
    b_host.copy_(b[klo:khi])
    b_blk = torch.empty((khi - klo, N), dtype=torch.bfloat16, device=dev) if share_b else None
    c_host = torch.empty((rows, N), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        # kcg_gemm_host_staged: chunked H2D, GEMM strips as chunks land, D2H of finished strips of C,
        # on the library's three streams; the current stream continues after the last D2H
        if not share_b:
            ops.matmul_host(a_host, b_host, c_host, a, b, c_local, relu=True, peers=peers, chunks=args.e2e_chunks)
        else:
            b_blk.copy_(b_host, non_blocking=True)
            dist.all_gather_into_tensor(b, b_blk)          # row blocks of B, rank order = row order
            ops.matmul_host(a_host, None, c_host, a, b, c_local, relu=True, peers=peers, chunks=args.e2e_chunks)
        if dist is not None:
            dist.all_reduce(sync_token)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms = time_steps(e2e_step, e2e_steps, 1, torch, dist) / e2e_steps
    e2e = {"value": flops / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
           "h2d_bytes_per_step": (M * K + K * N) * 2, "d2h_bytes_per_step": M * N * 2,
           "bound": "PCIe / host memory: 6.4 GB cross the host links every step, whatever the kernels do",
           "note": ("pinned host A + B -> device, GEMM, C -> host, every step, through kcg_gemm_host_staged (row chunks of A / "
                    "column chunks of B copied alternately, each GEMM strip launched when its operands have landed, finished "
                    "strips of C copied back meanwhile)") if not share_b else
                   ("per rank, every step: pinned host A row block and 1/N of B -> device, B all-gathered over NVLink (NCCL), "
                    "kcg_gemm_host_staged on the resident B (row chunks of A in, GEMM strips, strips of C out)")}
    # the strips that came back are the product the device holds
    e2e["c_host_equals_device"] = bool(torch.equal(c_host[:256], c_local[:256].cpu()) and
                                       torch.equal(c_host[-256:], c_local[-256:].cpu()))

    def e2e_sequential():  # for comparison only: every rank copies all it needs, then launches, then copies back
        a.copy_(a_host, non_blocking=True)
        b.copy_(b_full_host, non_blocking=True)
        ops.matmul_relu(a, b, out=c_local, peers=peers)
        if dist is not None:
            dist.all_reduce(sync_token)
        c_host.copy_(c_local, non_blocking=True)
    b_full_host = b_host if not share_b else torch.empty((K, N), dtype=torch.bfloat16).pin_memory()
    if share_b:
        b_full_host.copy_(b)
    e2e["ms_per_step_sequential"] = time_steps(e2e_sequential, 2, 1, torch, dist) / 2
    del a_host, b_host, b_full_host, b_blk, c_host

    others = []
    c1 = None
    tf32_peak = None
    # free the big operands before the other configs
    del a, b, c_local, c_fulls
    for cm in cmats:
        cm.close()
    cmats = []
    torch.cuda.empty_cache()
    if args.no_others:
        pass
    elif world == 1:
        flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        settle(torch)
        tf32_peak = measure_tf32_peak(torch, dev)
        c1 = c1_block(torch, dev, ops, tf32_peak / 3.0, tf32_peak, flush_buf, local_rank, with_cpu=not args.no_cpu_baseline)
        others = others_single_gpu(torch, dev, peaks, ops, tf32_peak, flush_buf, local_rank)
    else:
        blo, bhi = sharding.bh_shard(256, rank, world)
        others = [fmha_long(torch, dev, peaks, ops, blo, bhi, local_rank if rank == 0 else None, dist)]
    status2 = ops.last_device_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu = cpu_baseline()
        except Exception as ex:  # the oracle is test infrastructure; its absence must not hide the GPU number
            cpu = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "run": {
                "preheat": (f"untimed warm-up steps continue until {args.preheat_s:g} s of work have run, so that the timed steps "
                            "see the steady power-capped clocks at every N"),
                "completion": None if completion is None else (
                    "per-rank flags (st.release.sys by the launch's last CTA) + bounded device-side wait; "
                    + ("checked inside every step" if completion == "strict" else
                       "the flags of step i are checked while step i+1 runs (two copies of C alternate), all outstanding flags "
                       "inside the timed region")),
                "allgather_store": store,
                "row_blocks": None if world == 1 else ("equal" if rank_rates is None else
                                                       "in proportion to each GPU's rate measured on an equal block before the timed steps"),
            },
            "roofline": roofline, "e2e": e2e, "gpu_launches": launches_timed, "clocks": clocks,
            "device_status": [status, status2], "others": others,
            "parity": "partial: the CPU nest the kernels are held to is pinned only by this repository's own float64 fixtures "
                      "(the reference holds no vectors and cannot be built here)",
        }
        line.update(extra)
        if c1 is not None:
            line["c1"] = c1
        if allgather_check is not None:
            line["allgather_check"] = allgather_check
        if world > 1:
            line["row_blocks"] = [list(x) for x in blocks]
            if rank_rates is not None:
                line["rank_rates_tflops_equal_blocks_no_stores"] = rank_rates
        if tf32_peak is not None:
            line["tf32_cublas_tflops_live"] = tf32_peak
        if cpu is not None:
            line["cpu_baseline"] = cpu
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline legs (N=1)")
    ap.add_argument("--no-others", action="store_true", help="only the headline workload (for profiler launch lists)")
    ap.add_argument("--e2e-chunks", type=int, default=0, help="chunks per operand of the host-buffer GEMM (0 = library default)")
    ap.add_argument("--completion", choices=("deferred", "strict"), default="deferred",
                    help="N>1: when the other ranks' completion flags of a step are waited for")
    ap.add_argument("--peer-backend", choices=("auto", "ipc", "symmetric"), default="auto",
                    help="N>1: how the ranks' copies of C are made reachable (symmetric memory offers multicast)")
    ap.add_argument("--weighted-rows", action="store_true",
                    help="N>1: row blocks in proportion to each GPU's measured rate instead of equal blocks (on one 8-GPU "
                         "node the rates were within 4 % and the equal split was as fast)")
    ap.add_argument("--no-multicast", action="store_true", help="N>1: unicast peer stores even when a multicast mapping exists")
    ap.add_argument("--preheat-s", type=float, default=2.0,
                    help="untimed warm-up continues until this many seconds of steps have run (0 = exactly --warmup steps)")
    ap.add_argument("--case", default=None, help="run one small case (for profiler captures) and print its timing")
    ap.add_argument("--iters", type=int, default=3, help="launches of --case")
    ap.add_argument("--sweep", action="store_true", help="the reference harness's demo shape + 20 square sizes, with parity per size")
    ap.add_argument("--sweep-log", default=None, help="file for the output.log-format text of --sweep")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
        return
    if args.case:
        run_case(args)
        return
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = max(args.warmup, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
