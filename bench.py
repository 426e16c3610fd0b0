#!/usr/bin/env python
"""Benchmark of the matmul+ReLU / FMHA kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0).  The workload of `value` is the same at every N so that the
per-N values form a strong-scaling curve: the large bf16 matmul+ReLU (M=N=K=32768, inputs
N(0, 0.02) in bf16, fp32 accumulate, bf16 output), A and C sharded by row blocks over the ranks,
every finished C tile stored into all ranks' copies of C by the GEMM epilogue itself (fused
all-gather over NVLink peer memory), one step = one full C on every rank.
At N=1 the line also carries the other configurations (`others`): the fp32-contract
4096x1024x2048 matmul+ReLU (3xTF32), the fp32 square sweep, and the two FMHA configs; at N>1
it carries the bf16 causal FMHA sharded by batch*head.

`--impl reference` times the CPU restatement of the reference's loop nest (the reference has
no executable CPU or GPU path of its own in this environment) on the host cores.
"""
from __future__ import annotations

import argparse
import json
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

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the bf16 GEMM kernel, from the
# ncu capture summarised in profiles/ (8192^3 case) scaled to 32768^3 by tiles processed.
# (profiles/gemm_bf16_8192_ncu.md: 1.011 GB read + 0.130 GB written.)
GEMM_BF16_DRAM_BYTES_PER_LAUNCH_8192 = 1.141e9


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained")}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = f"/tmp/kcg_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # "under load": samples whose power is above half of the highest seen
        hi = max(power)
        loaded = [c for c, p in zip(sm, power) if p >= 0.5 * hi] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": hi}


# ------------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference's nest, all host threads
# ------------------------------------------------------------------------------------------------
LARGE = 32768


def cpu_sample_inputs(rows: int, cols: int, k: int):
    import numpy as np

    rng = np.random.default_rng(40)
    a = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal((k, cols)) * 0.02).astype(np.float32)
    # round to bf16 (the workload's input type), keep as float for the fp32 nest
    def bf16(x):
        u = x.view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)
    return bf16(a), bf16(b)


def cpu_time_sample(rows: int, cols: int, k: int, threads: int) -> float:
    from oracle import oracle

    a, b = cpu_sample_inputs(rows, cols, k)
    t0 = time.perf_counter()
    oracle.matmul_relu(a, b, threads=threads)
    return time.perf_counter() - t0


def cpu_baseline(target_s: float = 12.0):
    """TFLOP/s of the reference nest on the host cores, on a bounded sample of the large GEMM:
    `rows` rows x 2048 columns of C at the full K = 32768."""
    from oracle import oracle

    oracle.build()
    threads = oracle.max_threads()
    cols, k = 2048, LARGE
    rows = max(1, threads // 16)
    t = cpu_time_sample(rows, cols, k, 0)
    if t < target_s / 2:
        rows = max(rows, int(rows * target_s / max(t, 1e-3)))
        rows = min(rows, 4096)
        t = cpu_time_sample(rows, cols, k, 0)
    flops = 2.0 * rows * cols * k
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{rows} rows x {cols} cols of C at K={k} (bf16-rounded inputs, fp32 nest), {t:.1f} s"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    oracle.build()
    threads = oracle.max_threads()
    cols, k = 2048, LARGE
    rows = max(1, threads // 16)
    t = cpu_time_sample(rows, cols, k, 0)  # calibration (also a warm-up of the thread pool)
    per_step_target = 4.0
    rows = max(1, min(4096, int(rows * per_step_target / max(t, 1e-3))))
    for _ in range(args.warmup):
        cpu_time_sample(rows, cols, k, 0)
    times = [cpu_time_sample(rows, cols, k, 0) for _ in range(args.steps)]
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
        "note": "the reference has no CPU executor and cannot be built here (needs LLVM/MLIR 15); this is the "
                "C restatement of its loop nest on all host threads",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
METRIC = "TFLOP/s & % tensor roofline: matmul+ReLU 4096x1024x2048, FMHA; 1/2/4/8 GPU"


def workload_config(n):
    return {"workload": "large bf16 matmul+ReLU M=N=K=32768 (bf16 in N(0,0.02), fp32 accumulate, bf16 out), "
                        "A/C sharded by row blocks, C all-gathered by peer stores in the GEMM epilogue",
            "M": LARGE, "N": LARGE, "K": LARGE, "parallelism": f"row-block x{n}",
            "cache": "inputs (2 GiB per operand) are larger than L2 (126 MB); no flush needed"}


def time_steps(fn, steps, warmup, torch, dist=None):
    """W warm-ups, then K steps between barrier+synchronize, CUDA events on the current stream;
    returns max-over-ranks milliseconds for the K steps."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
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


def flush_l2(torch, buf):
    buf.zero_()


def time_flushed(fn, iters, torch, flush_buf):
    """Per-launch time (median) with an L2 flush (a write larger than L2) between timed launches."""
    times = []
    for _ in range(iters):
        flush_l2(torch, flush_buf)
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


def others_single_gpu(torch, dev, peaks, ops):
    """The other configurations of the metric, 1 GPU, CUDA-event timed, L2 flushed between
    launches where the working set fits L2; one second of idle time before each (see settle)."""
    res = []
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    settle(torch)
    tf32_peak = measure_tf32_peak(torch, dev)
    x3_peak = tf32_peak / 3.0

    def uniform(shape, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        return torch.rand(shape, generator=g, device=dev) * 2 - 1

    # fuse_matmul_relu fp32 4096x1024x2048
    a, b = uniform((4096, 1024), 0), uniform((1024, 2048), 1)
    c = torch.empty((4096, 2048), device=dev)
    fn = lambda: ops.matmul_relu(a, b, out=c)
    for _ in range(3):
        fn()
    settle(torch)
    ms_cold = time_flushed(fn, 20, torch, flush_buf)
    ms_warm = time_steps(fn, 20, 3, torch) / 20
    fl = 2.0 * 4096 * 2048 * 1024
    res.append({"workload": "fuse_matmul_relu fp32 4096x1024x2048 (3xTF32, incl. hi/lo split pass)",
                "tflops": fl / ms_cold / 1e9, "ms": ms_cold, "tflops_warm_l2": fl / ms_warm / 1e9, "ms_warm_l2": ms_warm,
                "roofline": {"bound": "tensor", "achieved": fl / ms_cold / 1e9, "peak": x3_peak, "unit": "TFLOP/s",
                             "frac": fl / ms_cold / 1e9 / x3_peak,
                             "peak_def": f"cuBLAS TF32 8192^3 measured live ({tf32_peak:.0f}) / 3"},
                "timing": "L2 flushed between launches (cold, median of 20); warm = 20 back-to-back; 1 s idle before"})
    # fp32 square sweep
    for i, n in enumerate((1024, 2048, 4096, 8192)):
        a, b = uniform((n, n), 10 + i), uniform((n, n), 10 + i + 100)
        c = torch.empty((n, n), device=dev)
        fn = lambda: ops.matmul_relu(a, b, out=c)
        for _ in range(3):
            fn()
        settle(torch)
        ms = time_flushed(fn, 10, torch, flush_buf)
        fl = 2.0 * n ** 3
        res.append({"workload": f"fp32 matmul+ReLU {n}^3 (3xTF32)", "tflops": fl / ms / 1e9, "ms": ms,
                    "roofline": {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": x3_peak, "unit": "TFLOP/s",
                                 "frac": fl / ms / 1e9 / x3_peak}})
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
    settle(torch)
    ms = time_flushed(fn, 20, torch, flush_buf)
    fl = 4.0 * 4 * 16 * 1024 * 1024 * 64
    res.append({"workload": "FMHA fp32-in/out non-causal B4 H16 S1024 D64 (both contractions TF32 on the fp32 tiles, no conversion pass)",
                "tflops": fl / ms / 1e9, "ms": ms, "tolerance": "5e-3 (TF32 internals)",
                "roofline": {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": tf32_peak, "unit": "TFLOP/s",
                             "frac": fl / ms / 1e9 / tf32_peak,
                             "peak_def": "cuBLAS TF32 8192^3 measured live"}})
    res.append(fmha_long(torch, dev, peaks, ops, 0, 256))
    del qkv, o
    # Transpose (HBM-bound): 8192 x 8192 fp32, 256 MiB in + 256 MiB out, larger than L2
    x = torch.randn((8192, 8192), device=dev)
    for _ in range(3):
        y = ops.transpose(x)
    settle(torch)
    ms = time_steps(lambda: ops.transpose(x), 10, 0, torch, None) / 10
    nbytes = 2.0 * x.numel() * 4
    res.append({"workload": "Transpose 8192x8192 fp32 (read once, write once)", "gbs": nbytes / ms / 1e6, "ms": ms,
                "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"]}})
    del x, y
    return res, tf32_peak


def fmha_long(torch, dev, peaks, ops, bh_lo, bh_hi, dist=None, steps=5):
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
    for _ in range(3):
        settle(torch)
        batches.append(time_steps(fn, steps, 0, torch, dist) / steps)
    batches.sort()
    ms = batches[1]
    fl = 2.0 * 256 * 8192 * 8192 * 128  # whole job: causal = half of 4*B*H*S^2*D
    world = dist.get_world_size() if dist is not None else 1
    peak = peaks["bf16_tflops"] * world
    return {"workload": f"FMHA bf16 causal B8 H32 S8192 D128, batch*head sharded x{world}, no collective",
            "tflops": fl / ms / 1e9, "ms": ms, "ms_batches": batches,
            "roofline": {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": peak, "unit": "TFLOP/s",
                         "frac": fl / ms / 1e9 / peak}}


def run_ours(args):
    # Keep stdout for the one JSON line: anything a library prints to fd 1 (NCCL's version
    # banner, for instance) goes to stderr instead.
    json_fd = os.dup(1)
    os.dup2(2, 1)
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
    lo, hi = sharding.row_block(M, rank, world)
    rows = hi - lo
    # inputs: generated per row block from the seed, so each rank only makes its shard of A
    g = torch.Generator(device=dev)
    g.manual_seed(40 * 100003 + lo)
    a = torch.empty((rows, K), dtype=torch.bfloat16, device=dev)
    chunk = 2048
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        a[r0:r1] = (torch.randn((r1 - r0, K), generator=g, device=dev) * 0.02).bfloat16()
    g.manual_seed(41)
    b = torch.empty((K, N), dtype=torch.bfloat16, device=dev)
    for r0 in range(0, K, chunk):
        b[r0:r0 + chunk] = (torch.randn((chunk, N), generator=g, device=dev) * 0.02).bfloat16()

    cmat = peer.PeerMatrix(M, N, torch.bfloat16, dev) if world > 1 else None
    c_full = cmat.tensor if cmat is not None else torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    c_local = c_full[lo:hi]
    peers = cmat.peer_row_ptrs(lo) if cmat is not None else []
    sync_token = torch.zeros(1, device=dev)

    def step():
        ops.matmul_relu(a, b, out=c_local, peers=peers)
        if dist is not None:
            # all ranks' kernels (and with them their stores into this rank's C) are complete
            # once this stream-ordered all-reduce has run on every rank
            dist.all_reduce(sync_token)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = lib.kcg_launch_count()
    if sampler:
        sampler.start()
    ms_total = time_steps(step, args.steps, args.warmup, torch, dist)
    clocks = sampler.stop() if sampler else None
    launches = lib.kcg_launch_count() - launches0 - 0
    # launches counted over warm-up + timed steps on this rank; keep the timed share
    launches_timed = launches * args.steps // max(1, args.steps + args.warmup)
    if dist is not None:
        t = torch.tensor([launches_timed], device=dev, dtype=torch.int64)
        dist.all_reduce(t)
        launches_timed = int(t.item())
    status = ops.last_device_status()
    ms_step = ms_total / args.steps
    flops = 2.0 * M * N * K
    value = flops / ms_step / 1e9

    # all-gather check (outside the timed region): the first 128 rows of the next rank's block, as
    # they arrived in THIS rank's copy of C, against a local recomputation from the same seed
    allgather_check = None
    if dist is not None:
        nxt = (rank + 1) % world
        plo, phi = sharding.row_block(M, nxt, world)
        g2 = torch.Generator(device=dev)
        g2.manual_seed(40 * 100003 + plo)
        a_peer = (torch.randn((min(chunk, phi - plo), K), generator=g2, device=dev) * 0.02).bfloat16()[:128]
        want = ops.matmul_relu(a_peer.contiguous(), b)
        diff = (c_full[plo:plo + 128].float() - want.float()).abs().max()
        dist.all_reduce(diff, op=dist.ReduceOp.MAX)
        allgather_check = {"rows_checked_per_rank": 128, "max_abs_diff": float(diff.item())}
        del a_peer, want

    # kernel-only duration (no barrier): CUDA events around the GEMM launch alone
    def gemm_only():
        ops.matmul_relu(a, b, out=c_local, peers=peers)
    if dist is not None:
        dist.barrier()
    kernel_ms = time_steps(gemm_only, max(3, args.steps // 2), 1, torch, dist) / max(3, args.steps // 2)
    kernel_tflops = 2.0 * rows * N * K / kernel_ms / 1e9  # this rank's share (max-over-ranks time)
    peak_sust = peaks["bf16_tflops_sustained"]
    traffic = None
    if GEMM_BF16_DRAM_BYTES_PER_LAUNCH_8192 is not None:
        traffic = GEMM_BF16_DRAM_BYTES_PER_LAUNCH_8192 * (rows / 8192.0) * (N / 8192.0) * (K / 8192.0)
    roofline = {"bound": "tensor", "achieved": kernel_tflops, "peak": peak_sust, "unit": "TFLOP/s",
                "frac": kernel_tflops / peak_sust, "traffic": traffic,
                "kernel": "gemm_kernel<bf16, 128x256x64, 4 stages> (tcgen05/TMEM)",
                "peak_def": f"cuBLAS bf16 sustained, {peak_src} (burst {peaks['bf16_tflops']:.0f}: frac {kernel_tflops / peaks['bf16_tflops']:.3f})",
                "per_gpu": True, "flop_per_launch": 2.0 * rows * N * K, "kernel_ms": kernel_ms}

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
    tf32_peak = None
    # free the big operands before the other configs
    del a, b, c_local, c_full
    if cmat is not None:
        cmat.close()
    torch.cuda.empty_cache()
    if args.no_others:
        pass
    elif world == 1:
        others, tf32_peak = others_single_gpu(torch, dev, peaks, ops)
    else:
        blo, bhi = sharding.bh_shard(256, rank, world)
        others = [fmha_long(torch, dev, peaks, ops, blo, bhi, dist)]
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
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            "roofline": roofline, "e2e": e2e, "gpu_launches": launches_timed, "clocks": clocks,
            "device_status": [status, status2], "others": others,
        }
        if allgather_check is not None:
            line["allgather_check"] = allgather_check
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
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1)")
    ap.add_argument("--no-others", action="store_true", help="only the headline workload (for profiler launch lists)")
    ap.add_argument("--e2e-chunks", type=int, default=0, help="chunks per operand of the host-buffer GEMM (0 = library default)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = max(args.warmup, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
