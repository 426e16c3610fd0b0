"""Small, self-contained invocations of each kernel for profiling (`ncu`) and quick timing.

    python -m kernelcodegen_b200.profile_cases <case> [--iters N]

Cases hold at most a few hundred MB on the device (but more than the 126 MB L2 where DRAM
figures matter) and launch the kernel a handful of times, so a profiler capture of one to
three launches ends by itself within a minute or two.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import ops


def _time(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def gemm_bf16(iters, size=8192):
    dev = torch.device("cuda:0")
    a = (torch.randn((size, size), device=dev) * 0.02).bfloat16()
    b = (torch.randn((size, size), device=dev) * 0.02).bfloat16()
    c = torch.empty((size, size), device=dev, dtype=torch.bfloat16)
    ms = _time(lambda: ops.matmul_relu(a, b, out=c), iters)
    return ms, 2.0 * size ** 3


def gemm_3xtf32(iters):
    dev = torch.device("cuda:0")
    a = torch.rand((4096, 1024), device=dev) * 2 - 1
    b = torch.rand((1024, 2048), device=dev) * 2 - 1
    c = torch.empty((4096, 2048), device=dev)
    ms = _time(lambda: ops.matmul_relu(a, b, out=c), iters)
    return ms, 2.0 * 4096 * 2048 * 1024


def gemm_3xtf32_large(iters):
    dev = torch.device("cuda:0")
    a = torch.rand((8192, 8192), device=dev) * 2 - 1
    b = torch.rand((8192, 8192), device=dev) * 2 - 1
    c = torch.empty((8192, 8192), device=dev)
    ms = _time(lambda: ops.matmul_relu(a, b, out=c), iters)
    return ms, 2.0 * 8192 ** 3


def fmha_causal(iters, b=2, h=16, s=8192, d=128):
    dev = torch.device("cuda:0")
    q, k, v = (torch.randn((b, h, s, d), device=dev).bfloat16() for _ in range(3))
    o = torch.empty_like(q)
    ms = _time(lambda: ops.fmha(q, k, v, scale=1.0 / math.sqrt(d), causal=True, out=o), iters)
    return ms, 2.0 * b * h * s * s * d


def fmha_fp32(iters):
    dev = torch.device("cuda:0")
    q, k, v = (torch.randn((4, 16, 1024, 64), device=dev) for _ in range(3))
    o = torch.empty_like(q)
    ms = _time(lambda: ops.fmha(q, k, v, scale=0.125, out=o), iters)
    return ms, 4.0 * 4 * 16 * 1024 * 1024 * 64


def transpose_fp32(iters):
    """8192 x 8192 fp32: 256 MiB in, 256 MiB out.  The second figure printed is bytes moved, so the
    rate reads as GB/s x 1000 in the TFLOP/s column's place (see main)."""
    dev = torch.device("cuda:0")
    x = torch.randn((8192, 8192), device=dev)
    ms = _time(lambda: ops.transpose(x), iters)
    return ms, 2.0 * x.numel() * 4


BYTE_CASES = {"transpose_fp32"}   # the work figure of these cases is bytes, not flop

CASES = {"transpose_fp32": transpose_fp32, "gemm_bf16": gemm_bf16, "gemm_3xtf32": gemm_3xtf32, "gemm_3xtf32_large": gemm_3xtf32_large,
         "fmha_causal": fmha_causal, "fmha_fp32": fmha_fp32}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    ms, flop = CASES[args.case](args.iters)
    rate = f"{flop / ms / 1e6:.0f} GB/s" if args.case in BYTE_CASES else f"{flop / ms / 1e9:.1f} TFLOP/s"
    print(f"{args.case}: {ms:.4f} ms/launch  {rate}  device_status={ops.last_device_status()}")


if __name__ == "__main__":
    main()
