"""Run-and-compare harness for the fp32 matmul, in the output format of the reference's own
(absent, git-ignored) `test/matmul` harness, evidenced by performance/output.log:1-13:

    Matrix size :
     --- M --- : 4096
     --- N --- : 2048
     --- K --- : 1024

    Occupancy: ...
    My Matmul Latency = 1.80746 ms

    cublas Latency(NN) = 1.70506 ms
    cublas Ratio(NN) = 94.3346%

    cublas Latency(TT) = ...
    cublas Ratio(TT) = ...

so that the reference's performance/plot.py parser (lines 50-86) can read the log unchanged.
"My Matmul" is the 3xTF32 tcgen05 kernel (fp32 contract, ReLU off, as in the reference's
measurements); the cuBLAS lines are `torch.matmul` in fp32 (TF32 off), NN and TT.

    python -m kernelcodegen_b200.harness [--sizes 256 512 ...] [--check]
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import ops

# the reference's sweep (test/test.cc:37)
SWEEP = [256, 512, 768, 1024, 1536, 2048, 3072, 4096, 5120, 6144, 7168, 8192, 9216, 10240, 11264, 12288, 13312, 14336,
         15360, 16384]


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _cta_threads(m: int, n: int, k: int) -> int:
    """Threads per CTA of the launch the library chooses for this fp32 product."""
    import ctypes

    from . import capi

    d = capi.GemmDesc()
    d.M, d.N, d.K = m, n, k
    d.lda, d.ldb, d.ldc = k, n, n
    d.dtype_in = d.dtype_out = capi.KCG_F32
    d.precision = capi.KCG_PREC_3XTF32
    geo = (ctypes.c_int32 * 6)()
    capi.check(capi.load().kcg_gemm_launch_geometry(ctypes.byref(d), geo), "kcg_gemm_launch_geometry")
    return int(geo[1])


def run_case(m: int, n: int, k: int, check: bool, out=sys.stdout) -> dict:
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(m * 31 + n * 17 + k)
    a = torch.rand((m, k), generator=g, device=dev) * 2 - 1
    b = torch.rand((k, n), generator=g, device=dev) * 2 - 1
    c = torch.empty((m, n), device=dev)
    iters = max(3, min(50, int(2e11 / (2.0 * m * n * k)) + 3))
    mine = _time(lambda: ops.matmul(a, b, out=c), iters)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = torch.empty_like(c)
    nn = _time(lambda: torch.matmul(a, b, out=ref), iters)
    at, bt = a.t().contiguous(), b.t().contiguous()
    ct = torch.empty((n, m), device=dev)
    tt = _time(lambda: torch.matmul(bt, at, out=ct), iters)   # (A.B)^T = B^T.A^T: both operands transposed
    torch.backends.cuda.matmul.allow_tf32 = True
    tf32 = _time(lambda: torch.matmul(a, b, out=ref), iters)    # the library's one-pass TF32 product, for scale
    torch.backends.cuda.matmul.allow_tf32 = False
    err = None
    if check:
        err = ((c.double() - a.double() @ b.double()).abs().max() / (a.double() @ b.double()).abs().max()).item()
    torch.backends.cuda.matmul.allow_tf32 = old
    print("Matrix size : ", file=out)
    print(f" --- M --- : {m}\n --- N --- : {n}\n --- K --- : {k}\n", file=out)
    threads = _cta_threads(m, n, k)
    print(f"Occupancy: {100.0 * threads / 2048:.1f}% (one {threads}-thread CTA per SM; the work is done by TMA and the tensor core)",
          file=out)
    print(f"My Matmul Latency = {mine:.6g} ms\n", file=out)
    print(f"cublas Latency(NN) = {nn:.6g} ms", file=out)
    print(f"cublas Ratio(NN) = {100.0 * nn / mine:.6g}%\n", file=out)
    print(f"cublas Latency(TT) = {tt:.6g} ms", file=out)
    print(f"cublas Ratio(TT) = {100.0 * tt / mine:.6g}%\n", file=out)
    if err is not None:
        print(f"max relative error vs fp64 = {err:.3e}", file=out)
    return {"m": m, "n": n, "k": k, "mine_ms": mine, "cublas_nn_ms": nn, "cublas_tt_ms": tt, "cublas_tf32_ms": tf32,
            "rel_err": err}


def parse_log(text: str):
    """Reads a log the way the reference's plot script does: the first 'Matrix size' block is the
    demo shape, the following ones are the square sweep.  Returns a list of
    (my_ms, cublas_nn_ms, cublas_tt_ms) per block."""
    rows, cur = [], None
    for line in text.splitlines():
        if "Matrix size" in line:
            cur = [None, None, None]
            rows.append(cur)
        elif cur is not None and line.startswith("My"):
            cur[0] = float(line.split(" ")[4])
        elif cur is not None and "cublas Latency(NN)" in line:
            cur[1] = float(line.split(" ")[3])
        elif cur is not None and "cublas Latency(TT)" in line:
            cur[2] = float(line.split(" ")[3])
    return [tuple(r) for r in rows]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="*", default=SWEEP)
    ap.add_argument("--check", action="store_true", help="also print the error against an fp64 product")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the harness needs a CUDA device")
    run_case(4096, 2048, 1024, args.check)      # the demo shape first, as in the reference's log
    for s in args.sizes:
        run_case(s, s, s, args.check)


if __name__ == "__main__":
    main()
