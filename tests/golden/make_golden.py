"""Generates tests/golden/kat_small.npz: small seeded inputs and float64 evaluations of the
operator definitions (independent of oracle.c: plain numpy float64 formulas).

The reference project has no numeric tests or golden vectors of its own and cannot be run here
(it needs LLVM/MLIR 15 and has no executor), so these vectors pin the oracle against an
independent evaluation of the same definitions:
  matmul   C[i,j] = sum_k A[i,k] B[k,j]              (src/Frontend/Operators.cc:140-173)
  relu     max(0, x)                                 (src/Frontend/Operators.cc:232-244)
  bmm NT   C[b,i,j] = sum_k A[b,i,k] B[b,j,k]        (src/Frontend/Operators.cc:353-414)
  softmax  exp(x) / sum(exp(x)) over the last axis   (src/Frontend/Operators.cc:474-536)
  fmha     softmax(scale * Q K^T [+causal]) V        (test/test.cc:88-90)

Run:  python tests/golden/make_golden.py
"""
from pathlib import Path

import numpy as np


def softmax64(x):
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def fmha64(q, k, v, scale, causal):
    s = np.einsum("...id,...jd->...ij", q.astype(np.float64), k.astype(np.float64)) * scale
    if causal:
        sq, skv = s.shape[-2:]
        i = np.arange(sq)[:, None]
        j = np.arange(skv)[None, :]
        s = np.where(j > i + (skv - sq), -np.inf, s)
    return softmax64(s) @ v.astype(np.float64)


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    a = rng.uniform(-1, 1, (37, 53)).astype(np.float32)
    b = rng.uniform(-1, 1, (53, 29)).astype(np.float32)
    out["mm_a"], out["mm_b"] = a, b
    out["mm_c"] = a.astype(np.float64) @ b.astype(np.float64)
    out["mm_relu"] = np.maximum(out["mm_c"], 0.0)
    # a tile-sized case for the GPU kernels (one 128x128 tile, K = 64)
    a2 = rng.uniform(-1, 1, (128, 64)).astype(np.float32)
    b2 = rng.uniform(-1, 1, (64, 128)).astype(np.float32)
    out["mm2_a"], out["mm2_b"] = a2, b2
    out["mm2_relu"] = np.maximum(a2.astype(np.float64) @ b2.astype(np.float64), 0.0).astype(np.float32)
    ba = rng.standard_normal((2, 3, 16, 8)).astype(np.float32)
    bb = rng.standard_normal((2, 3, 12, 8)).astype(np.float32)
    out["bmm_a"], out["bmm_b"] = ba, bb
    out["bmm_nt"] = np.einsum("...ik,...jk->...ij", ba.astype(np.float64), bb.astype(np.float64))
    sx = rng.standard_normal((5, 7, 33)).astype(np.float32) * 3
    out["sm_x"] = sx
    out["sm_y"] = softmax64(sx.astype(np.float64))
    q = rng.standard_normal((2, 2, 40, 16)).astype(np.float32)
    k = rng.standard_normal((2, 2, 56, 16)).astype(np.float32)
    v = rng.standard_normal((2, 2, 56, 16)).astype(np.float32)
    out["fa_q"], out["fa_k"], out["fa_v"] = q, k, v
    out["fa_o_ref"] = fmha64(q, k, v, 1.0, False)          # the reference graph: no scale, no mask
    out["fa_o_scaled_causal"] = fmha64(q, k, v, 0.25, True)
    # a kernel-sized case (128 queries, 256 keys, head dim 64), inputs exactly representable in bf16
    def bf16_round(x):
        u = x.astype(np.float32).view(np.uint32)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        return u.astype(np.uint32).view(np.float32)
    q2 = bf16_round(rng.standard_normal((1, 2, 128, 64)))
    k2 = bf16_round(rng.standard_normal((1, 2, 256, 64)))
    v2 = bf16_round(rng.standard_normal((1, 2, 256, 64)))
    out["fa2_q"], out["fa2_k"], out["fa2_v"] = q2, k2, v2
    out["fa2_o"] = fmha64(q2, k2, v2, 0.125, False).astype(np.float32)
    out["fa2_o_causal"] = fmha64(q2, k2, v2, 0.125, True).astype(np.float32)
    path = Path(__file__).resolve().parent / "kat_small.npz"
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
