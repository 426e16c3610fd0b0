"""ctypes/numpy front end of the C oracle (`oracle.c`).  TEST INFRASTRUCTURE ONLY.

Only tests/, `__graft_entry__.smoke()` and bench.py's CPU-baseline legs may import this; the
product package (`kernelcodegen_b200`) never does.  Parity is unpinned by the reference's own
tests (it has none for numbers); see the header of `oracle.c`.
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int64
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return LIB_PATH


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(str(LIB_PATH))
        fp, dp, ip = POINTER(c_float), POINTER(c_double), POINTER(c_int64)
        lib.oracle_matmul_f32.argtypes = [fp, fp, fp] + [c_int64] * 6
        lib.oracle_matmul_f32_mt.argtypes = [fp, fp, fp] + [c_int64] * 6 + [c_int]
        lib.oracle_matmul_rows_f32.argtypes = [fp, fp, fp, ip] + [c_int64] * 5
        lib.oracle_matmul_rows_f64.argtypes = [fp, fp, dp, ip] + [c_int64] * 5
        lib.oracle_relu_f32.argtypes = [fp, c_int64]
        lib.oracle_batched_matmul_f32.argtypes = [fp, fp, fp] + [c_int64] * 4 + [c_int]
        lib.oracle_softmax_f32.argtypes = [fp, c_int64, c_int64]
        lib.oracle_fmha_f32.argtypes = [fp, fp, fp, fp] + [c_int64] * 4 + [c_float, c_int, c_int]
        lib.oracle_fmha_rows_f64.argtypes = [fp, fp, fp, dp, c_int64, ip] + [c_int64] * 4 + [c_double, c_int]
        lib.oracle_max_threads.restype = c_int
        for name in ("oracle_matmul_f32", "oracle_matmul_f32_mt", "oracle_matmul_rows_f32", "oracle_matmul_rows_f64",
                     "oracle_relu_f32", "oracle_batched_matmul_f32", "oracle_softmax_f32", "oracle_fmha_f32",
                     "oracle_fmha_rows_f64"):
            getattr(lib, name).restype = None
        _lib = lib
    return _lib


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


def _p(a: np.ndarray, t=c_float):
    return a.ctypes.data_as(POINTER(t))


def max_threads() -> int:
    return int(_load().oracle_max_threads())


def matmul(a, b, threads: int = 1) -> np.ndarray:
    """C = A.B by the reference's nest (fp32, k innermost and sequential)."""
    a, b = _f32(a), _f32(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), dtype=np.float32)
    if threads == 1:
        _load().oracle_matmul_f32(_p(a), _p(b), _p(c), m, n, k, k, n, n)
    else:
        _load().oracle_matmul_f32_mt(_p(a), _p(b), _p(c), m, n, k, k, n, n, threads)
    return c


def relu(x) -> np.ndarray:
    y = _f32(x).copy()
    _load().oracle_relu_f32(_p(y), y.size)
    return y


def matmul_relu(a, b, threads: int = 1) -> np.ndarray:
    """The @fuse_matmul_relu graph: Matmul followed by in-place Relu."""
    c = matmul(a, b, threads)
    _load().oracle_relu_f32(_p(c), c.size)
    return c


def matmul_rows(a, b, rows, f64: bool = False) -> np.ndarray:
    """Rows `rows` of A.B; fp32 nest, or fp64 accumulation when `f64`."""
    a, b = _f32(a), _f32(b)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    k, n = b.shape
    if f64:
        c = np.empty((len(rows), n), dtype=np.float64)
        _load().oracle_matmul_rows_f64(_p(a), _p(b), _p(c, c_double), _p(rows, c_int64), len(rows), n, k, a.shape[1], n)
    else:
        c = np.empty((len(rows), n), dtype=np.float32)
        _load().oracle_matmul_rows_f32(_p(a), _p(b), _p(c), _p(rows, c_int64), len(rows), n, k, a.shape[1], n)
    return c


def batched_matmul(a, b, b_col_major: bool = False) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    batch = int(np.prod(a.shape[:-2])) if a.ndim > 2 else 1
    m, k = a.shape[-2:]
    n = b.shape[-2] if b_col_major else b.shape[-1]
    c = np.empty(a.shape[:-2] + (m, n), dtype=np.float32)
    _load().oracle_batched_matmul_f32(_p(a), _p(b), _p(c), batch, m, n, k, int(b_col_major))
    return c


def transpose(x) -> np.ndarray:
    """out[..., j, i] = in[..., i, j], copied.  The reference declares this operator
    (include/Frontend/Operators.h:100-102) without a body (src/Frontend/Operators.cc:422-423);
    the definition is the index swap its name states."""
    return np.ascontiguousarray(np.swapaxes(np.asarray(x), -1, -2))


def softmax(x) -> np.ndarray:
    y = _f32(x).copy()
    cols = y.shape[-1]
    _load().oracle_softmax_f32(_p(y), y.size // cols, cols)
    return y


def fmha(q, k, v, scale: float = 1.0, causal: bool = False, threads: int = 1) -> np.ndarray:
    """softmax(scale * Q K^T) V per (batch, head), fp32 nests composed as in the reference's graph."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    *lead, sq, d = q.shape
    skv = k.shape[-2]
    bh = int(np.prod(lead)) if lead else 1
    o = np.empty_like(q)
    _load().oracle_fmha_f32(_p(q), _p(k), _p(v), _p(o), bh, sq, skv, d, scale, int(causal), threads)
    return o


def fmha_rows_f64(q, k, v, bh: int, rows, scale: float = 1.0, causal: bool = False) -> np.ndarray:
    """float64 attention output for query rows `rows` of flattened (batch*head) index `bh`."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    sq, d = q.shape[-2:]
    skv = k.shape[-2]
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    o = np.empty((len(rows), d), dtype=np.float64)
    _load().oracle_fmha_rows_f64(_p(q), _p(k), _p(v), _p(o, c_double), bh, _p(rows, c_int64), len(rows), sq, skv, d,
                                 float(scale), int(causal))
    return o
