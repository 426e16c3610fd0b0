"""Operator-level entry points on torch CUDA tensors.

Names follow the reference's Frontend operators (include/Frontend/Operators.h:73-98):
`matmul` (+ fused `relu`, the `@fuse_matmul_relu` graph of README.md:9-26 with the ReLU of
src/Frontend/Operators.cc:232-244 folded into the epilogue) and `fmha`
(BatchedMatmul(Q, K^T) -> Softmax -> BatchedMatmul(P, V), test/test.cc:88-90).

torch is used for device memory and streams only; the arithmetic is done by the hand-written
sm_100a kernels behind the C-ABI.  Nothing here falls back to torch math.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import capi

_PRECISIONS = {"3xtf32": capi.KCG_PREC_3XTF32, "tf32": capi.KCG_PREC_TF32, "bf16": capi.KCG_PREC_BF16}
_workspaces: dict = {}


def _dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return capi.KCG_F32
    if dt == torch.bfloat16:
        return capi.KCG_BF16
    raise TypeError(f"unsupported dtype {dt}: the kernels take float32 or bfloat16")


def _workspace(device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Grow-only scratch buffer per (device, stream)."""
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("kernelcodegen_b200 operators need CUDA tensors; there is no CPU path")
        if t.device != dev:
            raise RuntimeError("all tensors must live on the same device")
    return dev


def matmul(a: torch.Tensor, b: torch.Tensor, *, relu: bool = False, precision: Optional[str] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           b_col_major: bool = False, tile_n: int = 0, stages: int = 0, group_m: int = 0,
           cta_group: int = 0, peers: Sequence[int] = (), mc: int = 0, done_flags: Sequence[int] = (),
           done_value: int = 0) -> torch.Tensor:
    """C = A . B (optionally ReLU'd).  A is [M, K] row-major; B is [K, N] row-major, or
    [N, K] when `b_col_major` (the reference's Layout::colMajor).  fp32 inputs use the
    3xTF32 path unless `precision="tf32"`; bf16 inputs use the bf16 path.
    `peers` are raw device pointers of other ranks' C buffers that also receive every tile;
    `mc` is the multicast address of `out` (every tile is then stored once and delivered to all
    ranks by the switch); `done_flags` are the words that receive `done_value` when the launch,
    and all its stores, have completed (see `peer.SymmetricMatrix`)."""
    dev = _require_cuda(a, b)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("matmul takes 2-D tensors")
    M, K = a.shape
    if b_col_major:
        N, Kb = b.shape
    else:
        Kb, N = b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: A is {tuple(a.shape)}, B is {tuple(b.shape)}")
    if a.dtype != b.dtype:
        raise TypeError("A and B must have the same dtype")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("A and B must be row-contiguous (stride 1 in the last dimension)")
    if precision is None:
        precision = "bf16" if a.dtype == torch.bfloat16 else "3xtf32"
    if precision not in _PRECISIONS:
        raise ValueError(f"precision must be one of {sorted(_PRECISIONS)}")
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    elif out.shape != (M, N) or out.stride(1) != 1 or out.device != dev:
        raise ValueError("out has the wrong shape, stride or device")
    d = capi.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.lda, d.ldb, d.ldc = a.stride(0), b.stride(0), out.stride(0)
    d.dtype_in, d.dtype_out = _dtype_code(a.dtype), _dtype_code(out.dtype)
    d.precision = _PRECISIONS[precision]
    d.epilogue = capi.KCG_EPI_RELU if relu else capi.KCG_EPI_NONE
    d.b_layout = capi.KCG_COL_MAJOR if b_col_major else capi.KCG_ROW_MAJOR
    d.tile_n, d.stages, d.group_m = tile_n, stages, group_m
    d.cta_group = cta_group
    d.n_peers = len(peers)
    for i, p in enumerate(peers):
        d.peer_c[i] = p
    d.mc_c = mc or None
    d.n_done_flags = len(done_flags)
    d.done_value = done_value & 0xFFFFFFFF
    for i, p in enumerate(done_flags):
        d.done_flags[i] = p
    lib = capi.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.kcg_gemm_workspace_bytes(ctypes.byref(d))
        ws = _workspace(dev, ws_bytes)
        stream = torch.cuda.current_stream(dev).cuda_stream
        st = lib.kcg_gemm_launch(ctypes.byref(d), a.data_ptr(), b.data_ptr(), out.data_ptr(),
                                 ws.data_ptr() if ws is not None else None, ws_bytes, stream)
    capi.check(st, "kcg_gemm_launch")
    return out


def matmul_host(a_host: torch.Tensor, b_host: Optional[torch.Tensor], c_host: torch.Tensor, a_dev: torch.Tensor,
                b_dev: torch.Tensor, c_dev: torch.Tensor, *, relu: bool = False, precision: Optional[str] = None,
                b_col_major: bool = False, chunks: int = 0, peers: Sequence[int] = ()) -> torch.Tensor:
    """c_host = A . B from HOST arrays (pin them for the copies to overlap), staged through the
    caller's device arrays of the same shapes: row chunks of A and column chunks of B are copied
    while the kernel already runs on the tiles that have arrived, and finished strips of C return
    to the host meanwhile (`kcg_gemm_host_staged`).  `b_host=None`: B is already in `b_dev`.
    Asynchronous: synchronise the current stream before reading `c_host`."""
    dev = _require_cuda(a_dev, b_dev, c_dev)
    for h, t in ((a_host, a_dev), (b_host, b_dev), (c_host, c_dev)):
        if h is None and t is b_dev:
            continue
        if h.is_cuda or h.shape != t.shape or h.dtype != t.dtype or h.stride() != t.stride():
            raise ValueError("host and device arrays must match in shape, dtype and strides")
        if h.dim() != 2 or h.stride(1) != 1:
            raise ValueError("2-D row-contiguous arrays expected")
    M, K = a_dev.shape
    N = b_dev.shape[0] if b_col_major else b_dev.shape[1]
    if (b_dev.shape[1] if b_col_major else b_dev.shape[0]) != K or c_dev.shape != (M, N):
        raise ValueError("shapes do not form a product")
    if precision is None:
        precision = "bf16" if a_dev.dtype == torch.bfloat16 else "3xtf32"
    d = capi.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.lda, d.ldb, d.ldc = a_dev.stride(0), b_dev.stride(0), c_dev.stride(0)
    d.dtype_in, d.dtype_out = _dtype_code(a_dev.dtype), _dtype_code(c_dev.dtype)
    d.precision = _PRECISIONS[precision]
    d.epilogue = capi.KCG_EPI_RELU if relu else capi.KCG_EPI_NONE
    d.b_layout = capi.KCG_COL_MAJOR if b_col_major else capi.KCG_ROW_MAJOR
    d.n_peers = len(peers)
    for i, p in enumerate(peers):
        d.peer_c[i] = p
    lib = capi.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.kcg_gemm_workspace_bytes(ctypes.byref(d))
        ws = _workspace(dev, ws_bytes)
        st = lib.kcg_gemm_host_staged(ctypes.byref(d), a_host.data_ptr(),
                                      b_host.data_ptr() if b_host is not None else None, c_host.data_ptr(),
                                      a_dev.data_ptr(), b_dev.data_ptr(), c_dev.data_ptr(),
                                      ws.data_ptr() if ws is not None else None, ws_bytes, chunks,
                                      torch.cuda.current_stream(dev).cuda_stream)
    capi.check(st, "kcg_gemm_host_staged")
    return c_host


def matmul_relu(a: torch.Tensor, b: torch.Tensor, **kw) -> torch.Tensor:
    """The `@fuse_matmul_relu` operator: max(0, A . B)."""
    return matmul(a, b, relu=True, **kw)


def fmha(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0, causal: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """O = softmax(scale * Q K^T [causal]) V over [B, H, S, D] tensors.
    scale=1, causal=False is exactly the reference's three-operator graph."""
    dev = _require_cuda(q, k, v)
    if q.dim() != 4 or k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
        raise ValueError("expected Q [B,H,Sq,D] and K, V [B,H,Skv,D]")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("Q, K, V must be contiguous [B,H,S,D]")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("Q, K, V must share a dtype")
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else q.dtype
    if out is None:
        out = torch.empty((B, H, Sq, D), dtype=out_dtype, device=dev)
    elif out.shape != q.shape or not out.is_contiguous() or out.device != dev:
        raise ValueError("out has the wrong shape, stride or device")
    d = capi.FmhaDesc()
    d.B, d.H, d.Sq, d.Skv, d.D = B, H, Sq, Skv, D
    d.dtype_in, d.dtype_out = _dtype_code(q.dtype), _dtype_code(out.dtype)
    d.causal = 1 if causal else 0
    d.scale = float(scale)
    lib = capi.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.kcg_fmha_workspace_bytes(ctypes.byref(d))
        ws = _workspace(dev, ws_bytes)
        stream = torch.cuda.current_stream(dev).cuda_stream
        st = lib.kcg_fmha_fwd_launch(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                     ws.data_ptr() if ws is not None else None, ws_bytes, stream)
    capi.check(st, "kcg_fmha_fwd_launch")
    return out


def softmax(x: torch.Tensor, *, inplace: bool = False) -> torch.Tensor:
    """Last-axis softmax of an fp32 tensor (the reference's standalone Softmax operator)."""
    dev = _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise TypeError("softmax takes a contiguous float32 tensor")
    y = x if inplace else torch.empty_like(x)
    cols = x.shape[-1]
    rows = x.numel() // cols
    with torch.cuda.device(dev):
        st = capi.load().kcg_softmax_launch(rows, cols, x.data_ptr(), y.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    capi.check(st, "kcg_softmax_launch")
    return y


def transpose(x: torch.Tensor) -> torch.Tensor:
    """y[..., j, i] = x[..., i, j] as a new contiguous tensor (the reference's Transpose operator,
    which it declares without a body); leading dimensions are batch dimensions."""
    dev = _require_cuda(x)
    if x.dim() < 2 or not x.is_contiguous():
        raise ValueError("transpose takes a contiguous tensor of at least 2 dimensions")
    rows, cols = x.shape[-2:]
    batch = x.numel() // max(1, rows * cols)
    y = torch.empty(x.shape[:-2] + (cols, rows), dtype=x.dtype, device=dev)
    if x.numel() == 0:
        return y
    with torch.cuda.device(dev):
        st = capi.load().kcg_transpose_launch(batch, rows, cols, _dtype_code(x.dtype), x.data_ptr(), y.data_ptr(),
                                              torch.cuda.current_stream(dev).cuda_stream)
    capi.check(st, "kcg_transpose_launch")
    return y


def batched_matmul(a: torch.Tensor, b: torch.Tensor, *, b_col_major: bool = False, precision: Optional[str] = None,
                   relu: bool = False) -> torch.Tensor:
    """C[..., m, n] = A[..., m, k] . B[..., k, n]  (B[..., n, k] when `b_col_major`): the
    reference's standalone BatchedMatmul operator; leading dimensions are batch dimensions."""
    dev = _require_cuda(a, b)
    if a.dim() < 2 or a.dim() != b.dim() or a.shape[:-2] != b.shape[:-2]:
        raise ValueError("A and B need equal batch dimensions")
    if not (a.is_contiguous() and b.is_contiguous()) or a.dtype != b.dtype:
        raise ValueError("A and B must be contiguous and share a dtype")
    m, k = a.shape[-2:]
    n, kb = (b.shape[-2], b.shape[-1]) if b_col_major else (b.shape[-1], b.shape[-2])
    if k != kb:
        raise ValueError("inner dimensions differ")
    batch = 1
    for s_ in a.shape[:-2]:
        batch *= s_
    out = torch.empty(a.shape[:-2] + (m, n), dtype=a.dtype, device=dev)
    if precision is None:
        precision = "bf16" if a.dtype == torch.bfloat16 else "3xtf32"
    d = capi.GemmDesc()
    d.M, d.N, d.K = m, n, k
    d.lda, d.ldb, d.ldc = k, (k if b_col_major else n), n
    d.dtype_in = d.dtype_out = _dtype_code(a.dtype)
    d.precision = _PRECISIONS[precision]
    d.epilogue = capi.KCG_EPI_RELU if relu else capi.KCG_EPI_NONE
    d.b_layout = capi.KCG_COL_MAJOR if b_col_major else capi.KCG_ROW_MAJOR
    lib = capi.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.kcg_batched_gemm_workspace_bytes(ctypes.byref(d), batch, m * k, k * n)
        ws = _workspace(dev, ws_bytes)
        st = lib.kcg_batched_gemm_launch(ctypes.byref(d), batch, m * k, k * n, m * n, a.data_ptr(), b.data_ptr(),
                                         out.data_ptr(), ws.data_ptr() if ws is not None else None, ws_bytes,
                                         torch.cuda.current_stream(dev).cuda_stream)
    capi.check(st, "kcg_batched_gemm_launch")
    return out


def peer_wait(flags_ptr: int, n: int, stride_words: int, value: int, device: torch.device, max_polls: int = 0) -> None:
    """Queues, on the current stream, a bounded device-side wait until the `n` flag words at
    `flags_ptr` (stride in 32-bit words) have reached `value`."""
    with torch.cuda.device(device):
        st = capi.load().kcg_peer_wait_launch(flags_ptr, n, stride_words, value & 0xFFFFFFFF, max_polls,
                                              torch.cuda.current_stream(device).cuda_stream)
    capi.check(st, "kcg_peer_wait_launch")


def peer_wait_status() -> None:
    """Synchronises and raises KcgError(KCG_PEER_TIMEOUT / KCG_DEVICE_TIMEOUT) if a bounded wait ran out."""
    capi.check(capi.load().kcg_peer_wait_status(), "kcg_peer_wait_status")


def last_device_status() -> int:
    """0, or the code of the bounded device-side wait that ran out (synchronises)."""
    return int(capi.load().kcg_last_device_status())


def launch_count() -> int:
    return int(capi.load().kcg_launch_count())
