"""The shared-K tail of the CTA-pair GEMM: when the tiles do not fill the last wave of the
persistent grid, the k-blocks of the left-over tiles are divided between all CTA pairs and the
partial accumulators are added up in the workspace.  Checked against the CPU oracle, against the
same launch without the tail (workspace withheld), and for run-to-run bit stability."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def rel_err(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))


def uniform(shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.rand(shape, generator=g, dtype=torch.float32) * 2 - 1


def _launch(a, b, relu, precision, with_tail, tile_n=0, b_col_major=False):
    """kcg_gemm_launch on CTA pairs, with the whole workspace or only the residual arrays."""
    from kernelcodegen_b200 import capi, ops
    lib = capi.load()
    m, k = a.shape
    n = b.shape[0] if b_col_major else b.shape[1]
    out = torch.empty((m, n), dtype=a.dtype, device=a.device)
    d = capi.GemmDesc()
    d.M, d.N, d.K = m, n, k
    d.lda, d.ldb, d.ldc = a.stride(0), b.stride(0), n
    d.dtype_in = d.dtype_out = capi.KCG_BF16 if a.dtype == torch.bfloat16 else capi.KCG_F32
    d.precision = {"bf16": capi.KCG_PREC_BF16, "tf32": capi.KCG_PREC_TF32, "3xtf32": capi.KCG_PREC_3XTF32}[precision]
    d.epilogue = capi.KCG_EPI_RELU if relu else capi.KCG_EPI_NONE
    d.b_layout = capi.KCG_COL_MAJOR if b_col_major else capi.KCG_ROW_MAJOR
    d.cta_group, d.tile_n = 2, tile_n
    tail_tiles = lib.kcg_gemm_shared_k_tiles(ctypes.byref(d))
    full = lib.kcg_gemm_workspace_bytes(ctypes.byref(d))
    lo = 4 * (m * k + k * n) if precision == "3xtf32" else 0
    nbytes = full if with_tail else lo
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=a.device)
    st = lib.kcg_gemm_launch(ctypes.byref(d), a.data_ptr(), b.data_ptr(), out.data_ptr(), ws.data_ptr(), nbytes,
                             torch.cuda.current_stream().cuda_stream)
    capi.check(st, "kcg_gemm_launch")
    torch.cuda.synchronize()
    assert ops.last_device_status() == 0
    return out, tail_tiles


@pytest.mark.parametrize("m,n,k,tile_n", [
    (4096, 2048, 1024, 0),     # the fuse_matmul_relu shape: 3 waves + 34 tiles
    (1024, 1024, 1024, 0),     # fewer tiles than pairs: every tile shares its K range
    (2048, 2048, 2048, 0),     # one wave + 54 tiles: ranges that end one tile and begin the next
    (1000, 1096, 1032, 0),     # ragged edges in M, N and K
    (1024, 2048, 1024, 256),   # 256-wide tiles
])
def test_fp32_contract_with_shared_k_tail(cuda_device, m, n, k, tile_n):
    a, b = uniform((m, k), 7 + m).to(cuda_device), uniform((k, n), 11 + n).to(cuda_device)
    got, tail_tiles = _launch(a, b, True, "3xtf32", True, tile_n)
    assert tail_tiles > 0, "this shape is meant to exercise the shared-K tail"
    rows = np.unique(np.linspace(0, m - 1, 48).astype(np.int64))
    want = np.maximum(oracle.matmul_rows(a.cpu().numpy(), b.cpu().numpy(), rows), 0)
    assert rel_err(got[torch.from_numpy(rows).to(cuda_device)].cpu().numpy(), want) <= 1e-4
    # the same launch without the tail: the K range is accumulated in two to four pieces instead of
    # one, which moves the fp32 accumulators' roundings (far inside the 1e-4 contract)
    plain, _ = _launch(a, b, True, "3xtf32", False, tile_n)
    assert rel_err(got.cpu().numpy(), plain.cpu().numpy()) <= 2e-5
    # whoever finishes last, the partial sums are added in a fixed order
    again, _ = _launch(a, b, True, "3xtf32", True, tile_n)
    assert torch.equal(got, again)


@pytest.mark.parametrize("b_col_major", [False, True])
def test_bf16_with_shared_k_tail(cuda_device, b_col_major):
    m = n = k = 4096           # 256 tiles of 256x256 on 74 pairs
    a = uniform((m, k), 3).bfloat16().to(cuda_device)
    b = uniform((n, k) if b_col_major else (k, n), 4).bfloat16().to(cuda_device)
    got, tail_tiles = _launch(a, b, True, "bf16", True, 0, b_col_major)
    assert tail_tiles == 34
    rows = np.unique(np.linspace(0, m - 1, 24).astype(np.int64))
    bb = b.float().cpu().numpy()
    want = np.maximum(oracle.matmul_rows(a.float().cpu().numpy(), bb.T.copy() if b_col_major else bb, rows, f64=True), 0)
    assert rel_err(got[torch.from_numpy(rows).to(cuda_device)].float().cpu().numpy(), want) <= 2e-2
    plain, _ = _launch(a, b, True, "bf16", False, 0, b_col_major)
    assert rel_err(got.float().cpu().numpy(), plain.float().cpu().numpy()) <= 8e-3   # one bf16 rounding step
    again, _ = _launch(a, b, True, "bf16", True, 0, b_col_major)
    assert torch.equal(got, again)


def test_tail_counters_are_left_clean(cuda_device):
    """Fifty launches in a row reuse the library's arrival counters; every result must match."""
    a, b = uniform((1024, 512), 5).to(cuda_device), uniform((512, 1024), 6).to(cuda_device)
    first, tail_tiles = _launch(a, b, False, "3xtf32", True)
    assert tail_tiles > 0
    for _ in range(50):
        again, _ = _launch(a, b, False, "3xtf32", True)
        assert torch.equal(first, again)
