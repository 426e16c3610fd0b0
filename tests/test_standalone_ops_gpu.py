"""GPU parity of the standalone BatchedMatmul and Softmax operators (the reference's Frontend
ops used outside an attention chain) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def rel_err(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.mark.parametrize("shape", [(5, 7, 33), (4, 128), (3, 1000), (2, 3, 1024), (6, 4100), (1, 1), (2, 8192), (300, 516), (3, 2050),
                                   (2, 16384), (1, 49152), (2, 50000)])
def test_softmax_matches_oracle(cuda_device, shape):
    from kernelcodegen_b200 import ops

    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g) * 3
    want = oracle.softmax(x.numpy())
    # The nest adds a row's exponentials one after the other in fp32; on rows of tens of thousands
    # of columns that sum alone drifts past 1e-5 of the exact quotient.  The kernel is held to
    # 1e-5 of the float64 value, and to the nest within the nest's own distance from it.
    x64 = x.numpy().astype(np.float64)
    e = np.exp(x64 - x64.max(-1, keepdims=True))
    exact = e / e.sum(-1, keepdims=True)
    nest_drift = rel_err(want, exact)
    got = ops.softmax(x.to(cuda_device))
    assert rel_err(got.cpu().numpy(), exact) <= 1e-5
    assert rel_err(got.cpu().numpy(), want) <= 1e-5 + nest_drift
    np.testing.assert_allclose(got.sum(-1).cpu().numpy(), 1.0, atol=1e-5)
    xin = x.to(cuda_device).clone()
    assert ops.softmax(xin, inplace=True) is xin
    assert rel_err(xin.cpu().numpy(), exact) <= 1e-5


def test_softmax_golden(cuda_device, golden):
    from kernelcodegen_b200 import ops

    got = ops.softmax(torch.from_numpy(golden["sm_x"]).to(cuda_device))
    assert rel_err(got.cpu().numpy(), golden["sm_y"]) <= 1e-5


@pytest.mark.parametrize("b_col_major", [False, True])
def test_batched_matmul_matches_oracle(cuda_device, b_col_major):
    from kernelcodegen_b200 import ops

    g = torch.Generator().manual_seed(7)
    a = torch.rand((2, 3, 200, 72), generator=g) * 2 - 1
    b = torch.rand((2, 3, 136, 72) if b_col_major else (2, 3, 72, 136), generator=g) * 2 - 1
    want = oracle.batched_matmul(a.numpy(), b.numpy(), b_col_major=b_col_major)
    got = ops.batched_matmul(a.to(cuda_device), b.to(cuda_device), b_col_major=b_col_major)
    assert rel_err(got.cpu().numpy(), want) <= 1e-4
    gb = ops.batched_matmul(a.bfloat16().to(cuda_device), b.bfloat16().to(cuda_device), b_col_major=b_col_major)
    wantb = oracle.batched_matmul(a.bfloat16().float().numpy(), b.bfloat16().float().numpy(), b_col_major=b_col_major)
    assert rel_err(gb.float().cpu().numpy(), wantb) <= 2e-2
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("batch,m,n,k", [(64, 128, 128, 64), (5, 300, 72, 40), (3, 130, 260, 132), (17, 64, 8, 8)])
@pytest.mark.parametrize("precision,tol", [("3xtf32", 1e-4), ("tf32", 5e-3)])
def test_batched_matmul_one_launch_many_entries(cuda_device, batch, m, n, k, precision, tol):
    """All entries go through one launch (batch = third tensor-map coordinate): ragged entries
    must not read their neighbours' rows, and the launch count says it was one GEMM launch."""
    from kernelcodegen_b200 import ops

    g = torch.Generator().manual_seed(batch * 1000 + m)
    a = torch.rand((batch, m, k), generator=g) * 2 - 1
    b = torch.rand((batch, k, n), generator=g) * 2 - 1
    want = oracle.batched_matmul(a.numpy(), b.numpy())
    before = ops.launch_count()
    got = ops.batched_matmul(a.to(cuda_device), b.to(cuda_device), precision=precision)
    launches = ops.launch_count() - before
    assert launches == (2 if precision == "3xtf32" else 1)      # residual pass + GEMM, or the GEMM alone
    assert rel_err(got.cpu().numpy(), want) <= tol
    assert ops.last_device_status() == 0


def test_batched_matmul_shared_operand(cuda_device):
    """stride 0: one B for every entry (split once for 3xTF32), through the C-ABI."""
    import ctypes

    from kernelcodegen_b200 import capi

    lib = capi.load()
    batch, m, n, k = 6, 200, 136, 72
    g = torch.Generator().manual_seed(9)
    a = (torch.rand((batch, m, k), generator=g) * 2 - 1).to(cuda_device)
    b = (torch.rand((k, n), generator=g) * 2 - 1).to(cuda_device)
    c = torch.full((batch, m, n), float("nan"), device=cuda_device)
    d = capi.GemmDesc()
    d.M, d.N, d.K = m, n, k
    d.lda, d.ldb, d.ldc = k, n, n
    d.dtype_in = d.dtype_out = capi.KCG_F32
    d.precision = capi.KCG_PREC_3XTF32
    need = lib.kcg_batched_gemm_workspace_bytes(ctypes.byref(d), batch, m * k, 0)
    assert need >= 4 * (batch * m * k + k * n)
    ws = torch.empty(need, dtype=torch.uint8, device=cuda_device)
    st = lib.kcg_batched_gemm_launch(ctypes.byref(d), batch, m * k, 0, m * n, a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                     ws.data_ptr(), need, None)
    assert st == capi.KCG_OK, capi.status_str(st)
    torch.cuda.synchronize()
    want = np.stack([oracle.matmul(a[i].cpu().numpy(), b.cpu().numpy()) for i in range(batch)])
    assert rel_err(c.cpu().numpy(), want) <= 1e-4
    # an entry stride that is not a multiple of 16 bytes is refused
    st = lib.kcg_batched_gemm_launch(ctypes.byref(d), batch, m * k + 1, 0, m * n, a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                     ws.data_ptr(), need, None)
    assert st == capi.KCG_BAD_ALIGN


def test_unfused_attention_graph_equals_fused_kernel(cuda_device):
    """BatchedMatmul(Q, K^T) -> Softmax -> BatchedMatmul(P, V) run operator by operator gives the
    fused FMHA kernel's answer (to the bf16 bar of the fused kernel)."""
    from kernelcodegen_b200 import ops

    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn((1, 2, 256, 64), generator=g).to(cuda_device) * s for s in (0.4, 0.4, 1.0))
    p = ops.softmax(ops.batched_matmul(q, k, b_col_major=True), inplace=True)
    o_graph = ops.batched_matmul(p, v)
    o_fused = ops.fmha(q, k, v, scale=1.0)
    want = oracle.fmha(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    assert rel_err(o_graph.cpu().numpy(), want) <= 1e-4          # fp32-contract operators
    assert rel_err(o_fused.cpu().numpy(), o_graph.cpu().numpy()) <= 2e-2


@pytest.mark.parametrize("shape", [(64, 64), (4096, 1024), (3, 300, 520), (2, 5, 130, 66), (1, 7), (129, 1), (1000, 1002),
                                   (2, 264, 392), (640, 136)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_transpose_is_exact(cuda_device, shape, dtype):
    """Moves bits only: the result must equal the index-swapped input exactly (vector path for
    multiples of 4, element-wise path for ragged tiles and odd shapes)."""
    from kernelcodegen_b200 import ops
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g).to(dtype)
    got = ops.transpose(x.to(cuda_device))
    want = oracle.transpose(x.float().numpy())
    assert got.shape == want.shape and got.is_contiguous()
    assert np.array_equal(got.float().cpu().numpy(), want)
    # twice is the identity
    assert torch.equal(ops.transpose(got).cpu(), x)
    assert ops.last_device_status() == 0
