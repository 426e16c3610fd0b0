"""Host-buffer GEMM with overlapped copies (`kcg_gemm_host_staged`) against the device-resident
entry point and the CPU oracle: every chunking must give the product the single launch gives."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _mk(shape, dtype, seed, dev):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return ((torch.rand(shape, generator=g) * 2 - 1).to(dtype)).to(dev)


@pytest.mark.parametrize("chunks", [0, 1, 2, 3, 5, 16])
@pytest.mark.parametrize("m,n,k,dtype,b_col_major", [
    (2304, 3080, 512, torch.bfloat16, False),
    (1000, 4104, 320, torch.bfloat16, True),
    (1536, 1284, 260, torch.float32, False),
    (300, 520, 128, torch.float32, True),
])
def test_staged_equals_single_launch(m, n, k, dtype, b_col_major, chunks):
    from kernelcodegen_b200 import ops
    dev = torch.device("cuda:0")
    a = _mk((m, k), dtype, 1, dev)
    b = _mk((n, k) if b_col_major else (k, n), dtype, 2, dev)
    want = ops.matmul(a, b, relu=True, b_col_major=b_col_major)
    a_h, b_h = a.cpu().pin_memory(), b.cpu().pin_memory()
    c_h = torch.full((m, n), float("nan"), dtype=dtype).pin_memory()
    a_d, b_d, c_d = torch.zeros_like(a), torch.zeros_like(b), torch.zeros_like(want)
    for _ in range(2):  # the second call reuses the library's streams and events
        c_h.fill_(float("nan"))
        ops.matmul_host(a_h, b_h, c_h, a_d, b_d, c_d, relu=True, b_col_major=b_col_major, chunks=chunks)
        torch.cuda.synchronize()
        assert ops.last_device_status() == 0
        assert torch.equal(c_h, want.cpu())
        assert torch.equal(c_d, want)


def test_staged_with_b_already_on_the_device():
    """hB = NULL: only A moves in and C out; B is whatever the device array holds."""
    from kernelcodegen_b200 import ops
    dev = torch.device("cuda:0")
    m, n, k = 4300, 2056, 512
    a, b = _mk((m, k), torch.bfloat16, 7, dev), _mk((k, n), torch.bfloat16, 8, dev)
    want = ops.matmul(a, b, relu=True)
    a_h = a.cpu().pin_memory()
    c_h = torch.full((m, n), float("nan"), dtype=torch.bfloat16).pin_memory()
    a_d, c_d = torch.zeros_like(a), torch.zeros_like(want)
    ops.matmul_host(a_h, None, c_h, a_d, b, c_d, relu=True)
    torch.cuda.synchronize()
    assert torch.equal(c_h, want.cpu()) and torch.equal(c_d, want)
    assert ops.last_device_status() == 0


def test_staged_pageable_host_memory_and_oracle():
    from kernelcodegen_b200 import ops
    from oracle import oracle
    dev = torch.device("cuda:0")
    m, n, k = 2100, 2056, 192
    a_h = _mk((m, k), torch.float32, 3, "cpu")
    b_h = _mk((k, n), torch.float32, 4, "cpu")
    c_h = torch.empty((m, n), dtype=torch.float32)
    a_d, b_d, c_d = a_h.to(dev) * 0, b_h.to(dev) * 0, torch.empty((m, n), device=dev)
    ops.matmul_host(a_h, b_h, c_h, a_d, b_d, c_d, relu=True)
    torch.cuda.synchronize()
    want = oracle.relu(oracle.matmul(a_h.numpy(), b_h.numpy()))
    scale = np.abs(want).max()
    assert np.abs(c_h.numpy() - want).max() / scale <= 1e-4  # the fp32 contract of the 3xTF32 path


def test_host_entry_allocates_and_pipelines():
    """`kcg_gemm_host` (allocating form) runs the same schedule."""
    import ctypes
    from kernelcodegen_b200 import capi, ops
    lib = capi.load()
    m, n, k = 4200, 4104, 256
    a = _mk((m, k), torch.bfloat16, 5, "cpu")
    b = _mk((k, n), torch.bfloat16, 6, "cpu")
    c = torch.empty((m, n), dtype=torch.bfloat16)
    d = capi.GemmDesc()
    d.M, d.N, d.K, d.lda, d.ldb, d.ldc = m, n, k, k, n, n
    d.dtype_in = d.dtype_out = capi.KCG_BF16
    d.precision = capi.KCG_PREC_BF16
    d.epilogue = capi.KCG_EPI_RELU
    capi.check(lib.kcg_gemm_host(ctypes.byref(d), a.data_ptr(), b.data_ptr(), c.data_ptr()), "kcg_gemm_host")
    want = ops.matmul(a.cuda(), b.cuda(), relu=True).cpu()
    assert torch.equal(c, want)


def test_staged_rejects_bad_arguments():
    import ctypes
    from kernelcodegen_b200 import capi
    lib = capi.load()
    d = capi.GemmDesc()
    d.M, d.N, d.K, d.lda, d.ldb, d.ldc = 256, 256, 64, 64, 256, 256
    d.dtype_in = d.dtype_out = capi.KCG_BF16
    d.precision = capi.KCG_PREC_BF16
    buf = torch.zeros(256 * 256, dtype=torch.bfloat16, device="cuda:0")
    host = torch.zeros(256 * 256, dtype=torch.bfloat16)
    p, h = buf.data_ptr(), host.data_ptr()
    assert lib.kcg_gemm_host_staged(ctypes.byref(d), h, h, h, p, p, None, None, 0, 0, None) == capi.KCG_BAD_ARGUMENT
    assert lib.kcg_gemm_host_staged(ctypes.byref(d), h, h, h, p, p, p, None, 0, 17, None) == capi.KCG_BAD_ARGUMENT
    d.ldc = 128
    assert lib.kcg_gemm_host_staged(ctypes.byref(d), h, h, h, p, p, p, None, 0, 0, None) == capi.KCG_BAD_SHAPE
