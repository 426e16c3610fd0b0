"""The entry point that allocates nothing (`kcg_gemm_launch_static`).

Some users of this library cannot allocate device memory when they call it -- a plug-in inside
a host program whose own allocator already owns the whole GPU, or a serving loop that must not
hit the device-wide synchronisation an allocation brings -- so they cannot pass the workspace
`kcg_gemm_launch` wants for the fp32-contract (3xTF32) path.  For them the library carries a
fixed 32 MiB scratch array per GPU.  This test calls that entry point through the C-ABI twice
in a row, with different shapes and data, and holds each result to the workspace-taking entry
point's result (same kernels, so the same 1e-4 bar as the other fp32 tests; in practice they
agree bit for bit) and to the CPU nest.  It also checks that repeated calls change neither the
device's free memory nor torch's allocator statistics, and that a problem beyond the built-in
scratch is refused.

The file name sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4


def _desc(capi, m, n, k, relu=True):
    d = capi.GemmDesc()
    d.M, d.N, d.K = m, n, k
    d.lda, d.ldb, d.ldc = k, n, n
    d.dtype_in = d.dtype_out = capi.KCG_F32
    d.precision = capi.KCG_PREC_3XTF32
    d.epilogue = capi.KCG_EPI_RELU if relu else capi.KCG_EPI_NONE
    return d


def _rel_err(x, ref):
    return ((x.double() - ref.double()).abs().max() / ref.double().abs().max().clamp_min(1e-30)).item()


def test_static_scratch_entry_matches_workspace_entry_twice(cuda_device):
    import numpy as np

    from kernelcodegen_b200 import capi, ops
    from oracle import oracle

    lib = capi.load()
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    # second call is smaller than the first: anything the first call left in the shared scratch
    # beyond the second call's extent must not leak into its result
    for call, (m, n, k, seed) in enumerate([(512, 1024, 768, 1), (256, 384, 200, 2)]):
        g = torch.Generator().manual_seed(seed)
        a_h = torch.rand((m, k), generator=g) * 2 - 1
        b_h = torch.rand((k, n), generator=g) * 2 - 1
        a, b = a_h.to(cuda_device), b_h.to(cuda_device)
        want = ops.matmul_relu(a, b)  # existing entry point, workspace allocated by the caller
        got = torch.full((m, n), float("nan"), device=cuda_device)
        d = _desc(capi, m, n, k)
        st = lib.kcg_gemm_launch_static(ctypes.byref(d), a.data_ptr(), b.data_ptr(), got.data_ptr(), stream)
        assert st == capi.KCG_OK, f"call {call}: {capi.status_str(st)}"
        torch.cuda.synchronize()
        assert ops.last_device_status() == 0
        assert torch.isfinite(got).all()
        assert _rel_err(got, want) <= FP32_TOL, f"call {call}"
        # and against the CPU nest itself, not only against the library's other entry point
        cpu = torch.from_numpy(oracle.matmul_relu(a_h.numpy(), b_h.numpy()))
        assert _rel_err(got.cpu(), cpu) <= FP32_TOL, f"call {call} vs the CPU nest"


def test_static_scratch_entry_allocates_nothing(cuda_device):
    """After a first call (which loads the module holding the scratch array and looks up its
    address), further calls leave the device's free memory and torch's allocator untouched."""
    from kernelcodegen_b200 import capi

    lib = capi.load()
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    m, n, k = 384, 512, 256
    a = torch.rand((m, k), device=cuda_device)
    b = torch.rand((k, n), device=cuda_device)
    c = torch.empty((m, n), device=cuda_device)
    d = _desc(capi, m, n, k)
    assert lib.kcg_gemm_launch_static(ctypes.byref(d), a.data_ptr(), b.data_ptr(), c.data_ptr(), stream) == capi.KCG_OK
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(cuda_device)
    stats0 = (torch.cuda.memory_allocated(cuda_device), torch.cuda.memory_reserved(cuda_device))
    for _ in range(5):
        assert lib.kcg_gemm_launch_static(ctypes.byref(d), a.data_ptr(), b.data_ptr(), c.data_ptr(), stream) == capi.KCG_OK
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(cuda_device)
    assert free1 == free0, "device free memory changed across calls that must not allocate"
    assert (torch.cuda.memory_allocated(cuda_device), torch.cuda.memory_reserved(cuda_device)) == stats0


def test_static_scratch_entry_refuses_what_does_not_fit(cuda_device):
    from kernelcodegen_b200 import capi

    lib = capi.load()
    m, n, k = 4096, 2048, 2048  # needs 4 * (m*k + k*n) = 48 MiB of scratch, the array holds 32 MiB
    d = _desc(capi, m, n, k)
    assert lib.kcg_gemm_workspace_bytes(ctypes.byref(d)) > capi.KCG_STATIC_SCRATCH_BYTES
    a = torch.zeros((m, k), device=cuda_device)
    b = torch.zeros((k, n), device=cuda_device)
    c = torch.zeros((m, n), device=cuda_device)
    st = lib.kcg_gemm_launch_static(ctypes.byref(d), a.data_ptr(), b.data_ptr(), c.data_ptr(), None)
    assert st == capi.KCG_TOO_LARGE, capi.status_str(st)
    d2 = _desc(capi, 128, 128, 128)
    d2.precision = capi.KCG_PREC_TF32  # paths without scratch are not served by this entry point
    st = lib.kcg_gemm_launch_static(ctypes.byref(d2), a.data_ptr(), b.data_ptr(), c.data_ptr(), None)
    assert st == capi.KCG_UNSUPPORTED, capi.status_str(st)
