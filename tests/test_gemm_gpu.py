"""GPU parity tests of the matmul(+ReLU) kernels against the CPU oracle, through the C-ABI.

Error metric (same for every case): max|x - ref| / max|ref| over the compared elements.
Bars: fp32 contract (3xTF32) <= 1e-4; bf16 paths <= 2e-2 against an fp32/fp64-accumulated
product of the bf16-rounded inputs; single-pass TF32 <= 5e-3 (stated, not a headline path).
"""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 2e-2
TF32_TOL = 5e-3


def rel_err(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))


def uniform(shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.rand(shape, generator=g, dtype=torch.float32) * 2 - 1


def test_golden_tile_fp32_and_bf16(cuda_device, golden):
    from kernelcodegen_b200 import ops

    a = torch.from_numpy(golden["mm2_a"]).to(cuda_device)
    b = torch.from_numpy(golden["mm2_b"]).to(cuda_device)
    c = ops.matmul_relu(a, b)
    assert rel_err(c.cpu().numpy(), golden["mm2_relu"]) <= FP32_TOL
    cb = ops.matmul_relu(a.bfloat16(), b.bfloat16())
    ref = oracle.matmul_relu(a.bfloat16().float().cpu().numpy(), b.bfloat16().float().cpu().numpy())
    assert rel_err(cb.float().cpu().numpy(), ref) <= BF16_TOL
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("m,n,k", [(128, 128, 32), (256, 512, 256), (200, 328, 136), (1, 8, 8), (130, 260, 36), (640, 384, 1000)])
@pytest.mark.parametrize("b_col_major", [False, True])
def test_fp32_contract_small_shapes(cuda_device, m, n, k, b_col_major):
    from kernelcodegen_b200 import ops

    a, b = uniform((m, k), 100 + m), uniform((k, n), 200 + n)
    want = oracle.matmul_relu(a.numpy(), b.numpy())
    bd = b.t().contiguous() if b_col_major else b
    for tile_n in (128, 256):
        for cta_group in (1, 2):   # single CTAs and CTA pairs (tcgen05 cta_group::2)
            got = ops.matmul_relu(a.to(cuda_device), bd.to(cuda_device), b_col_major=b_col_major, tile_n=tile_n,
                                  cta_group=cta_group)
            assert rel_err(got.cpu().numpy(), want) <= FP32_TOL
            assert (got >= 0).all()
    plain = ops.matmul(a.to(cuda_device), bd.to(cuda_device), b_col_major=b_col_major)
    assert rel_err(plain.cpu().numpy(), oracle.matmul(a.numpy(), b.numpy())) <= FP32_TOL
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (200, 328, 136), (8, 8, 8), (384, 640, 320)])
@pytest.mark.parametrize("b_col_major", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_bf16_small_shapes(cuda_device, m, n, k, b_col_major, out_dtype):
    from kernelcodegen_b200 import ops

    a, b = uniform((m, k), 300 + m).bfloat16(), uniform((k, n), 400 + n).bfloat16()
    want = oracle.matmul_relu(a.float().numpy(), b.float().numpy())
    bd = b.t().contiguous() if b_col_major else b
    for tile_n in (128, 256):
        for cta_group in (1, 2):
            got = ops.matmul_relu(a.to(cuda_device), bd.to(cuda_device), b_col_major=b_col_major, tile_n=tile_n,
                                  out_dtype=out_dtype, cta_group=cta_group)
            assert got.dtype == out_dtype
            tol = BF16_TOL if out_dtype == torch.bfloat16 else 5e-5  # fp32 output: exact products, fp32 sums
            assert rel_err(got.float().cpu().numpy(), want) <= tol
    assert ops.last_device_status() == 0


def test_tf32_single_pass(cuda_device):
    from kernelcodegen_b200 import ops

    a, b = uniform((256, 192), 1), uniform((192, 384), 2)
    want = oracle.matmul_relu(a.numpy(), b.numpy())
    for b_col_major in (False, True):
        bd = b.t().contiguous() if b_col_major else b
        got = ops.matmul_relu(a.to(cuda_device), bd.to(cuda_device), precision="tf32", b_col_major=b_col_major)
        assert rel_err(got.cpu().numpy(), want) <= TF32_TOL


def test_config_fuse_matmul_relu_4096x1024x2048(cuda_device):
    """The headline fp32 config: A 4096x1024, B 1024x2048, uniform[-1,1], seeds 0/1.
    Oracle on 256 sampled rows (all columns); full-tensor properties on the GPU result."""
    from kernelcodegen_b200 import ops

    a, b = uniform((4096, 1024), 0), uniform((1024, 2048), 1)
    ad, bd = a.to(cuda_device), b.to(cuda_device)
    c = ops.matmul_relu(ad, bd)
    rows = np.random.default_rng(0).choice(4096, size=256, replace=False)
    rows.sort()
    want = np.maximum(oracle.matmul_rows(a.numpy(), b.numpy(), rows), 0)
    assert rel_err(c[torch.from_numpy(rows).to(cuda_device)].cpu().numpy(), want) <= FP32_TOL
    # ReLU is exactly max(0, .) of the un-fused product
    plain = ops.matmul(ad, bd)
    assert torch.equal(c, torch.clamp_min(plain, 0))
    # linearity in A (size-independent property): (2A).B == 2(A.B) exactly in binary fp
    assert torch.equal(ops.matmul(ad * 2, bd), plain * 2)
    # both tile widths, single CTAs and CTA pairs agree to rounding
    assert rel_err(ops.matmul_relu(ad, bd, tile_n=256).cpu().numpy(), c.cpu().numpy()) <= 1e-5
    assert rel_err(ops.matmul_relu(ad, bd, cta_group=1).cpu().numpy(), c.cpu().numpy()) <= 1e-5
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("size,nrows", [(1024, 64), (2048, 64), (4096, 32), (8192, 16)])
def test_config_square_sweep_fp32(cuda_device, size, nrows):
    from kernelcodegen_b200 import ops

    idx = {1024: 0, 2048: 1, 4096: 2, 8192: 3}[size]
    g = torch.Generator(device=cuda_device).manual_seed(10 + idx)
    a = torch.rand((size, size), generator=g, device=cuda_device) * 2 - 1
    b = torch.rand((size, size), generator=g, device=cuda_device) * 2 - 1
    c = ops.matmul_relu(a, b)
    rows = np.linspace(0, size - 1, nrows).astype(np.int64)
    ncols = 512  # sampled columns keep the scalar oracle to seconds
    cols = np.linspace(0, size - 1, ncols).astype(np.int64)
    a_rows = a[torch.from_numpy(rows).to(cuda_device)].cpu().numpy()
    b_cols = b[:, torch.from_numpy(cols).to(cuda_device)].contiguous().cpu().numpy()
    want = np.maximum(oracle.matmul(a_rows, b_cols, threads=0), 0)
    got = c[torch.from_numpy(rows).to(cuda_device)][:, torch.from_numpy(cols).to(cuda_device)].cpu().numpy()
    assert rel_err(got, want) <= FP32_TOL
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("size", [4096, 32768])
def test_config_large_bf16_matmul_relu(cuda_device, size):
    """bf16 inputs N(0, 0.02), fp32 accumulate, bf16 output; sampled rows/columns in fp64."""
    from kernelcodegen_b200 import ops

    g = torch.Generator(device=cuda_device).manual_seed(40)
    a = (torch.randn((size, size), generator=g, device=cuda_device) * 0.02).bfloat16()
    g.manual_seed(41)
    b = (torch.randn((size, size), generator=g, device=cuda_device) * 0.02).bfloat16()
    c = ops.matmul_relu(a, b)
    rows = np.array([0, 1, 127, 128, size // 2 + 3, size - 129, size - 1], dtype=np.int64)
    cols = np.linspace(0, size - 1, 256).astype(np.int64)
    a_rows = a[torch.from_numpy(rows).to(cuda_device)].float().cpu().numpy()
    b_cols = b[:, torch.from_numpy(cols).to(cuda_device)].float().contiguous().cpu().numpy()
    want = np.maximum(oracle.matmul_rows(a_rows, b_cols, np.arange(len(rows)), f64=True), 0)
    got = c[torch.from_numpy(rows).to(cuda_device)][:, torch.from_numpy(cols).to(cuda_device)].float().cpu().numpy()
    assert rel_err(got, want) <= BF16_TOL
    assert (c >= 0).all()
    # halving A halves the product exactly (power of two), up to the bf16 output rounding being identical
    assert torch.equal(ops.matmul_relu(a * 0.5, b), c * 0.5)
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("m,n,k,b_col_major", [(128, 256, 16384, False), (200, 136, 9000, True), (256, 128, 12288, False)])
def test_fp32_contract_holds_for_long_k(cuda_device, m, n, k, b_col_major):
    """Products with K > 8192 run as several launches over K ranges that add into C with
    round-to-nearest fp32 adds: the tensor core's truncating accumulator would otherwise drift
    past the 1e-4 contract near K = 12000 (1.45e-4 at 16384 in one launch)."""
    from kernelcodegen_b200 import ops

    a = uniform((m, k), 70)
    b = uniform((n, k) if b_col_major else (k, n), 71)
    bb = b.t().contiguous() if b_col_major else b
    rows = list(range(0, m, max(1, m // 16)))
    want = np.maximum(oracle.matmul_rows(a.numpy(), bb.numpy(), rows), 0.0)
    exact = np.maximum(oracle.matmul_rows(a.numpy(), bb.numpy(), rows, f64=True), 0.0)
    before = ops.launch_count()
    c = ops.matmul_relu(a.to(cuda_device), b.to(cuda_device), b_col_major=b_col_major)
    assert ops.launch_count() - before == 1 + (k + 4095) // 4096      # residual pass + one launch per K range
    got = c.cpu().numpy()[rows]
    assert rel_err(got, want) <= FP32_TOL
    assert rel_err(got, exact) <= 5e-5
    assert (c >= 0).all() and ops.last_device_status() == 0


def test_strided_operands_and_out(cuda_device):
    from kernelcodegen_b200 import ops

    a_full, b_full = uniform((256, 320), 7).to(cuda_device), uniform((192, 512), 8).to(cuda_device)
    a, b = a_full[:, :192], b_full[:, :256]  # leading dimensions larger than the extents
    out_full = torch.full((256, 384), -7.0, device=cuda_device)
    out = out_full[:, :256]
    ops.matmul_relu(a, b, out=out)
    want = oracle.matmul_relu(a.contiguous().cpu().numpy(), b.contiguous().cpu().numpy())
    assert rel_err(out.cpu().numpy(), want) <= FP32_TOL
    assert (out_full[:, 256:] == -7.0).all()  # nothing written past N


def test_error_statuses(cuda_device):
    from kernelcodegen_b200 import capi, ops

    a = torch.zeros((128, 130), device=cuda_device)
    b = torch.zeros((130, 128), device=cuda_device)
    with pytest.raises(capi.KcgError) as ei:  # row pitch of A is not a multiple of 16 bytes
        ops.matmul(a, b)
    assert ei.value.status == capi.KCG_BAD_ALIGN
    with pytest.raises(ValueError):
        ops.matmul(torch.zeros((128, 64), device=cuda_device), torch.zeros((32, 128), device=cuda_device))
    with pytest.raises(TypeError):
        ops.matmul(torch.zeros((128, 64), device=cuda_device, dtype=torch.float16),
                   torch.zeros((64, 128), device=cuda_device, dtype=torch.float16))


def test_host_buffer_entry_point(cuda_device):
    import ctypes

    from kernelcodegen_b200 import capi

    lib = capi.load()
    a, b = uniform((256, 128), 11).numpy(), uniform((128, 384), 12).numpy()
    c = np.empty((256, 384), dtype=np.float32)
    d = capi.GemmDesc()
    d.M, d.N, d.K = 256, 384, 128
    d.lda, d.ldb, d.ldc = 128, 384, 384
    d.dtype_in = d.dtype_out = capi.KCG_F32
    d.precision = capi.KCG_PREC_3XTF32
    d.epilogue = capi.KCG_EPI_RELU
    st = lib.kcg_gemm_host(ctypes.byref(d), a.ctypes.data, b.ctypes.data, c.ctypes.data)
    assert st == capi.KCG_OK, capi.status_str(st)
    assert rel_err(c, oracle.matmul_relu(a, b)) <= FP32_TOL


def test_bounded_wait_reports_timeout_and_context_survives(cuda_device):
    """A device-side wait on a barrier nothing arrives on gives up after its iteration cap,
    records a status code and returns; the context stays usable."""
    from kernelcodegen_b200 import capi, ops

    lib = capi.load()
    assert lib.kcg_selftest_wait_timeout(2000) == capi.KCG_DEVICE_TIMEOUT
    assert ops.last_device_status() == 0  # the self-test consumed and cleared the word
    a = uniform((128, 64), 1).to(cuda_device)
    b = uniform((64, 128), 2).to(cuda_device)
    assert rel_err(ops.matmul(a, b).cpu().numpy(), oracle.matmul(a.cpu().numpy(), b.cpu().numpy())) <= FP32_TOL


def test_harness_log_is_readable_like_the_reference_log(cuda_device):
    """The run-and-compare harness prints the reference's log format (performance/output.log)
    and its lines parse back with the plot script's field positions."""
    import io

    from kernelcodegen_b200 import harness

    buf = io.StringIO()
    r0 = harness.run_case(4096, 2048, 1024, True, out=buf)
    r1 = harness.run_case(512, 512, 512, True, out=buf)
    text = buf.getvalue()
    assert "My Matmul Latency = " in text and "cublas Ratio(TT) = " in text and " --- K --- : 1024" in text
    rows = harness.parse_log(text)
    assert len(rows) == 2 and all(all(x and x > 0 for x in row) for row in rows)
    assert abs(rows[0][0] - r0["mine_ms"]) / r0["mine_ms"] < 1e-3
    assert r0["rel_err"] <= FP32_TOL and r1["rel_err"] <= FP32_TOL
