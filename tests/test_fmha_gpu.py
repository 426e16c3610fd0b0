"""GPU parity tests of the FMHA kernel against the CPU oracle, through the C-ABI.

bf16 inputs, and fp32 inputs with head dimension 128 (rounded to bf16 by a pre-pass), run bf16
tensor-core contractions with fp32 accumulation and are held to the bf16 bar:
max|x - ref| / max|ref| <= 2e-2 against the oracle evaluated on the bf16-rounded inputs.
fp32 inputs with head dimension 64 run both contractions as TF32 products straight from the fp32
tiles and are held to 5e-3 against the oracle on the un-rounded inputs.
"""
import math

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2
TF32_TOL = 5e-3   # fp32 inputs, head dimension 64: both contractions as TF32 products


def rel_err(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))


def normal(shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32)


def test_golden_attention(cuda_device, golden):
    from kernelcodegen_b200 import ops

    q, k, v = (torch.from_numpy(golden[n]).to(cuda_device).bfloat16() for n in ("fa2_q", "fa2_k", "fa2_v"))
    o = ops.fmha(q, k, v, scale=0.125, out_dtype=torch.float32)
    assert rel_err(o.cpu().numpy(), golden["fa2_o"]) <= BF16_TOL
    oc = ops.fmha(q, k, v, scale=0.125, causal=True, out_dtype=torch.float32)
    assert rel_err(oc.cpu().numpy(), golden["fa2_o_causal"]) <= BF16_TOL
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("b,h,sq,skv,d", [(1, 1, 128, 128, 64), (1, 2, 256, 256, 128), (2, 3, 200, 200, 64),
                                          (1, 2, 200, 328, 128), (1, 1, 1, 17, 64), (1, 2, 384, 130, 128)])
@pytest.mark.parametrize("causal", [False, True])
def test_small_shapes_vs_oracle(cuda_device, b, h, sq, skv, d, causal):
    from kernelcodegen_b200 import ops

    q, k, v = normal((b, h, sq, d), 1).bfloat16(), normal((b, h, skv, d), 2).bfloat16(), normal((b, h, skv, d), 3).bfloat16()
    scale = 1.0 / math.sqrt(d)
    want = oracle.fmha(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale=scale, causal=causal, threads=0)
    for out_dtype in (torch.bfloat16, torch.float32):
        got = ops.fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=scale, causal=causal,
                       out_dtype=out_dtype)
        assert torch.isfinite(got.float()).all()
        assert rel_err(got.float().cpu().numpy(), want) <= BF16_TOL
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("b,h,sq,skv,d", [(1, 1, 128, 128, 64), (2, 3, 200, 200, 64), (1, 1, 1, 17, 64), (1, 2, 520, 392, 64),
                                          (3, 1, 256, 1030, 64), (1, 2, 200, 328, 128)])
@pytest.mark.parametrize("causal", [False, True])
def test_fp32_inputs_small_shapes_vs_oracle(cuda_device, b, h, sq, skv, d, causal):
    """fp32 Q, K, V.  Head dimension 64: TF32 contractions straight from the fp32 tiles, held to
    the TF32 bar against the oracle on the un-rounded inputs.  Head dimension 128: rounded to bf16
    by a separate pass, the same bits as the bf16-input kernel gets from pre-rounded inputs."""
    from kernelcodegen_b200 import ops

    q, k, v = normal((b, h, sq, d), 11), normal((b, h, skv, d), 12), normal((b, h, skv, d), 13)
    scale = 1.0 / math.sqrt(d)
    got = ops.fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=scale, causal=causal)
    assert got.dtype == torch.float32 and torch.isfinite(got).all()
    if d == 64:
        want = oracle.fmha(q.numpy(), k.numpy(), v.numpy(), scale=scale, causal=causal, threads=0)
        err = rel_err(got.cpu().numpy(), want)
        assert err <= TF32_TOL, err
    else:
        want = oracle.fmha(q.bfloat16().float().numpy(), k.bfloat16().float().numpy(), v.bfloat16().float().numpy(),
                           scale=scale, causal=causal, threads=0)
        assert rel_err(got.cpu().numpy(), want) <= BF16_TOL
        pre = ops.fmha(q.bfloat16().to(cuda_device), k.bfloat16().to(cuda_device), v.bfloat16().to(cuda_device),
                       scale=scale, causal=causal, out_dtype=torch.float32)
        assert torch.equal(got, pre)
    assert ops.last_device_status() == 0


def test_reference_graph_no_scale_no_mask(cuda_device):
    """scale = 1, causal = off: exactly BatchedMatmul -> Softmax -> BatchedMatmul of the reference."""
    from kernelcodegen_b200 import ops

    q, k, v = normal((1, 2, 256, 64), 4) * 0.5, normal((1, 2, 256, 64), 5) * 0.5, normal((1, 2, 256, 64), 6)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    s = oracle.batched_matmul(q.float().numpy(), k.float().numpy(), b_col_major=True)
    want = oracle.batched_matmul(oracle.softmax(s), v.float().numpy())
    got = ops.fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), out_dtype=torch.float32)
    assert rel_err(got.cpu().numpy(), want) <= BF16_TOL


def test_config_fp32_b4_h16_s1024_d64(cuda_device):
    """fp32 in / fp32 out, N(0,1), seeds 20/21/22, scale 1/8, non-causal.
    Oracle on 8 of the 64 (batch, head) pairs; properties on the whole tensor."""
    from kernelcodegen_b200 import ops

    q, k, v = normal((4, 16, 1024, 64), 20), normal((4, 16, 1024, 64), 21), normal((4, 16, 1024, 64), 22)
    got = ops.fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=0.125)
    assert got.dtype == torch.float32
    pick = [0, 9, 18, 27, 36, 45, 54, 63]
    # head dimension 64 with fp32 inputs runs both contractions as TF32 products of the fp32
    # tiles: compared with the oracle on the un-rounded inputs, at the TF32 bar
    want32 = oracle.fmha(*(t.reshape(64, 1024, 64)[pick].numpy() for t in (q, k, v)), scale=0.125, threads=0)
    err = rel_err(got.reshape(64, 1024, 64)[pick].cpu().numpy(), want32)
    assert err <= TF32_TOL, err
    assert ops.last_device_status() == 0


def test_config_bf16_causal_b8_h32_s8192_d128(cuda_device):
    """The long-sequence config at full size; fp64 oracle on sampled (pair, row)s, plus
    size-independent properties."""
    from kernelcodegen_b200 import ops

    B, H, S, D = 8, 32, 8192, 128
    g = torch.Generator(device=cuda_device)
    tensors = []
    for seed in (30, 31, 32):
        g.manual_seed(seed)
        tensors.append(torch.randn((B, H, S, D), generator=g, device=cuda_device).bfloat16())
    q, k, v = tensors
    scale = D ** -0.5
    o = ops.fmha(q, k, v, scale=scale, causal=True)
    assert ops.last_device_status() == 0
    rows = np.array([0, 1, 127, 128, 129, 4095, 4096, 8063, 8064, 8191], dtype=np.int64)
    for bh in (0, 97, 255):
        b, h = divmod(bh, H)
        qn, kn, vn = (t[b, h].float().cpu().numpy()[None] for t in (q, k, v))
        want = oracle.fmha_rows_f64(qn, kn, vn, 0, rows, scale=scale, causal=True)
        got = o[b, h][torch.from_numpy(rows).to(cuda_device)].float().cpu().numpy()
        assert rel_err(got, want) <= BF16_TOL
    # causal: the first query only sees the first key
    assert torch.equal(o[:, :, 0, :], v[:, :, 0, :])
    # rows of P sum to one: with V = 1 the output is 1 (bf16 rounding of P aside)
    ones = torch.ones_like(v)
    o1 = ops.fmha(q, k, ones, scale=scale, causal=True, out_dtype=torch.float32)
    assert (o1 - 1).abs().max().item() <= 1e-2


def test_key_permutation_invariance(cuda_device):
    """Without a mask the result does not depend on the order of the keys."""
    from kernelcodegen_b200 import ops

    q, k, v = (normal((2, 4, 512, 128), s).bfloat16().to(cuda_device) for s in (7, 8, 9))
    perm = torch.randperm(512, generator=torch.Generator().manual_seed(1)).to(cuda_device)
    a = ops.fmha(q, k, v, scale=0.1, out_dtype=torch.float32)
    b = ops.fmha(q, k[:, :, perm].contiguous(), v[:, :, perm].contiguous(), scale=0.1, out_dtype=torch.float32)
    assert rel_err(a.cpu().numpy(), b.cpu().numpy()) <= 1e-2


def test_queries_without_visible_keys_give_zero(cuda_device):
    from kernelcodegen_b200 import ops

    q, k, v = normal((1, 1, 256, 64), 1).bfloat16(), normal((1, 1, 128, 64), 2).bfloat16(), normal((1, 1, 128, 64), 3).bfloat16()
    got = ops.fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=0.125, causal=True,
                   out_dtype=torch.float32)
    want = oracle.fmha(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale=0.125, causal=True)
    assert (got[0, 0, :128] == 0).all()
    assert rel_err(got.cpu().numpy(), want) <= BF16_TOL


def test_host_buffer_entry_point(cuda_device):
    import ctypes

    from kernelcodegen_b200 import capi

    lib = capi.load()
    q, k, v = (normal((1, 2, 128, 64), s).numpy() for s in (1, 2, 3))
    o = np.empty_like(q)
    d = capi.FmhaDesc()
    d.B, d.H, d.Sq, d.Skv, d.D = 1, 2, 128, 128, 64
    d.dtype_in = d.dtype_out = capi.KCG_F32
    d.scale = 0.125
    st = lib.kcg_fmha_fwd_host(ctypes.byref(d), q.ctypes.data, k.ctypes.data, v.ctypes.data, o.ctypes.data)
    assert st == capi.KCG_OK, capi.status_str(st)
    assert rel_err(o, oracle.fmha(q, k, v, scale=0.125)) <= BF16_TOL


def test_error_statuses(cuda_device):
    from kernelcodegen_b200 import capi, ops

    z = torch.zeros((1, 1, 128, 96), device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(capi.KcgError) as ei:
        ops.fmha(z, z, z)
    assert ei.value.status == capi.KCG_BAD_SHAPE
    z = torch.zeros((1, 1, 128, 64), device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(capi.KcgError) as ei:
        ops.fmha(z, z, z, scale=-1.0)
    assert ei.value.status == capi.KCG_BAD_ARGUMENT


@pytest.mark.parametrize("growth", [0.05, 0.6, 3.0])
def test_row_maximum_that_keeps_growing(cuda_device, growth):
    """Logits that increase along the key axis make the running row maximum move in every key
    block: slowly (below the lazy-rescale threshold, so O is never rescaled), moderately, and
    fast (rescale in every block).  All three must agree with the oracle."""
    from kernelcodegen_b200 import ops

    b, h, s, d = 1, 2, 1024, 64
    q = torch.ones((b, h, s, d)) * 0.25 + normal((b, h, s, d), 11) * 0.05
    ramp = torch.linspace(0.0, growth * (s / 128), s)[None, None, :, None]        # per-key offset
    k = normal((b, h, s, d), 12) * 0.05 + ramp / (0.25 * d)                         # q.k grows by `growth` per block
    v = normal((b, h, s, d), 13)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    for causal in (False, True):
        want = oracle.fmha(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale=1.0, causal=causal, threads=0)
        got = ops.fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=1.0, causal=causal,
                       out_dtype=torch.float32)
        assert torch.isfinite(got).all()
        assert rel_err(got.cpu().numpy(), want) <= BF16_TOL
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("spread", [4.0, 40.0, 400.0])
def test_wide_logit_spread_head_dimension_64(cuda_device, spread):
    """bf16, head dimension 64: a fixed share of the exponentials is taken from a cubic on the FMA
    pipe, which clamps its argument at -125 (2^-125 instead of an underflow to 0).  Scores that
    lie up to `spread` (natural-log units) below the row maximum, far tails included, must agree
    with the oracle, row sums and all; masked keys must contribute nothing."""
    from kernelcodegen_b200 import ops

    b, h, s, d = 1, 2, 512, 64
    q = torch.zeros((b, h, s, d))
    q[..., 0] = 1.0
    k = normal((b, h, s, d), 31) * 0.01
    k[..., 0] = -torch.rand((b, h, s), generator=torch.Generator().manual_seed(32)) * spread   # the score itself
    k[:, :, ::37, 0] = 0.0                                                                      # a few keys at the maximum
    v = normal((b, h, s, d), 33)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    for causal in (False, True):
        want = oracle.fmha(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale=1.0, causal=causal, threads=0)
        got = ops.fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=1.0, causal=causal,
                       out_dtype=torch.float32)
        assert torch.isfinite(got).all()
        assert rel_err(got.cpu().numpy(), want) <= BF16_TOL
    assert ops.last_device_status() == 0
