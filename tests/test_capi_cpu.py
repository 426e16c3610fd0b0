"""CPU checks of the C-ABI library: it loads without a GPU, exports every symbol the header
declares, and its argument validation answers before any device work."""
import ctypes
import re
from pathlib import Path

import pytest

from kernelcodegen_b200 import capi

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "kcg_capi.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kcg_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native_lib):
    names = declared_functions()
    assert "kcg_gemm_launch" in names and "kcg_fmha_fwd_launch" in names
    for name in names:
        assert hasattr(native_lib, name), f"{name} declared in kcg_capi.h but not exported"
    assert set(capi.EXPORTED_SYMBOLS) <= set(names)


def test_struct_layouts_match_header(tmp_path):
    """sizeof / offsetof of every descriptor field as a C compiler lays out include/kcg_capi.h,
    against the ctypes mirrors the Python callers use."""
    import subprocess

    lines = []
    for cname, cls in (("kcg_gemm_desc", capi.GemmDesc), ("kcg_fmha_desc", capi.FmhaDesc)):
        lines.append(f'printf("%zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'printf("%zu\\n", offsetof({cname}, {fname}));')
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "kcg_capi.h"\nint main(void) {\n'
                   + "\n".join(lines) + "\nreturn 0; }\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = []
    for cls in (capi.GemmDesc, capi.FmhaDesc):
        want.append(ctypes.sizeof(cls))
        want += [getattr(cls, fname).offset for fname, _ in cls._fields_]
    assert got == want


def test_status_strings(native_lib):
    assert capi.status_str(capi.KCG_OK) == "KCG_OK"
    assert capi.status_str(capi.KCG_DEVICE_TIMEOUT) == "KCG_DEVICE_TIMEOUT"
    assert capi.status_str(12345) == "KCG_UNKNOWN"
    assert b"sm_100a" in native_lib.kcg_version()


def _gemm_desc(m=256, n=256, k=256, prec=capi.KCG_PREC_3XTF32, dt=capi.KCG_F32):
    d = capi.GemmDesc()
    d.M, d.N, d.K = m, n, k
    d.lda, d.ldb, d.ldc = k, n, n
    d.dtype_in = d.dtype_out = dt
    d.precision = prec
    return d


def test_workspace_sizes(native_lib):
    d = _gemm_desc()
    assert native_lib.kcg_gemm_workspace_bytes(ctypes.byref(d)) == 2 * 256 * 256 * 4
    d = _gemm_desc(prec=capi.KCG_PREC_BF16, dt=capi.KCG_BF16)
    assert native_lib.kcg_gemm_workspace_bytes(ctypes.byref(d)) == 0
    # shared-K tail: 4096x2048x1024 fp32 makes 256 pair tiles of 256x128 = 3 waves of 74 pairs + 34
    d = _gemm_desc(4096, 2048, 1024)
    assert native_lib.kcg_gemm_shared_k_tiles(ctypes.byref(d)) == 34
    lo = 4 * (4096 * 1024 + 1024 * 2048)
    assert native_lib.kcg_gemm_workspace_bytes(ctypes.byref(d)) == lo + 34 * 8 * 2 * 32 * 128 * 4
    d.cta_group = 1                       # single CTAs: no tail sharing, residual arrays only
    assert native_lib.kcg_gemm_shared_k_tiles(ctypes.byref(d)) == 0
    assert native_lib.kcg_gemm_workspace_bytes(ctypes.byref(d)) == lo
    d = _gemm_desc(1024, 1024, 1024)      # 32 pair tiles on 74 pairs: all of them share K
    assert native_lib.kcg_gemm_shared_k_tiles(ctypes.byref(d)) == 32
    d = _gemm_desc(32768, 32768, 32768, prec=capi.KCG_PREC_BF16, dt=capi.KCG_BF16)   # long launch: single CTAs
    assert native_lib.kcg_gemm_shared_k_tiles(ctypes.byref(d)) == 0
    assert native_lib.kcg_gemm_workspace_bytes(ctypes.byref(d)) == 0
    d = _gemm_desc(4096, 4096, 4096, prec=capi.KCG_PREC_BF16, dt=capi.KCG_BF16)      # 256 tiles of 256x256
    assert native_lib.kcg_gemm_shared_k_tiles(ctypes.byref(d)) == 34
    f = capi.FmhaDesc()
    f.B, f.H, f.Sq, f.Skv, f.D = 2, 3, 128, 256, 128
    f.dtype_in = capi.KCG_F32          # head dimension 128: bf16 copies of Q, K, V in the workspace
    assert native_lib.kcg_fmha_workspace_bytes(ctypes.byref(f)) == 2 * 3 * 128 * 2 * (128 + 2 * 256)
    f.D = 64                           # head dimension 64: TF32 contractions on the fp32 tiles, no scratch
    assert native_lib.kcg_fmha_workspace_bytes(ctypes.byref(f)) == 0
    f.D = 128
    f.dtype_in = capi.KCG_BF16
    assert native_lib.kcg_fmha_workspace_bytes(ctypes.byref(f)) == 0


@pytest.mark.parametrize("mutate,want", [
    (lambda d: setattr(d, "M", 0), capi.KCG_BAD_SHAPE),
    (lambda d: setattr(d, "lda", 8), capi.KCG_BAD_SHAPE),
    (lambda d: setattr(d, "precision", 7), capi.KCG_UNSUPPORTED),
    (lambda d: setattr(d, "dtype_in", capi.KCG_BF16), capi.KCG_UNSUPPORTED),
    (lambda d: setattr(d, "epilogue", 5), capi.KCG_UNSUPPORTED),
    (lambda d: setattr(d, "tile_n", 192), capi.KCG_UNSUPPORTED),
    (lambda d: setattr(d, "ldc", 258), capi.KCG_BAD_ALIGN),
    (lambda d: setattr(d, "n_peers", 9), capi.KCG_BAD_ARGUMENT),
])
def test_gemm_argument_validation_needs_no_gpu(native_lib, mutate, want):
    d = _gemm_desc()
    mutate(d)
    fake = 0x10000  # never dereferenced: validation fails first
    st = native_lib.kcg_gemm_launch(ctypes.byref(d), fake, fake, fake, fake, 1 << 30, None)
    assert st == want, capi.status_str(st)


def test_gemm_null_and_misaligned_pointers(native_lib):
    d = _gemm_desc()
    assert native_lib.kcg_gemm_launch(None, 16, 16, 16, None, 0, None) == capi.KCG_BAD_ARGUMENT
    assert native_lib.kcg_gemm_launch(ctypes.byref(d), None, 16, 16, None, 0, None) == capi.KCG_BAD_ARGUMENT
    assert native_lib.kcg_gemm_launch(ctypes.byref(d), 0x10004, 0x10000, 0x10000, None, 0, None) == capi.KCG_BAD_ALIGN
    # 3xTF32 needs its scratch
    assert native_lib.kcg_gemm_launch(ctypes.byref(d), 0x10000, 0x10000, 0x10000, None, 0, None) == capi.KCG_BAD_WORKSPACE
    assert native_lib.kcg_gemm_launch(ctypes.byref(d), 0x10000, 0x10000, 0x10000, 0x20000, 16, None) == capi.KCG_BAD_WORKSPACE


def test_fmha_argument_validation_needs_no_gpu(native_lib):
    f = capi.FmhaDesc()
    f.B, f.H, f.Sq, f.Skv, f.D = 1, 1, 128, 128, 64
    f.dtype_in = f.dtype_out = capi.KCG_BF16
    f.scale = 1.0
    fake = 0x10000
    call = lambda: native_lib.kcg_fmha_fwd_launch(ctypes.byref(f), fake, fake, fake, fake, None, 0, None)
    f.D = 96
    assert call() == capi.KCG_BAD_SHAPE
    f.D = 64
    f.Skv = 0
    assert call() == capi.KCG_BAD_SHAPE
    f.Skv = 128
    f.scale = 0.0
    assert call() == capi.KCG_BAD_ARGUMENT
    f.scale = 1.0
    f.dtype_in = 3
    assert call() == capi.KCG_UNSUPPORTED
    f.dtype_in = capi.KCG_F32  # f32 inputs with head dimension 128 need scratch for their bf16 copies
    f.D = 128
    assert call() == capi.KCG_BAD_WORKSPACE
    assert native_lib.kcg_fmha_fwd_launch(None, fake, fake, fake, fake, None, 0, None) == capi.KCG_BAD_ARGUMENT


def test_ops_refuse_cpu_tensors(native_lib):
    import torch

    from kernelcodegen_b200 import ops

    a = torch.zeros(128, 128)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.matmul(a, a)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.fmha(torch.zeros(1, 1, 128, 64), torch.zeros(1, 1, 128, 64), torch.zeros(1, 1, 128, 64))


def test_product_package_does_not_touch_the_oracle():
    pkg = ROOT / "kernelcodegen_b200"
    for path in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")):
        text = path.read_text()
        assert "oracle" not in text.lower(), f"{path} mentions the oracle"


def test_shared_k_plan_covers_every_k_block_once(native_lib):
    """Walks the plan the way the kernel's work iterator does (range u = positions [u*share,
    (u+1)*share) of the tail tiles laid end to end, `span` positions per tile, positions past
    num_kb are padding) and checks that every k-block of every tail tile is covered exactly once,
    that no range is longer than a tile, and that no tile has more contributors than announced."""
    out = (ctypes.c_int32 * 5)()
    planned = 0
    for pairs in (74, 66, 9):
        for num_kb in (8, 9, 15, 16, 31, 32, 33, 64, 100, 512):
            for tiles in range(1, 3 * pairs + 1):
                for i in range(5):
                    out[i] = 0
                native_lib.kcg_gemm_shared_k_plan(tiles, num_kb, pairs, 128, out)
                tail, units, share, span, maxc = list(out)
                if tail == 0:
                    continue
                planned += 1
                assert tail == tiles % pairs and 0 < units <= pairs and span >= num_kb and share <= num_kb
                cover = [[0] * num_kb for _ in range(tail)]
                contrib = [set() for _ in range(tail)]
                for u in range(units):
                    lin0, lin1 = min(tail * span, u * share), min(tail * span, (u + 1) * share)
                    while lin0 < lin1:
                        ti, off = divmod(lin0, span)
                        end = min(span, off + (lin1 - lin0))
                        lin0 += end - off
                        if off < num_kb:
                            for kb in range(off, min(num_kb, end)):
                                cover[ti][kb] += 1
                            contrib[ti].add(u)
                assert all(c == 1 for row in cover for c in row), (tiles, num_kb, pairs)
                for ti in range(tail):
                    first = (ti * span) // share
                    last = min(units - 1, (ti * span + num_kb - 1) // share)
                    assert contrib[ti] == set(range(first, last + 1))      # what the epilogue counts on
                    assert len(contrib[ti]) <= maxc
    assert planned > 100


def test_launch_geometry_follows_the_variant_choice(native_lib):
    """The geometry the generated launcher text quotes: CTA pairs with 256x128 tiles for the
    short fp32 launch, single 320-thread CTAs with 128x256 tiles for the long bf16 one; one CTA
    per 256 queries and (batch, head) for attention."""
    out = (ctypes.c_int32 * 6)()
    d = _gemm_desc(4096, 2048, 1024)
    assert native_lib.kcg_gemm_launch_geometry(ctypes.byref(d), out) == capi.KCG_OK
    assert list(out) == [148, 192, 2, 256, 128, 256]
    d = _gemm_desc(32768, 32768, 32768, prec=capi.KCG_PREC_BF16, dt=capi.KCG_BF16)
    assert native_lib.kcg_gemm_launch_geometry(ctypes.byref(d), out) == capi.KCG_OK
    assert list(out) == [148, 320, 1, 128, 256, 256 * 128]
    d = _gemm_desc(128, 128, 128)           # one tile
    assert native_lib.kcg_gemm_launch_geometry(ctypes.byref(d), out) == capi.KCG_OK
    assert list(out)[:5] == [1, 320, 1, 128, 128]
    f = capi.FmhaDesc()
    f.B, f.H, f.Sq, f.Skv, f.D = 8, 32, 8192, 8192, 128
    out4 = (ctypes.c_int32 * 4)()
    assert native_lib.kcg_fmha_launch_geometry(ctypes.byref(f), out4) == capi.KCG_OK
    assert list(out4) == [32 * 256, 384, 256, 128]
