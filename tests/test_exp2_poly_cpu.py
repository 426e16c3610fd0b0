"""The cubic the FMHA kernel uses for a share of its exponentials (ex2_poly2 in
kernelcodegen_b200/csrc/ptx.cuh), restated in numpy float32 operation by operation: the error bound
the kernel's comment states, and the behaviour at the clamp, hold for these coefficients."""
import re
from pathlib import Path

import numpy as np

PTX = Path(__file__).resolve().parents[1] / "kernelcodegen_b200" / "csrc" / "ptx.cuh"


def coefficients():
    text = PTX.read_text()
    body = text[text.index("float2 ex2_poly2(float2 x)"):]
    body = body[:body.index("return r;")]
    c = [float(v) for v in re.findall(r"make_float2\((0\.\d+)f,", body)]
    assert len(c) == 4, c
    return c   # c3, c2, c1, c0 in Horner order


def ex2_poly(x):
    c3, c2, c1, c0 = (np.float32(v) for v in coefficients())
    x = np.asarray(x, dtype=np.float32)
    magic = np.float32(12582912.0)
    t = (x + magic).astype(np.float32)
    n = (t - magic).astype(np.float32)
    f = (x - n).astype(np.float32)
    p = (f * c3 + c2).astype(np.float32)
    p = (p * f + c1).astype(np.float32)
    p = (p * f + c0).astype(np.float32)
    bits = p.view(np.uint32) + (t.view(np.uint32) << np.uint32(23))
    return bits.view(np.float32)


def test_relative_error_below_bf16_and_tf32_rounding():
    x = np.linspace(-125.0, 8.0, 400001, dtype=np.float32)
    got = ex2_poly(x).astype(np.float64)
    want = np.exp2(x.astype(np.float64))
    rel = np.abs(got / want - 1.0)
    assert rel.max() < 1.0e-4          # bf16 rounds at 3.9e-3, TF32 at 4.9e-4


def test_clamped_argument_gives_a_tiny_normal_number():
    got = ex2_poly(np.array([-125.0], dtype=np.float32))[0]
    assert 0.0 < got < 1e-37 and np.isfinite(got)
