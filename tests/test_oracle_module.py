"""The module the Frontend builds, executed on the CPU, against the hand-written CPU nest.

`oracle/module_lower.cc` lowers the loop nests `Matmul / Relu / BatchedMatmul / Softmax /
Transpose::build` emit (the product's own graph builder) to scalar LLVM IR and
`oracle/module_jit.py` JIT-compiles them: the reference's missing "affine module lowered to CPU"
(include/Optimizer/Rewriter.h:221, body commented out at src/Optimizer/Rewriter.cc:1605-1612).
`oracle/oracle.c` states the same operator definitions by hand.  Two independently derived
executions of src/Frontend/Operators.cc:140-173, 232-244, 353-414, 474-536 must agree bit for
bit; neither is pinned by a vector of the reference's own (it holds none)."""
import numpy as np
import pytest

from oracle import oracle

module_jit = pytest.importorskip("oracle.module_jit")
pytest.importorskip("llvmlite")


@pytest.fixture(scope="module")
def rng():
    return np.random.default_rng(11)


def _u(rng, shape):
    return rng.uniform(-1, 1, shape).astype(np.float32)


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (37, 29, 53), (64, 96, 128)])
def test_matmul_and_fused_relu(rng, m, n, k):
    a, b = _u(rng, (m, k)), _u(rng, (k, n))
    got = module_jit.LoweredModule("matmul", (m, n, k)).run(a, b)
    assert np.array_equal(got, oracle.matmul(a, b))
    fused = module_jit.LoweredModule("matmul_relu", (m, n, k))
    want = oracle.matmul_relu(a, b)
    assert np.array_equal(fused.run(a, b), want)
    assert np.array_equal(fused.run(a, b, threads=3), want)      # rows over host threads: same bits
    if m > 1:
        assert (want == 0).any() and (want > 0).any()


def test_relu_keeps_nan_and_negative_zero(rng):
    x = _u(rng, (5, 9))
    x[0, 0], x[1, 1], x[2, 2] = np.nan, -0.0, -np.inf
    got = module_jit.LoweredModule("relu", (5, 9)).run(x)
    want = oracle.relu(x)
    assert np.array_equal(got, want, equal_nan=True)
    assert np.isnan(got[0, 0]) and got[2, 2] == 0


@pytest.mark.parametrize("nt", [False, True])
def test_batched_matmul_both_layouts(rng, nt):
    a = _u(rng, (2, 3, 20, 16))
    b = _u(rng, (2, 3, 24, 16) if nt else (2, 3, 16, 24))
    mod = module_jit.LoweredModule("batched_matmul_nt" if nt else "batched_matmul_nn", (2, 3, 20, 24, 16))
    assert np.array_equal(mod.run(a, b), oracle.batched_matmul(a, b, b_col_major=nt))


def test_softmax_in_place_without_max_subtraction(rng):
    x = (rng.normal(size=(5, 7, 33)) * 3).astype(np.float32)
    got = module_jit.LoweredModule("softmax", (5, 7, 33)).run(x)
    assert np.array_equal(got, oracle.softmax(x))
    np.testing.assert_allclose(got.sum(-1), 1.0, atol=1e-5)


def test_three_operator_attention_graph(rng):
    """BatchedMatmul(Q, K colMajor) -> Softmax -> BatchedMatmul(P, V), test/test.cc:88-90."""
    q = (rng.normal(size=(2, 2, 48, 16)) * 0.5).astype(np.float32)
    k = (rng.normal(size=(2, 2, 40, 16)) * 0.5).astype(np.float32)
    v = rng.normal(size=(2, 2, 40, 16)).astype(np.float32)
    mod = module_jit.LoweredModule("attention", (2, 2, 48, 40, 16))
    assert [c[0].split("_")[0] for c in mod.calls] == ["BatchMatmul", "Softmax", "BatchMatmul"]
    assert np.array_equal(mod.run(q, k, v), oracle.fmha(q, k, v))


def test_transpose(rng):
    x = _u(rng, (3, 5, 7))
    mod = module_jit.LoweredModule("transpose", (3, 5, 7))
    assert np.array_equal(mod.run(x), oracle.transpose(x))
    assert np.array_equal(mod.run(x, threads=2), oracle.transpose(x))


def test_golden_vectors(golden):
    """The committed float64-derived fixtures, through the lowered module."""
    a, b = golden["mm_a"], golden["mm_b"]
    m, k = a.shape
    n = b.shape[1]
    got = module_jit.LoweredModule("matmul", (m, n, k)).run(a, b)
    assert np.abs(got - golden["mm_c"]).max() / np.abs(golden["mm_c"]).max() <= 1e-6


def test_lowered_code_has_no_fast_math_and_is_scalar():
    text = module_jit.lower("matmul", (8, 8, 8))
    ir = text.split(";;;IR\n", 1)[1]
    assert "fmul float" in ir and "fadd float" in ir
    for flag in ("fast", "contract", "reassoc", "fmuladd", "llvm.fma"):
        assert flag not in ir
    assert "phi float" in ir            # the k loop's carried accumulator


def test_scheduled_modules_and_bad_graphs_are_refused():
    with pytest.raises(RuntimeError, match="unknown graph"):
        module_jit.lower("conv2d", (1, 2, 3))
    with pytest.raises(RuntimeError, match="m n k"):
        module_jit.lower("matmul", (4, 4))
