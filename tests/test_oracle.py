"""CPU tests of the oracle (oracle/oracle.c) against the committed golden vectors and against
properties of the operator definitions.  No GPU, no product code."""
import numpy as np
import pytest

from oracle import oracle


def test_matmul_matches_golden(golden):
    c = oracle.matmul(golden["mm_a"], golden["mm_b"])
    np.testing.assert_allclose(c, golden["mm_c"], rtol=0, atol=2e-5)
    r = oracle.matmul_relu(golden["mm_a"], golden["mm_b"])
    np.testing.assert_allclose(r, golden["mm_relu"], rtol=0, atol=2e-5)
    assert (r >= 0).all()


def test_matmul_is_sequential_fp32_sum():
    # The nest accumulates k in ascending order with separate fp32 roundings:
    # reproduce it literally in numpy float32 for a tiny case and demand bit equality.
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (5, 19)).astype(np.float32)
    b = rng.uniform(-1, 1, (19, 4)).astype(np.float32)
    want = np.zeros((5, 4), dtype=np.float32)
    for i in range(5):
        for j in range(4):
            acc = np.float32(0)
            for k in range(19):
                acc = np.float32(np.float32(a[i, k] * b[k, j]) + acc)
            want[i, j] = acc
    assert np.array_equal(oracle.matmul(a, b), want)


def test_threads_and_row_sampling_are_bit_identical():
    rng = np.random.default_rng(2)
    a = rng.uniform(-1, 1, (33, 70)).astype(np.float32)
    b = rng.uniform(-1, 1, (70, 21)).astype(np.float32)
    c = oracle.matmul(a, b)
    assert np.array_equal(oracle.matmul(a, b, threads=3), c)
    rows = [0, 7, 32]
    assert np.array_equal(oracle.matmul_rows(a, b, rows), c[rows])
    np.testing.assert_allclose(oracle.matmul_rows(a, b, rows, f64=True), c[rows], atol=2e-5)


def test_relu_edge_values():
    x = np.array([-1.5, -0.0, 0.0, 2.0, np.inf, -np.inf], dtype=np.float32)
    y = oracle.relu(x)
    assert np.array_equal(y, np.array([0, 0, 0, 2, np.inf, 0], dtype=np.float32))
    assert np.isnan(oracle.relu(np.array([np.nan], dtype=np.float32))[0])


def test_batched_matmul_col_major_matches_golden(golden):
    c = oracle.batched_matmul(golden["bmm_a"], golden["bmm_b"], b_col_major=True)
    np.testing.assert_allclose(c, golden["bmm_nt"], atol=1e-5)
    # rowMajor B = the transposed tensor
    bt = np.ascontiguousarray(np.swapaxes(golden["bmm_b"], -1, -2))
    assert np.array_equal(oracle.batched_matmul(golden["bmm_a"], bt, b_col_major=False), c)


def test_softmax_matches_golden_and_sums_to_one(golden):
    y = oracle.softmax(golden["sm_x"])
    np.testing.assert_allclose(y, golden["sm_y"], rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(y.sum(-1), 1.0, atol=1e-5)


def test_fmha_is_the_three_operator_graph(golden):
    q, k, v = golden["fa_q"], golden["fa_k"], golden["fa_v"]
    s = oracle.batched_matmul(q, k, b_col_major=True)
    p = oracle.softmax(s)
    o_graph = oracle.batched_matmul(p, v)
    o = oracle.fmha(q, k, v)  # scale 1, no mask: the reference graph
    assert np.array_equal(o, o_graph)
    np.testing.assert_allclose(o, golden["fa_o_ref"], atol=2e-5)


def test_fmha_extensions_match_golden(golden):
    q, k, v = golden["fa_q"], golden["fa_k"], golden["fa_v"]
    o = oracle.fmha(q, k, v, scale=0.25, causal=True, threads=2)
    np.testing.assert_allclose(o, golden["fa_o_scaled_causal"], atol=2e-5)
    rows = [0, 1, 39]
    o64 = oracle.fmha_rows_f64(q, k, v, 3, rows, scale=0.25, causal=True)
    np.testing.assert_allclose(o64, golden["fa_o_scaled_causal"].reshape(4, 40, 16)[3][rows], atol=1e-12)


def test_fmha_causal_first_row_is_first_value_when_square():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 1, 9, 8)).astype(np.float32)
    k = rng.standard_normal((1, 1, 9, 8)).astype(np.float32)
    v = rng.standard_normal((1, 1, 9, 8)).astype(np.float32)
    o = oracle.fmha(q, k, v, causal=True)
    np.testing.assert_allclose(o[0, 0, 0], v[0, 0, 0], rtol=1e-6)


def test_fmha_rows_without_visible_keys_are_zero():
    # Sq > Skv with a causal mask: the first Sq-Skv queries see no key at all.
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 1, 6, 8)).astype(np.float32)
    k = rng.standard_normal((1, 1, 4, 8)).astype(np.float32)
    v = rng.standard_normal((1, 1, 4, 8)).astype(np.float32)
    o = oracle.fmha(q, k, v, causal=True)
    assert np.array_equal(o[0, 0, :2], np.zeros((2, 8), dtype=np.float32))
    assert np.isfinite(o).all()


def test_transpose_swaps_the_last_two_axes():
    x = np.arange(2 * 3 * 5, dtype=np.float32).reshape(2, 3, 5)
    y = oracle.transpose(x)
    assert y.shape == (2, 5, 3) and y.flags["C_CONTIGUOUS"]
    for b in range(2):
        for i in range(3):
            for j in range(5):
                assert y[b, j, i] == x[b, i, j]
