/*
 * CPU oracle -- TEST INFRASTRUCTURE ONLY.  Not part of the product path: only tests/,
 * __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may load this.
 *
 * A plain-C restatement of the loop nests the reference's Frontend builds
 * (yao-jiashu/KernelCodeGen, src/Frontend/Operators.cc).  The reference never executes these
 * nests on a CPU itself (it has no CPU lowering and its numeric harness is absent), and it
 * ships no golden vectors or known-answer tests for them: PARITY UNPINNED by the reference's
 * own tests.  What pins this file instead: the operator definitions cited at each function,
 * and an independent numpy float64 evaluation of the same formulas (tests/golden/).
 *
 * Build with  gcc -O2 -ffp-contract=off -fno-fast-math  so that every `a*b + acc` is a
 * separately rounded fp32 multiply and add, as the arith.mulf / arith.addf pair in the nest.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* Matmul::build, src/Frontend/Operators.cc:140-173:
 *   for i < m, j < n { acc = 0; for k < K: acc = A[i,k]*B[k,j] + acc; C[i,j] = acc } */
void oracle_matmul_f32(const float* A, const float* B, float* C, int64_t m, int64_t n, int64_t k,
                       int64_t lda, int64_t ldb, int64_t ldc) {
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int64_t kk = 0; kk < k; ++kk) {
        float mul = A[i * lda + kk] * B[kk * ldb + j];
        acc = mul + acc;
      }
      C[i * ldc + j] = acc;
    }
  }
}

/* Same nest restricted to the rows listed in `rows` (C_rows is [nrows, n] compact): used to
 * check very large products on a sample of rows. Row results are independent of each other
 * in the nest, so each sampled row equals the corresponding row of the full result. */
void oracle_matmul_rows_f32(const float* A, const float* B, float* C_rows, const int64_t* rows,
                            int64_t nrows, int64_t n, int64_t k, int64_t lda, int64_t ldb) {
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t i = rows[r];
    for (int64_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int64_t kk = 0; kk < k; ++kk) {
        float mul = A[i * lda + kk] * B[kk * ldb + j];
        acc = mul + acc;
      }
      C_rows[r * n + j] = acc;
    }
  }
}

/* The same nest with rows distributed over host threads (bit-identical to the sequential
 * form: rows do not interact).  Used only to time the CPU baseline with all cores.
 * The k loop is kept innermost and sequential, as in the reference nest. */
void oracle_matmul_f32_mt(const float* A, const float* B, float* C, int64_t m, int64_t n,
                          int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#pragma omp parallel for schedule(static) collapse(2)
#endif
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int64_t kk = 0; kk < k; ++kk) {
        float mul = A[i * lda + kk] * B[kk * ldb + j];
        acc = mul + acc;
      }
      C[i * ldc + j] = acc;
    }
  }
  (void)threads;
}

/* float64-accumulated product of float inputs: the arbiter for the bf16 paths
 * ("fp32-accumulated reference" of bf16-rounded inputs; fp64 bounds it from above). */
void oracle_matmul_rows_f64(const float* A, const float* B, double* C_rows, const int64_t* rows,
                            int64_t nrows, int64_t n, int64_t k, int64_t lda, int64_t ldb) {
  double* acc = (double*)malloc((size_t)n * sizeof(double));
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t i = rows[r];
    memset(acc, 0, (size_t)n * sizeof(double));
    for (int64_t kk = 0; kk < k; ++kk) {
      const double a = A[i * lda + kk];
      const float* brow = B + kk * ldb;
      for (int64_t j = 0; j < n; ++j) acc[j] += a * (double)brow[j];
    }
    memcpy(C_rows + r * n, acc, (size_t)n * sizeof(double));
  }
  free(acc);
}

/* Relu::build, src/Frontend/Operators.cc:232-244: out[idx] = arith.maxf(0, in[idx]),
 * in place when the memory space is `inplace` (:221-227). */
void oracle_relu_f32(float* x, int64_t count) {
  for (int64_t i = 0; i < count; ++i) {
    float v = x[i];
    x[i] = (v != v) ? v : (v > 0.0f ? v : 0.0f); /* maxf propagates NaN */
  }
}

/* BatchedMatmul::build, src/Frontend/Operators.cc:353-414.  A is [batch, m, k] row-major;
 * B is [batch, k, n] (b_col_major = 0) or [batch, n, k] (Layout::colMajor, :394-398). */
void oracle_batched_matmul_f32(const float* A, const float* B, float* C, int64_t batch, int64_t m,
                               int64_t n, int64_t k, int b_col_major) {
  for (int64_t b = 0; b < batch; ++b) {
    const float* a = A + b * m * k;
    const float* bb = B + b * k * n;
    float* c = C + b * m * n;
    for (int64_t i = 0; i < m; ++i) {
      for (int64_t j = 0; j < n; ++j) {
        float acc = 0.0f;
        for (int64_t kk = 0; kk < k; ++kk) {
          float bv = b_col_major ? bb[j * k + kk] : bb[kk * n + j];
          float mul = a[i * k + kk] * bv;
          acc = mul + acc;
        }
        c[i * n + j] = acc;
      }
    }
  }
}

/* Softmax::build, src/Frontend/Operators.cc:474-536, last axis, in place:
 *   sum = 0; for k: sum = exp(x[k]) + sum;  for k: x[k] = exp(x[k]) / sum.
 * No max subtraction, no scale, no mask (as in the reference). */
void oracle_softmax_f32(float* x, int64_t rows, int64_t cols) {
  for (int64_t r = 0; r < rows; ++r) {
    float* row = x + r * cols;
    float sum = 0.0f;
    for (int64_t c = 0; c < cols; ++c) sum = expf(row[c]) + sum;
    for (int64_t c = 0; c < cols; ++c) row[c] = expf(row[c]) / sum;
  }
}

/* FMHA = the three-operator graph of test/test.cc:88-90 evaluated per (batch, head):
 *   S = Q . K^T  (BatchedMatmul, K colMajor);  P = Softmax(S) in place;  O = P . V.
 * `scale` and `causal` are explicit extensions (scale = 1, causal = 0 is the reference):
 * the logits are multiplied by `scale` before exp, and with `causal` query i only sees keys
 * j <= i + (skv - sq) (the others drop out of both the sum and P.V).
 * The score matrix is formed one query row at a time, so nothing of size sq*skv is stored.
 * `bh_count` (batch*heads) pairs, tensors [bh, s, d] contiguous. */
void oracle_fmha_f32(const float* Q, const float* K, const float* V, float* O, int64_t bh_count,
                     int64_t sq, int64_t skv, int64_t d, float scale, int causal, int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
#endif
  for (int64_t bh = 0; bh < bh_count; ++bh) {
    for (int64_t i = 0; i < sq; ++i) {
      const float* q = Q + (bh * sq + i) * d;
      const float* kbase = K + bh * skv * d;
      const float* vbase = V + bh * skv * d;
      float* o = O + (bh * sq + i) * d;
      float* s = (float*)malloc((size_t)skv * sizeof(float));
      const int64_t jmax = causal ? (i + (skv - sq) + 1) : skv;
      const int64_t jn = jmax < 0 ? 0 : (jmax > skv ? skv : jmax);
      for (int64_t j = 0; j < jn; ++j) {
        float acc = 0.0f;
        for (int64_t kk = 0; kk < d; ++kk) {
          float mul = q[kk] * kbase[j * d + kk];
          acc = mul + acc;
        }
        s[j] = acc * scale;
      }
      float sum = 0.0f;
      for (int64_t j = 0; j < jn; ++j) sum = expf(s[j]) + sum;
      for (int64_t j = 0; j < jn; ++j) s[j] = expf(s[j]) / sum;
      for (int64_t c = 0; c < d; ++c) {
        float acc = 0.0f;
        for (int64_t j = 0; j < jn; ++j) {
          float mul = s[j] * vbase[j * d + c];
          acc = mul + acc;
        }
        o[c] = acc;
      }
      free(s);
    }
  }
  (void)threads;
}

/* float64 evaluation of the same formula with max subtraction (mathematically identical,
 * immune to overflow): the arbiter for bf16 attention and for long rows.  Evaluates only the
 * query rows listed in `rows` of the (batch*head) pair `bh`; O_rows is [nrows, d]. */
void oracle_fmha_rows_f64(const float* Q, const float* K, const float* V, double* O_rows,
                          int64_t bh, const int64_t* rows, int64_t nrows, int64_t sq, int64_t skv,
                          int64_t d, double scale, int causal) {
  double* s = (double*)malloc((size_t)skv * sizeof(double));
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t i = rows[r];
    const float* q = Q + (bh * sq + i) * d;
    const float* kbase = K + bh * skv * d;
    const float* vbase = V + bh * skv * d;
    const int64_t jmax = causal ? (i + (skv - sq) + 1) : skv;
    const int64_t jn = jmax < 0 ? 0 : (jmax > skv ? skv : jmax);
    double mx = -INFINITY;
    for (int64_t j = 0; j < jn; ++j) {
      double acc = 0.0;
      for (int64_t kk = 0; kk < d; ++kk) acc += (double)q[kk] * (double)kbase[j * d + kk];
      s[j] = acc * scale;
      if (s[j] > mx) mx = s[j];
    }
    double sum = 0.0;
    for (int64_t j = 0; j < jn; ++j) {
      s[j] = exp(s[j] - mx);
      sum += s[j];
    }
    for (int64_t c = 0; c < d; ++c) {
      double acc = 0.0;
      for (int64_t j = 0; j < jn; ++j) acc += s[j] * (double)vbase[j * d + c];
      O_rows[r * d + c] = jn > 0 ? acc / sum : NAN;
    }
  }
  free(s);
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
