// Host-buffer GEMM with the PCIe copies overlapped with the tensor-core work.
//
// The reference's harness around a generated kernel is "cudaMalloc, copy A and B in, launch, copy
// C out" (performance/output.log:6-13), one after the other.  On a B200 the 32768^3 bf16 product
// takes ~55 ms on the tensor cores and its 6 GiB of operands ~110 ms on PCIe Gen5, so the copies,
// not the kernel, set the end-to-end time.  Here A is cut into row chunks and B into column
// chunks, copied alternately (A0, B0, A1, B1, ...).  When row chunk k of A has landed the kernel
// runs on it against the column chunks 0..k-1 that are already there; when column chunk k of B has
// landed the kernel runs on it against row chunks 0..k.  Every C tile is computed once, as early
// as its operands allow, and only 1/chunks of the work is left when the last copy ends.  Finished
// strips of C go back to the host on a third stream, in the other PCIe direction.  Three streams,
// ordered by events only; nothing blocks the host.  With B already on the device (hB == nullptr: a
// caller that fetched B some other way, e.g. 1/N of it over PCIe and the rest from its peers over
// NVLink) only the row chunks of A and the strips of C move.
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace kcg {

namespace {

constexpr int MAX_CHUNKS = 16;

// Streams and events of one device, made on first use and kept for the life of the process.
struct PipeCtx {
  bool ready = false;
  cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
  cudaEvent_t begin = nullptr, out_done = nullptr;
  cudaEvent_t in_done[2 * MAX_CHUNKS] = {}, c_done[2 * MAX_CHUNKS] = {};  // [2k] row chunk k, [2k+1] column chunk k
};

kcg_status_t pipe_ctx(PipeCtx** out) {
  static std::mutex mu;
  static PipeCtx ctx[64];
  int dev = 0;
  KCG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return KCG_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  PipeCtx& c = ctx[dev];
  if (!c.ready) {
    KCG_CUDA_TRY(cudaStreamCreateWithFlags(&c.h2d, cudaStreamNonBlocking));
    KCG_CUDA_TRY(cudaStreamCreateWithFlags(&c.compute, cudaStreamNonBlocking));
    KCG_CUDA_TRY(cudaStreamCreateWithFlags(&c.d2h, cudaStreamNonBlocking));
    KCG_CUDA_TRY(cudaEventCreateWithFlags(&c.begin, cudaEventDisableTiming));
    KCG_CUDA_TRY(cudaEventCreateWithFlags(&c.out_done, cudaEventDisableTiming));
    for (int i = 0; i < 2 * MAX_CHUNKS; ++i) {
      KCG_CUDA_TRY(cudaEventCreateWithFlags(&c.in_done[i], cudaEventDisableTiming));
      KCG_CUDA_TRY(cudaEventCreateWithFlags(&c.c_done[i], cudaEventDisableTiming));
    }
    c.ready = true;
  }
  *out = &c;
  return KCG_OK;
}

inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

// rows x cols elements of `es` bytes, leading dimension `ld` elements, between host and device
inline cudaError_t copy_block(void* dst, const void* src, long long ld, long long row0, long long col0,
                              long long rows, long long cols, size_t es, cudaMemcpyKind kind, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  const size_t off = (static_cast<size_t>(row0) * ld + col0) * es;
  return cudaMemcpy2DAsync(static_cast<uint8_t*>(dst) + off, static_cast<size_t>(ld) * es,
                           static_cast<const uint8_t*>(src) + off, static_cast<size_t>(ld) * es,
                           static_cast<size_t>(cols) * es, static_cast<size_t>(rows), kind, s);
}

}  // namespace

kcg_status_t gemm_host_staged_impl(const kcg_gemm_desc* d, const void* hA, const void* hB, void* hC, void* dA,
                                   void* dB, void* dC, void* ws, size_t ws_bytes, int chunks,
                                   cudaStream_t stream) {
  if (!d || !hA || !hC || !dA || !dB || !dC) return KCG_BAD_ARGUMENT;
  const bool b_resident = hB == nullptr;   // B is already in dB (put there by the caller, e.g. gathered from peers)
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return KCG_BAD_SHAPE;
  if (chunks < 0 || chunks > MAX_CHUNKS) return KCG_BAD_ARGUMENT;
  if (d->n_peers < 0 || d->n_peers > 8) return KCG_BAD_ARGUMENT;
  if (d->dtype_in != KCG_BF16 && d->dtype_in != KCG_F32) return KCG_UNSUPPORTED;
  if (d->dtype_out != KCG_BF16 && d->dtype_out != KCG_F32) return KCG_UNSUPPORTED;
  const size_t es = d->dtype_in == KCG_BF16 ? 2 : 4;
  const size_t os = d->dtype_out == KCG_BF16 ? 2 : 4;
  const bool bk = d->b_layout == KCG_COL_MAJOR;
  if (d->lda < d->K || d->ldc < d->N || d->ldb < (bk ? d->K : d->N)) return KCG_BAD_SHAPE;
  const long long M = d->M, N = d->N, K = d->K;

  // chunks of about 2048 rows / columns, at most 16 per dimension; one chunk (no overlap) for
  // products too small to hide a copy behind
  const int nr_want = chunks ? chunks : static_cast<int>(std::max<long long>(1, std::min<long long>(MAX_CHUNKS, M / 2048)));
  const int nc_want = b_resident ? 1 : (chunks ? chunks : static_cast<int>(std::max<long long>(1, std::min<long long>(MAX_CHUNKS, N / 2048))));
  const long long rh = round_up((M + nr_want - 1) / nr_want, 256);  // rows of A per chunk (tile aligned)
  const long long cw = round_up((N + nc_want - 1) / nc_want, 256);  // columns of B per chunk
  const int nr = static_cast<int>((M + rh - 1) / rh), nc = static_cast<int>((N + cw - 1) / cw);
  const int steps = std::max(nr, nc);

  const double work = 2.0 * static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K);
  const bool long_job = work >= 4e12;

  PipeCtx* cx = nullptr;
  kcg_status_t st = pipe_ctx(&cx);
  if (st != KCG_OK) return st;
  // one call at a time queues its work on the shared streams
  static std::mutex enqueue_mu;
  std::lock_guard<std::mutex> enqueue_lock(enqueue_mu);
  // everything below starts after what the caller already queued on `stream`
  KCG_CUDA_TRY(cudaEventRecord(cx->begin, stream));
  KCG_CUDA_TRY(cudaStreamWaitEvent(cx->h2d, cx->begin, 0));
  KCG_CUDA_TRY(cudaStreamWaitEvent(cx->compute, cx->begin, 0));
  KCG_CUDA_TRY(cudaStreamWaitEvent(cx->d2h, cx->begin, 0));

  auto strip = [&](long long r0, long long r1, long long c0, long long c1) -> kcg_status_t {
    if (r1 <= r0 || c1 <= c0) return KCG_OK;
    kcg_gemm_desc s = *d;
    s.M = r1 - r0;
    s.N = c1 - c0;
    // the parts of one long product run back to back: keep the choices made for long launches
    if (s.cta_group == 0 && long_job) s.cta_group = 1;
    if (s.tile_n == 0 && long_job) s.tile_n = 256;
    const uint8_t* a = static_cast<const uint8_t*>(dA) + static_cast<size_t>(r0) * d->lda * es;
    const uint8_t* b = static_cast<const uint8_t*>(dB) +
                       (bk ? static_cast<size_t>(c0) * d->ldb : static_cast<size_t>(c0)) * es;
    const size_t c_off = (static_cast<size_t>(r0) * d->ldc + c0) * os;
    for (int i = 0; i < d->n_peers; ++i) s.peer_c[i] = static_cast<uint8_t*>(d->peer_c[i]) + c_off;
    return gemm_launch_impl(&s, a, b, static_cast<uint8_t*>(dC) + c_off, ws, ws_bytes, cx->compute);
  };

  // a failure part-way falls through to the join below
#define PIPE_TRY(expr)                       \
  if ((expr) != cudaSuccess) {               \
    cudaGetLastError();                      \
    st = KCG_CUDA_ERROR;                     \
    break;                                   \
  }
  for (int k = 0; k < steps; ++k) {
    const long long r0 = std::min(M, k * rh), r1 = std::min(M, (k + 1) * rh);  // row chunk k
    const long long c0 = std::min(N, k * cw), c1 = std::min(N, (k + 1) * cw);  // column chunk k
    // row chunk k of A, then the kernel on it against the columns that arrived before (chunks 0..k-1)
    const long long c_lo = std::min(N, std::min(k, nc) * cw);
    PIPE_TRY(copy_block(dA, hA, d->lda, r0, 0, r1 - r0, K, es, cudaMemcpyHostToDevice, cx->h2d));
    PIPE_TRY(cudaEventRecord(cx->in_done[2 * k], cx->h2d));
    PIPE_TRY(cudaStreamWaitEvent(cx->compute, cx->in_done[2 * k], 0));
    st = strip(r0, r1, 0, c_lo);
    if (st != KCG_OK) break;
    PIPE_TRY(cudaEventRecord(cx->c_done[2 * k], cx->compute));
    PIPE_TRY(cudaStreamWaitEvent(cx->d2h, cx->c_done[2 * k], 0));
    PIPE_TRY(copy_block(hC, dC, d->ldc, r0, 0, r1 - r0, c_lo, os, cudaMemcpyDeviceToHost, cx->d2h));
    // column chunk k of B (B stored [N, K]: a block of rows of the array), then the kernel on it
    // against every row that has arrived (chunks 0..k)
    const long long r_hi = std::min(M, (std::min(k, nr - 1) + 1) * rh);
    const long long b_r0 = bk ? c0 : 0, b_c0 = bk ? 0 : c0;
    const long long b_rows = bk ? c1 - c0 : K, b_cols = bk ? K : c1 - c0;
    if (!b_resident)
      { PIPE_TRY(copy_block(dB, hB, d->ldb, b_r0, b_c0, b_rows, b_cols, es, cudaMemcpyHostToDevice, cx->h2d)); }
    PIPE_TRY(cudaEventRecord(cx->in_done[2 * k + 1], cx->h2d));
    PIPE_TRY(cudaStreamWaitEvent(cx->compute, cx->in_done[2 * k + 1], 0));
    st = strip(0, r_hi, c0, c1);
    if (st != KCG_OK) break;
    PIPE_TRY(cudaEventRecord(cx->c_done[2 * k + 1], cx->compute));
    PIPE_TRY(cudaStreamWaitEvent(cx->d2h, cx->c_done[2 * k + 1], 0));
    PIPE_TRY(copy_block(hC, dC, d->ldc, 0, c0, r_hi, c1 - c0, os, cudaMemcpyDeviceToHost, cx->d2h));
  }
#undef PIPE_TRY
  // the caller's stream continues once the last strip is back on the host (which implies that
  // every copy in and every launch has completed)
  KCG_CUDA_TRY(cudaEventRecord(cx->out_done, cx->d2h));
  KCG_CUDA_TRY(cudaStreamWaitEvent(stream, cx->out_done, 0));
  if (st != KCG_OK) {  // rare: drain what was queued, so that no buffer is still in use
    cudaStreamSynchronize(cx->h2d);
    cudaStreamSynchronize(cx->compute);
    cudaStreamSynchronize(cx->d2h);
  }
  return st;
}

}  // namespace kcg
