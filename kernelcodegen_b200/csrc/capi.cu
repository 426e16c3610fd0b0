// extern "C" surface of the library (declared in include/kcg_capi.h) plus the host-side
// plumbing the launchers share.
#include <cstring>
#include <functional>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace kcg {

std::atomic<uint64_t> g_launches{0};
std::atomic<uint32_t> g_spin_limit{0};

// One status word per device (a __device__ variable is instantiated on every device that
// loads the module).  Kernels receive its address as a parameter.
__device__ int g_device_status;

kcg_status_t device_status_ptr(int** out) {
  static std::mutex mu;
  static int* cache[64] = {};
  int dev = 0;
  KCG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return KCG_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    KCG_CUDA_TRY(cudaGetSymbolAddress(&p, g_device_status));
    KCG_CUDA_TRY(cudaMemset(p, 0, sizeof(int)));
    cache[dev] = static_cast<int*>(p);
  }
  *out = cache[dev];
  return KCG_OK;
}

// Detail record of the bounds-checking build: {offending byte offset, extent it was checked against}.
__device__ unsigned long long g_bounds_detail[2];
std::atomic<unsigned long long> g_extent_limit{0};

kcg_status_t debug_bounds_detail_ptr(unsigned long long** out) {
#ifdef KCG_DEBUG_BOUNDS
  static std::mutex mu;
  static unsigned long long* cache[64] = {};
  int dev = 0;
  KCG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return KCG_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    KCG_CUDA_TRY(cudaGetSymbolAddress(&p, g_bounds_detail));
    KCG_CUDA_TRY(cudaMemset(p, 0, sizeof(unsigned long long) * 2));
    cache[dev] = static_cast<unsigned long long*>(p);
  }
  *out = cache[dev];
#else
  *out = nullptr;
#endif
  return KCG_OK;
}

unsigned long long debug_extent_limit() {
#ifdef KCG_DEBUG_BOUNDS
  return g_extent_limit.load();
#else
  return 0;
#endif
}

int device_sm_count() {
  static int cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (!cache[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 1;
    cache[dev] = n;
  }
  return cache[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

kcg_status_t encode_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base,
                         const uint64_t* dims, const uint64_t* strides_bytes,
                         const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    std::fprintf(stderr, "kcg: cuTensorMapEncodeTiled not available (no CUDA driver?)\n");
    return KCG_CUDA_ERROR;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
  CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides,
                  gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::fprintf(stderr, "kcg: cuTensorMapEncodeTiled failed with CUresult %d\n",
                 static_cast<int>(r));
    return KCG_CUDA_ERROR;
  }
  return KCG_OK;
}

// One thread waits on an mbarrier that nothing ever arrives on: exercises the bounded wait the
// kernels use (iteration cap -> status word -> clean return) without involving any other unit.
__global__ void selftest_wait_kernel(int* status, uint32_t limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
    mbar_wait(smem_u32(&bar), 0, &abort_flag, status, DEV_TIMEOUT_EPILOGUE, limit);
  }
}

// Host-buffer helper: device buffer that frees itself.
struct DevBuf {
  void* p = nullptr;
  ~DevBuf() {
    if (p) cudaFree(p);
  }
  cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 1); }
};

}  // namespace kcg

using namespace kcg;

extern "C" {

size_t kcg_gemm_workspace_bytes(const kcg_gemm_desc* d) { return gemm_workspace_impl(d); }
size_t kcg_fmha_workspace_bytes(const kcg_fmha_desc* d) { return fmha_workspace_impl(d); }
int kcg_gemm_shared_k_tiles(const kcg_gemm_desc* d) { return gemm_shared_k_tiles_impl(d); }
kcg_status_t kcg_gemm_launch_geometry(const kcg_gemm_desc* d, int32_t* out6) { return gemm_launch_geometry_impl(d, out6); }
kcg_status_t kcg_fmha_launch_geometry(const kcg_fmha_desc* d, int32_t* out4) { return fmha_launch_geometry_impl(d, out4); }
void kcg_gemm_shared_k_plan(int32_t tiles, int32_t num_kb, int32_t pairs, int32_t tile_n, int32_t* out5) {
  if (out5 && tiles > 0 && num_kb > 0 && pairs > 0) gemm_shared_k_plan_impl(tiles, num_kb, pairs, tile_n, out5);
}

kcg_status_t kcg_gemm_launch(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                             void* workspace, size_t workspace_bytes, void* stream) {
  return gemm_launch_impl(d, A, B, C, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream));
}

kcg_status_t kcg_gemm_launch_static(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                                    void* stream) {
  return gemm_launch_static_impl(d, A, B, C, static_cast<cudaStream_t>(stream));
}

kcg_status_t kcg_softmax_launch(int64_t rows, int64_t cols, const void* x, void* y, void* stream) {
  return softmax_launch_impl(rows, cols, x, y, static_cast<cudaStream_t>(stream));
}

kcg_status_t kcg_transpose_launch(int64_t batch, int64_t rows, int64_t cols, int32_t dtype, const void* x, void* y,
                                  void* stream) {
  return transpose_launch_impl(batch, rows, cols, dtype, x, y, static_cast<cudaStream_t>(stream));
}

kcg_status_t kcg_batched_gemm_launch(const kcg_gemm_desc* d, int64_t batch, int64_t stride_a, int64_t stride_b,
                                     int64_t stride_c, const void* A, const void* B, void* C, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  return gemm_batched_launch_impl(d, batch, stride_a, stride_b, stride_c, A, B, C, workspace, workspace_bytes,
                                  static_cast<cudaStream_t>(stream));
}

size_t kcg_batched_gemm_workspace_bytes(const kcg_gemm_desc* d, int64_t batch, int64_t stride_a, int64_t stride_b) {
  return gemm_batched_workspace_impl(d, batch, stride_a, stride_b);
}

kcg_status_t kcg_fmha_fwd_launch(const kcg_fmha_desc* d, const void* Q, const void* K,
                                 const void* V, void* O, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  return fmha_launch_impl(d, Q, K, V, O, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream));
}

kcg_status_t kcg_gemm_host(const kcg_gemm_desc* d, const void* hA, const void* hB, void* hC) {
  if (!d || !hA || !hB || !hC) return KCG_BAD_ARGUMENT;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return KCG_BAD_SHAPE;
  if (d->n_peers != 0) return KCG_UNSUPPORTED;
  const size_t es = d->dtype_in == KCG_BF16 ? 2 : 4;
  const size_t os = d->dtype_out == KCG_BF16 ? 2 : 4;
  const bool bk = d->b_layout == KCG_COL_MAJOR;
  if (d->lda < d->K || d->ldc < d->N || d->ldb < (bk ? d->K : d->N)) return KCG_BAD_SHAPE;
  const size_t a_bytes = static_cast<size_t>(d->M) * d->lda * es;
  const size_t b_bytes = static_cast<size_t>(bk ? d->N : d->K) * d->ldb * es;
  const size_t c_bytes = static_cast<size_t>(d->M) * d->ldc * os;
  const size_t ws_bytes = gemm_workspace_impl(d);
  DevBuf a, b, c, ws;
  KCG_CUDA_TRY(a.alloc(a_bytes));
  KCG_CUDA_TRY(b.alloc(b_bytes));
  KCG_CUDA_TRY(c.alloc(c_bytes));
  KCG_CUDA_TRY(ws.alloc(ws_bytes));
  kcg_status_t st = gemm_host_staged_impl(d, hA, hB, hC, a.p, b.p, c.p, ws.p, ws_bytes, 0, nullptr);
  if (st != KCG_OK) {
    cudaDeviceSynchronize();  // nothing may still use the buffers when they are freed
    return st;
  }
  KCG_CUDA_TRY(cudaStreamSynchronize(nullptr));
  return kcg_last_device_status() ? KCG_DEVICE_TIMEOUT : KCG_OK;
}

kcg_status_t kcg_gemm_host_staged(const kcg_gemm_desc* d, const void* hA, const void* hB, void* hC, void* dA,
                                  void* dB, void* dC, void* workspace, size_t workspace_bytes, int chunks,
                                  void* stream) {
  return gemm_host_staged_impl(d, hA, hB, hC, dA, dB, dC, workspace, workspace_bytes, chunks,
                               static_cast<cudaStream_t>(stream));
}

kcg_status_t kcg_fmha_fwd_host(const kcg_fmha_desc* d, const void* hQ, const void* hK,
                               const void* hV, void* hO) {
  if (!d || !hQ || !hK || !hV || !hO) return KCG_BAD_ARGUMENT;
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Skv <= 0 || d->D <= 0) return KCG_BAD_SHAPE;
  const size_t es = d->dtype_in == KCG_BF16 ? 2 : 4;
  const size_t os = d->dtype_out == KCG_BF16 ? 2 : 4;
  const size_t bh = static_cast<size_t>(d->B) * d->H;
  const size_t q_bytes = bh * d->Sq * d->D * es;
  const size_t kv_bytes = bh * d->Skv * d->D * es;
  const size_t o_bytes = bh * d->Sq * d->D * os;
  const size_t ws_bytes = fmha_workspace_impl(d);
  DevBuf q, k, v, o, ws;
  KCG_CUDA_TRY(q.alloc(q_bytes));
  KCG_CUDA_TRY(k.alloc(kv_bytes));
  KCG_CUDA_TRY(v.alloc(kv_bytes));
  KCG_CUDA_TRY(o.alloc(o_bytes));
  KCG_CUDA_TRY(ws.alloc(ws_bytes));
  KCG_CUDA_TRY(cudaMemcpy(q.p, hQ, q_bytes, cudaMemcpyHostToDevice));
  KCG_CUDA_TRY(cudaMemcpy(k.p, hK, kv_bytes, cudaMemcpyHostToDevice));
  KCG_CUDA_TRY(cudaMemcpy(v.p, hV, kv_bytes, cudaMemcpyHostToDevice));
  kcg_status_t st = fmha_launch_impl(d, q.p, k.p, v.p, o.p, ws.p, ws_bytes, nullptr);
  if (st != KCG_OK) return st;
  KCG_CUDA_TRY(cudaMemcpy(hO, o.p, o_bytes, cudaMemcpyDeviceToHost));
  return kcg_last_device_status() ? KCG_DEVICE_TIMEOUT : KCG_OK;
}

int kcg_last_device_status(void) {
  int* p = nullptr;
  if (device_status_ptr(&p) != KCG_OK) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) {
    cudaMemset(p, 0, sizeof(int));
    // a kernel that gave up may have left arrival counters of the shared-K tail half counted
    gemm_reset_shared_k_counters();
  }
  return v;
}

// ---- peer-visible buffers (fused all-gather) ---------------------------------------------------
kcg_status_t kcg_peer_alloc(size_t bytes, void** out_ptr, void* out_handle64) {
  if (!out_ptr || !out_handle64 || bytes == 0) return KCG_BAD_ARGUMENT;
  void* p = nullptr;
  KCG_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "kcg: cudaIpcGetMemHandle failed: %s\n", cudaGetErrorString(e));
    cudaFree(p);
    return KCG_CUDA_ERROR;
  }
  static_assert(sizeof(h) == 64, "IPC handle is 64 bytes");
  std::memcpy(out_handle64, &h, 64);
  *out_ptr = p;
  return KCG_OK;
}

kcg_status_t kcg_peer_open(const void* handle64, void** out_ptr) {
  if (!handle64 || !out_ptr) return KCG_BAD_ARGUMENT;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  KCG_CUDA_TRY(cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return KCG_OK;
}

kcg_status_t kcg_peer_close(void* ptr) {
  if (!ptr) return KCG_BAD_ARGUMENT;
  KCG_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return KCG_OK;
}

kcg_status_t kcg_peer_free(void* ptr) {
  if (!ptr) return KCG_BAD_ARGUMENT;
  KCG_CUDA_TRY(cudaFree(ptr));
  return KCG_OK;
}

// ---- completion flags --------------------------------------------------------------------------
// One thread per flag polls with acquire loads at system scope until the flag has reached
// `value`; bounded, see kcg_peer_wait_launch.
__global__ void peer_wait_kernel(const uint32_t* flags, int n, int stride_words, uint32_t value, uint32_t max_polls,
                                 int* status) {
  const int i = threadIdx.x;
  if (i >= n) return;
  const uint32_t* f = flags + static_cast<size_t>(i) * stride_words;
  for (uint32_t it = 0; it < max_polls; ++it) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(f) - value) >= 0) return;
    __nanosleep(200);
  }
  atomicCAS(status, 0, static_cast<int>(DEV_TIMEOUT_PEER));
}

kcg_status_t kcg_peer_wait_launch(const void* flags, int32_t n, int32_t stride_words, uint32_t value,
                                  uint32_t max_polls, void* stream) {
  if (!flags || n <= 0 || n > 32 || stride_words <= 0) return KCG_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(flags) & 3u) return KCG_BAD_ALIGN;
  int* status = nullptr;
  kcg_status_t st = device_status_ptr(&status);
  if (st != KCG_OK) return st;
  const uint32_t polls = max_polls ? max_polls : (1u << 22);   // x (200 ns sleep + a load) ~ 1-2 s
  peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(flags), n,
                                                                    stride_words, value, polls, status);
  g_launches.fetch_add(1);
  KCG_CUDA_TRY(cudaGetLastError());
  return KCG_OK;
}

kcg_status_t kcg_peer_wait_status(void) {
  const int v = kcg_last_device_status();
  if (v < 0) return KCG_CUDA_ERROR;
  if (v == 0) return KCG_OK;
  return v == static_cast<int>(DEV_TIMEOUT_PEER) ? KCG_PEER_TIMEOUT : KCG_DEVICE_TIMEOUT;
}

// ---- timing helpers (the cost function of the operator API's configuration search) -------------
static kcg_status_t time_launches(const std::function<kcg_status_t()>& launch, int iters, float* ms) {
  cudaEvent_t e0, e1;
  KCG_CUDA_TRY(cudaEventCreate(&e0));
  KCG_CUDA_TRY(cudaEventCreate(&e1));
  kcg_status_t st = KCG_OK;
  for (int i = 0; i < 2 && st == KCG_OK; ++i) st = launch();
  if (st == KCG_OK) {
    cudaEventRecord(e0, nullptr);
    for (int i = 0; i < iters && st == KCG_OK; ++i) st = launch();
    cudaEventRecord(e1, nullptr);
    if (cudaEventSynchronize(e1) != cudaSuccess) st = KCG_CUDA_ERROR;
    float t = 0.f;
    if (st == KCG_OK && cudaEventElapsedTime(&t, e0, e1) == cudaSuccess) *ms = t / iters;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (st == KCG_OK && kcg_last_device_status() != 0) st = KCG_DEVICE_TIMEOUT;
  return st;
}

kcg_status_t kcg_gemm_time(const kcg_gemm_desc* d, int iters, float* ms_per_launch) {
  if (!d || !ms_per_launch || iters <= 0) return KCG_BAD_ARGUMENT;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return KCG_BAD_SHAPE;
  if (d->n_peers != 0) return KCG_UNSUPPORTED;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return KCG_CUDA_ERROR;
  const size_t es = d->dtype_in == KCG_BF16 ? 2 : 4, os = d->dtype_out == KCG_BF16 ? 2 : 4;
  const bool bk = d->b_layout == KCG_COL_MAJOR;
  const size_t ws_bytes = gemm_workspace_impl(d);
  DevBuf a, b, c, ws;
  KCG_CUDA_TRY(a.alloc(static_cast<size_t>(d->M) * d->lda * es));
  KCG_CUDA_TRY(b.alloc(static_cast<size_t>(bk ? d->N : d->K) * d->ldb * es));
  KCG_CUDA_TRY(c.alloc(static_cast<size_t>(d->M) * d->ldc * os));
  KCG_CUDA_TRY(ws.alloc(ws_bytes));
  KCG_CUDA_TRY(cudaMemset(a.p, 0, static_cast<size_t>(d->M) * d->lda * es));
  KCG_CUDA_TRY(cudaMemset(b.p, 0, static_cast<size_t>(bk ? d->N : d->K) * d->ldb * es));
  return time_launches([&] { return gemm_launch_impl(d, a.p, b.p, c.p, ws.p, ws_bytes, nullptr); }, iters,
                       ms_per_launch);
}

kcg_status_t kcg_fmha_time(const kcg_fmha_desc* d, int iters, float* ms_per_launch) {
  if (!d || !ms_per_launch || iters <= 0) return KCG_BAD_ARGUMENT;
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Skv <= 0 || d->D <= 0) return KCG_BAD_SHAPE;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return KCG_CUDA_ERROR;
  const size_t es = d->dtype_in == KCG_BF16 ? 2 : 4, os = d->dtype_out == KCG_BF16 ? 2 : 4;
  const size_t bh = static_cast<size_t>(d->B) * d->H;
  const size_t ws_bytes = fmha_workspace_impl(d);
  DevBuf q, k, v, o, ws;
  KCG_CUDA_TRY(q.alloc(bh * d->Sq * d->D * es));
  KCG_CUDA_TRY(k.alloc(bh * d->Skv * d->D * es));
  KCG_CUDA_TRY(v.alloc(bh * d->Skv * d->D * es));
  KCG_CUDA_TRY(o.alloc(bh * d->Sq * d->D * os));
  KCG_CUDA_TRY(ws.alloc(ws_bytes));
  KCG_CUDA_TRY(cudaMemset(q.p, 0, bh * d->Sq * d->D * es));
  KCG_CUDA_TRY(cudaMemset(k.p, 0, bh * d->Skv * d->D * es));
  KCG_CUDA_TRY(cudaMemset(v.p, 0, bh * d->Skv * d->D * es));
  return time_launches([&] { return fmha_launch_impl(d, q.p, k.p, v.p, o.p, ws.p, ws_bytes, nullptr); }, iters,
                       ms_per_launch);
}

kcg_status_t kcg_selftest_wait_timeout(uint32_t iterations) {
  int* status = nullptr;
  kcg_status_t st = device_status_ptr(&status);
  if (st != KCG_OK) return st;
  if (iterations == 0 || iterations > (1u << 20)) return KCG_BAD_ARGUMENT;
  selftest_wait_kernel<<<1, 32>>>(status, iterations);
  g_launches.fetch_add(1);
  KCG_CUDA_TRY(cudaGetLastError());
  const int v = kcg_last_device_status();
  if (v < 0) return KCG_CUDA_ERROR;
  return v == 0 ? KCG_OK : KCG_DEVICE_TIMEOUT;
}

void kcg_set_spin_limit(uint32_t iterations) { g_spin_limit.store(iterations); }

int kcg_debug_bounds_enabled(void) {
#ifdef KCG_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}

void kcg_debug_set_extent_limit(uint64_t bytes) { g_extent_limit.store(bytes); }

kcg_status_t kcg_debug_bounds_detail(uint64_t* out2) {
  if (!out2) return KCG_BAD_ARGUMENT;
  out2[0] = out2[1] = 0;
  unsigned long long* p = nullptr;
  kcg_status_t st = debug_bounds_detail_ptr(&p);
  if (st != KCG_OK || !p) return st;
  unsigned long long v[2] = {0, 0};
  KCG_CUDA_TRY(cudaMemcpy(v, p, sizeof(v), cudaMemcpyDeviceToHost));
  out2[0] = v[0];
  out2[1] = v[1];
  return KCG_OK;
}

uint64_t kcg_launch_count(void) { return g_launches.load(); }

const char* kcg_status_str(kcg_status_t s) {
  switch (s) {
    case KCG_OK: return "KCG_OK";
    case KCG_BAD_SHAPE: return "KCG_BAD_SHAPE";
    case KCG_BAD_ALIGN: return "KCG_BAD_ALIGN";
    case KCG_UNSUPPORTED: return "KCG_UNSUPPORTED";
    case KCG_CUDA_ERROR: return "KCG_CUDA_ERROR";
    case KCG_DEVICE_TIMEOUT: return "KCG_DEVICE_TIMEOUT";
    case KCG_PEER_TIMEOUT: return "KCG_PEER_TIMEOUT";
    case KCG_BAD_WORKSPACE: return "KCG_BAD_WORKSPACE";
    case KCG_BAD_ARGUMENT: return "KCG_BAD_ARGUMENT";
    case KCG_TOO_LARGE: return "KCG_TOO_LARGE";
  }
  return "KCG_UNKNOWN";
}

const char* kcg_version(void) { return "kcg-b200 0.1 (sm_100a)"; }

}  // extern "C"
