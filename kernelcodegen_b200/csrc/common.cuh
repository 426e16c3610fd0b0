// Host-side helpers shared by the launchers: status plumbing, device properties, tensor-map
// encoding through the driver entry point (so the library links against cudart only and can
// be loaded on a machine without a driver, where every launch then reports an error).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstdint>
#include <cstdio>

#include "../../include/kcg_capi.h"

namespace kcg {

extern std::atomic<uint64_t> g_launches;
extern std::atomic<uint32_t> g_spin_limit;

// Address of the per-device status word (a __device__ int owned by capi.cu).
kcg_status_t device_status_ptr(int** out);
int device_sm_count();
// Bounds-checking build (KCG_DEBUG_BOUNDS): address of the two-word detail record on the current
// device, and the test hook that caps the extents the kernels check against (0 = no cap).  In the
// normal build the pointer stays null and the cap is 0.
kcg_status_t debug_bounds_detail_ptr(unsigned long long** out);
unsigned long long debug_extent_limit();

// dims/strides innermost first, strides in bytes for dims 1..rank-1.
kcg_status_t encode_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base,
                         const uint64_t* dims, const uint64_t* strides_bytes,
                         const uint32_t* box,
                         CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define KCG_CUDA_TRY(expr)                                                        \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      std::fprintf(stderr, "kcg: %s failed: %s\n", #expr, cudaGetErrorString(_e)); \
      return KCG_CUDA_ERROR;                                                      \
    }                                                                             \
  } while (0)

kcg_status_t gemm_launch_impl(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                              void* ws, size_t ws_bytes, cudaStream_t stream);
size_t gemm_workspace_impl(const kcg_gemm_desc* d);
size_t gemm_batched_workspace_impl(const kcg_gemm_desc* d, long long batch, long long stride_a, long long stride_b);
kcg_status_t gemm_batched_launch_impl(const kcg_gemm_desc* d, long long batch, long long stride_a, long long stride_b,
                                      long long stride_c, const void* A, const void* B, void* C, void* ws,
                                      size_t ws_bytes, cudaStream_t stream);
kcg_status_t gemm_launch_geometry_impl(const kcg_gemm_desc* d, int* out);
kcg_status_t fmha_launch_geometry_impl(const kcg_fmha_desc* d, int* out);
int gemm_shared_k_tiles_impl(const kcg_gemm_desc* d);
void gemm_reset_shared_k_counters();
void gemm_shared_k_plan_impl(int tiles, int num_kb, int pairs, int bn, int* out);
kcg_status_t transpose_launch_impl(int64_t batch, int64_t rows, int64_t cols, int dtype, const void* x, void* y,
                                   cudaStream_t stream);
kcg_status_t gemm_launch_static_impl(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                                     cudaStream_t stream);
kcg_status_t gemm_host_staged_impl(const kcg_gemm_desc* d, const void* hA, const void* hB, void* hC, void* dA,
                                   void* dB, void* dC, void* ws, size_t ws_bytes, int chunks,
                                   cudaStream_t stream);
kcg_status_t fmha_launch_impl(const kcg_fmha_desc* d, const void* Q, const void* K, const void* V,
                              void* O, void* ws, size_t ws_bytes, cudaStream_t stream);
size_t fmha_workspace_impl(const kcg_fmha_desc* d);
kcg_status_t softmax_launch_impl(long long rows, long long cols, const void* x, void* y, cudaStream_t stream);

}  // namespace kcg
