// Y[b, j, i] = X[b, i, j]: the Transpose operator the reference declares
// (include/Frontend/Operators.h:100-102) and leaves without a body
// (src/Frontend/Operators.cc:422-423).
//
// HBM-bound: every element is read once and written once.  A CTA moves one 64 x 64 tile through
// shared memory: rows of X are read with 4-element vector loads (16 threads cover a 64-element
// row segment), the tile is stored transposed-readable ([64][65] words, the odd pitch spreads a
// column over the banks), and rows of Y are written with 4-element vector stores.  Tiles on a
// ragged edge, and shapes whose rows or columns are not multiples of 4, take an element-wise
// path of the same structure.
#include "common.cuh"

namespace kcg {

namespace {

constexpr int TT = 64;           // tile edge
constexpr int TR_THREADS = 256;

template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  using type = float4;
};
template <>
struct Vec4<uint16_t> {
  using type = uint2;            // four 16-bit elements
};

template <typename T>
__device__ __forceinline__ void unpack4(const typename Vec4<T>::type& v, T* e);
template <>
__device__ __forceinline__ void unpack4<float>(const float4& v, float* e) {
  e[0] = v.x;
  e[1] = v.y;
  e[2] = v.z;
  e[3] = v.w;
}
template <>
__device__ __forceinline__ void unpack4<uint16_t>(const uint2& v, uint16_t* e) {
  e[0] = static_cast<uint16_t>(v.x & 0xFFFFu);
  e[1] = static_cast<uint16_t>(v.x >> 16);
  e[2] = static_cast<uint16_t>(v.y & 0xFFFFu);
  e[3] = static_cast<uint16_t>(v.y >> 16);
}
template <typename T>
__device__ __forceinline__ typename Vec4<T>::type pack4(const T* e);
template <>
__device__ __forceinline__ float4 pack4<float>(const float* e) {
  return make_float4(e[0], e[1], e[2], e[3]);
}
template <>
__device__ __forceinline__ uint2 pack4<uint16_t>(const uint16_t* e) {
  return make_uint2(static_cast<uint32_t>(e[0]) | (static_cast<uint32_t>(e[1]) << 16),
                    static_cast<uint32_t>(e[2]) | (static_cast<uint32_t>(e[3]) << 16));
}

template <typename T>
__global__ void __launch_bounds__(TR_THREADS) transpose_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                               long long rows, long long cols, int tiles_c,
                                                               long long tiles_per_mat, long long total_tiles,
                                                               int vec_ok) {
  using V = typename Vec4<T>::type;
  __shared__ T tile[TT][TT + (sizeof(T) == 4 ? 1 : 2)];
  const int tr = threadIdx.x >> 4;        // 0..15: row within a 16-row pass
  const int tc = (threadIdx.x & 15) * 4;  // first of this thread's 4 columns
  for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const long long b = t / tiles_per_mat;
    const long long r = t - b * tiles_per_mat;
    const long long i0 = (r / tiles_c) * TT, j0 = (r % tiles_c) * TT;
    const T* xb = x + b * rows * cols;
    T* yb = y + b * rows * cols;
    const bool full = vec_ok && i0 + TT <= rows && j0 + TT <= cols;
    if (full) {
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int i = tr + 16 * p;
        const V v = *reinterpret_cast<const V*>(xb + (i0 + i) * cols + j0 + tc);
        T e[4];
        unpack4<T>(v, e);
#pragma unroll
        for (int k = 0; k < 4; ++k) tile[i][tc + k] = e[k];
      }
      __syncthreads();
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int j = tr + 16 * p;        // row of Y inside the tile = column of X
        T e[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) e[k] = tile[tc + k][j];
        *reinterpret_cast<V*>(yb + (j0 + j) * rows + i0 + tc) = pack4<T>(e);
      }
    } else {
      for (int idx = threadIdx.x; idx < TT * TT; idx += TR_THREADS) {
        const int i = idx / TT, j = idx % TT;
        if (i0 + i < rows && j0 + j < cols) tile[i][j] = xb[(i0 + i) * cols + j0 + j];
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < TT * TT; idx += TR_THREADS) {
        const int j = idx / TT, i = idx % TT;
        if (i0 + i < rows && j0 + j < cols) yb[(j0 + j) * rows + i0 + i] = tile[i][j];
      }
    }
    __syncthreads();
  }
}

}  // namespace

kcg_status_t transpose_launch_impl(int64_t batch, int64_t rows, int64_t cols, int dtype, const void* x, void* y,
                                   cudaStream_t stream) {
  if (!x || !y) return KCG_BAD_ARGUMENT;
  if (x == y) return KCG_UNSUPPORTED;   // out of place only
  if (batch <= 0 || rows <= 0 || cols <= 0) return KCG_BAD_SHAPE;
  if (dtype != KCG_F32 && dtype != KCG_BF16) return KCG_UNSUPPORTED;
  const long long tiles_r = (rows + TT - 1) / TT, tiles_c = (cols + TT - 1) / TT;
  if (tiles_c > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  const long long per_mat = tiles_r * tiles_c;
  const long long total = per_mat * batch;
  const size_t es = dtype == KCG_F32 ? 4 : 2;
  // vector path: rows and columns multiples of 4 elements and 4-element-aligned bases
  const int vec_ok = (rows % 4 == 0) && (cols % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % (4 * es) == 0) &&
                     (reinterpret_cast<uintptr_t>(y) % (4 * es) == 0);
  const long long cap = static_cast<long long>(device_sm_count()) * 8;   // 8 resident CTAs per SM
  const int grid = static_cast<int>(total < cap ? total : cap);
  if (dtype == KCG_F32)
    transpose_kernel<float><<<grid, TR_THREADS, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y),
                                                             rows, cols, static_cast<int>(tiles_c), per_mat, total,
                                                             vec_ok);
  else
    transpose_kernel<uint16_t><<<grid, TR_THREADS, 0, stream>>>(static_cast<const uint16_t*>(x),
                                                                static_cast<uint16_t*>(y), rows, cols,
                                                                static_cast<int>(tiles_c), per_mat, total, vec_ok);
  g_launches.fetch_add(1);
  KCG_CUDA_TRY(cudaGetLastError());
  return KCG_OK;
}

}  // namespace kcg
