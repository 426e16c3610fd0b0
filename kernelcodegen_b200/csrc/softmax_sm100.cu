// Row softmax over the last axis, y = exp(x) / sum(exp(x)), the standalone form of the
// reference's Softmax operator (src/Frontend/Operators.cc:474-536; in place when x == y).
// Outside the attention chain (where it is fused into fmha_fwd_kernel) this is plain HBM-bound
// work: 4 bytes read + 4 bytes written per element, nothing for the tensor cores.
//
// One warp per row when the row fits in registers (<= 1024 columns: 32 per lane), one 256-thread
// CTA per row otherwise.  The row maximum is subtracted before exp (mathematically the same
// quotient, no overflow); max and sum are reduced with warp shuffles.
#include "common.cuh"
#include "ptx.cuh"

namespace kcg {

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

constexpr float LOG2E = 1.4426950408889634f;

// rows x cols, cols <= 1024: a warp keeps its row in registers (one HBM read, one write)
template <int PER_LANE>
__global__ void softmax_warp_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int cols) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    const float* xr = x + r * cols;
    float v[PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int c = lane + 32 * i;
      v[i] = c < cols ? xr[c] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      v[i] = ex2_approx((v[i] - mx) * LOG2E);
      sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    float* yr = y + r * cols;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int c = lane + 32 * i;
      if (c < cols) yr[c] = v[i] * inv;
    }
  }
}

// any cols: a CTA per row, three passes over the row (the second and third hit L2)
__global__ void softmax_block_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int cols) {
  __shared__ float red[8];
  __shared__ float bcast;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + r * cols;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, xr[c]);
    mx = warp_max(mx);
    if (lane == 0) red[w] = mx;
    __syncthreads();
    if (w == 0) {
      float t = lane < 8 ? red[lane] : -INFINITY;
      t = warp_max(t);
      if (lane == 0) bcast = t;
    }
    __syncthreads();
    mx = bcast;
    float sum = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) sum += ex2_approx((xr[c] - mx) * LOG2E);
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[w] = sum;
    __syncthreads();
    if (w == 0) {
      float t = lane < 8 ? red[lane] : 0.f;
      t = warp_sum(t);
      if (lane == 0) bcast = t;
    }
    __syncthreads();
    const float inv = 1.f / bcast;
    float* yr = y + r * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = ex2_approx((xr[c] - mx) * LOG2E) * inv;
    __syncthreads();
  }
}

}  // namespace

kcg_status_t softmax_launch_impl(long long rows, long long cols, const void* x, void* y, cudaStream_t stream) {
  if (!x || !y) return KCG_BAD_ARGUMENT;
  if (rows <= 0 || cols <= 0 || cols > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  const int sms = device_sm_count();
  const float* xs = static_cast<const float*>(x);
  float* ys = static_cast<float*>(y);
  const int c = static_cast<int>(cols);
  if (cols <= 1024) {
    const long long warps_needed = rows;
    long long blocks = (warps_needed + 7) / 8;
    const long long cap = static_cast<long long>(sms) * 8;
    if (blocks > cap) blocks = cap;
    const int g = static_cast<int>(blocks);
    if (cols <= 128) softmax_warp_kernel<4><<<g, 256, 0, stream>>>(xs, ys, rows, c);
    else if (cols <= 256) softmax_warp_kernel<8><<<g, 256, 0, stream>>>(xs, ys, rows, c);
    else if (cols <= 512) softmax_warp_kernel<16><<<g, 256, 0, stream>>>(xs, ys, rows, c);
    else softmax_warp_kernel<32><<<g, 256, 0, stream>>>(xs, ys, rows, c);
  } else {
    long long blocks = rows;
    const long long cap = static_cast<long long>(sms) * 8;
    if (blocks > cap) blocks = cap;
    softmax_block_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(xs, ys, rows, c);
  }
  g_launches.fetch_add(1);
  KCG_CUDA_TRY(cudaGetLastError());
  return KCG_OK;
}

}  // namespace kcg
