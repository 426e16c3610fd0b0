// Row softmax over the last axis, y = exp(x) / sum(exp(x)), the standalone form of the
// reference's Softmax operator (src/Frontend/Operators.cc:474-536; in place when x == y).
// Outside the attention chain (where it is fused into fmha_fwd_kernel) this is plain HBM-bound
// work: 4 bytes read + 4 bytes written per element, nothing for the tensor cores.
//
// One warp per row when the row fits in registers (<= 1024 columns: 32 per lane); longer rows get
// a 256-thread CTA that stages the row in shared memory, so either way every element is read from
// HBM once and written once, with 16-byte accesses when the row length is a multiple of 4.  Rows
// too long for shared memory, or not a multiple of 4, take a three-pass / 4-byte path.  The row
// maximum is subtracted before exp (mathematically the same quotient, no overflow); max and sum
// are reduced with warp shuffles.
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

// x and y may be the same array (the operator is in place in the reference), so neither pointer is
// declared __restrict__ / const-cached: every element is read before it is written by the same
// thread, and nothing is read twice after a write.

// rows x cols, cols <= 1024, cols % 4 == 0: a warp keeps its row in registers (one HBM read, one
// write), 16 bytes per lane per access: lane l holds columns 4*l + 128*i .. +3.
template <int V4>
__global__ void __launch_bounds__(256) softmax_warp_vec_kernel(const float* x, float* y, long long rows, int cols) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    const float4* xr = reinterpret_cast<const float4*>(x + r * cols);
    float4 v[V4];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < V4; ++i) {
      const int c4 = lane + 32 * i;
      v[i] = (4 * c4 < cols) ? xr[c4] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      mx = fmaxf(fmaxf(mx, fmaxf(v[i].x, v[i].y)), fmaxf(v[i].z, v[i].w));
    }
    mx = warp_max(mx);
    const float off = mx * LOG2E;
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < V4; ++i) {
      v[i].x = ex2_approx(fmaf(v[i].x, LOG2E, -off));
      v[i].y = ex2_approx(fmaf(v[i].y, LOG2E, -off));
      v[i].z = ex2_approx(fmaf(v[i].z, LOG2E, -off));
      v[i].w = ex2_approx(fmaf(v[i].w, LOG2E, -off));
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    float4* yr = reinterpret_cast<float4*>(y + r * cols);
#pragma unroll
    for (int i = 0; i < V4; ++i) {
      const int c4 = lane + 32 * i;
      if (4 * c4 < cols) yr[c4] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
    }
  }
}

// the same for any cols <= 1024 (4-byte accesses)
template <int PER_LANE>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const float* x, float* y, long long rows, int cols) {
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

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red, float* bcast) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();                 // red / bcast of the previous reduction have been consumed
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < 8 ? red[lane] : (is_max ? -INFINITY : 0.f);
    t = is_max ? warp_max(t) : warp_sum(t);
    if (lane == 0) *bcast = t;
  }
  __syncthreads();
  return *bcast;
}

// Longer rows, cols % 4 == 0: a 256-thread CTA per row, the row staged in shared memory (one HBM
// read, one write), 16 bytes per thread per access.
__global__ void __launch_bounds__(256) softmax_block_smem_kernel(const float* x, float* y, long long rows, int cols) {
  extern __shared__ float4 row4[];
  __shared__ float red[8];
  __shared__ float bcast;
  const int n4 = cols >> 2;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float4* xr = reinterpret_cast<const float4*>(x + r * cols);
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < n4; c += blockDim.x) {
      const float4 v = xr[c];
      row4[c] = v;
      mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    mx = block_reduce(mx, true, red, &bcast);
    const float off = mx * LOG2E;
    float sum = 0.f;
    for (int c = threadIdx.x; c < n4; c += blockDim.x) {     // each thread revisits its own elements
      float4 v = row4[c];
      v.x = ex2_approx(fmaf(v.x, LOG2E, -off));
      v.y = ex2_approx(fmaf(v.y, LOG2E, -off));
      v.z = ex2_approx(fmaf(v.z, LOG2E, -off));
      v.w = ex2_approx(fmaf(v.w, LOG2E, -off));
      row4[c] = v;
      sum += (v.x + v.y) + (v.z + v.w);
    }
    sum = block_reduce(sum, false, red, &bcast);
    const float inv = 1.f / sum;
    float4* yr = reinterpret_cast<float4*>(y + r * cols);
    for (int c = threadIdx.x; c < n4; c += blockDim.x) {
      const float4 v = row4[c];
      yr[c] = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
    }
  }
}

// any cols: a CTA per row, three passes over the row (the second and third hit L2)
__global__ void __launch_bounds__(256) softmax_block_kernel(const float* x, float* y, long long rows, int cols) {
  __shared__ float red[8];
  __shared__ float bcast;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + r * cols;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, xr[c]);
    mx = block_reduce(mx, true, red, &bcast);
    float sum = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) sum += ex2_approx((xr[c] - mx) * LOG2E);
    sum = block_reduce(sum, false, red, &bcast);
    const float inv = 1.f / sum;
    float* yr = y + r * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = ex2_approx((xr[c] - mx) * LOG2E) * inv;
  }
}

constexpr int SOFTMAX_SMEM_MAX_COLS = 48 * 1024;   // 192 KB of shared memory for one row

}  // namespace

kcg_status_t softmax_launch_impl(long long rows, long long cols, const void* x, void* y, cudaStream_t stream) {
  if (!x || !y) return KCG_BAD_ARGUMENT;
  if (rows <= 0 || cols <= 0 || cols > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  const int sms = device_sm_count();
  const float* xs = static_cast<const float*>(x);
  float* ys = static_cast<float*>(y);
  const int c = static_cast<int>(cols);
  const bool vec = (cols % 4 == 0) && aligned16(x) && aligned16(y);
  if (cols <= 1024) {
    const long long warps_needed = rows;
    long long blocks = (warps_needed + 7) / 8;
    const long long cap = static_cast<long long>(sms) * 8;
    if (blocks > cap) blocks = cap;
    const int g = static_cast<int>(blocks);
    if (vec) {
      if (cols <= 128) softmax_warp_vec_kernel<1><<<g, 256, 0, stream>>>(xs, ys, rows, c);
      else if (cols <= 256) softmax_warp_vec_kernel<2><<<g, 256, 0, stream>>>(xs, ys, rows, c);
      else if (cols <= 512) softmax_warp_vec_kernel<4><<<g, 256, 0, stream>>>(xs, ys, rows, c);
      else softmax_warp_vec_kernel<8><<<g, 256, 0, stream>>>(xs, ys, rows, c);
    } else if (cols <= 128) softmax_warp_kernel<4><<<g, 256, 0, stream>>>(xs, ys, rows, c);
    else if (cols <= 256) softmax_warp_kernel<8><<<g, 256, 0, stream>>>(xs, ys, rows, c);
    else if (cols <= 512) softmax_warp_kernel<16><<<g, 256, 0, stream>>>(xs, ys, rows, c);
    else softmax_warp_kernel<32><<<g, 256, 0, stream>>>(xs, ys, rows, c);
  } else if (vec && cols <= SOFTMAX_SMEM_MAX_COLS) {
    const int smem = c * 4;
    if (smem > 48 * 1024)
      KCG_CUDA_TRY(cudaFuncSetAttribute(softmax_block_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int per_sm = smem > 0 ? (200 * 1024) / smem : 1;
    long long blocks = rows;
    const long long cap = static_cast<long long>(sms) * (per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm));
    if (blocks > cap) blocks = cap;
    softmax_block_smem_kernel<<<static_cast<int>(blocks), 256, smem, stream>>>(xs, ys, rows, c);
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
