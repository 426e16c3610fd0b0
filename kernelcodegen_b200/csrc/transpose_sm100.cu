// Y[b, j, i] = X[b, i, j]: the Transpose operator the reference declares
// (include/Frontend/Operators.h:100-102) and leaves without a body
// (src/Frontend/Operators.cc:422-423).
//
// HBM-bound: every element is read once and written once.  A CTA moves one square tile (256
// bytes on a side: 64 x 64 fp32 or 128 x 128 bf16) through shared memory: rows of X are read with
// 16-byte vector loads (16 threads cover a row segment), the tile sits in shared memory with an
// odd pitch in words (a column spreads over the banks), and rows of Y are written with 16-byte
// vector stores.  Tiles on a ragged edge, and shapes whose rows or columns are not multiples of a
// vector, take an element-wise path of the same structure.  16-bit elements have their own kernel
// (transpose16_kernel) that keeps the tile as 32-bit words.
#include "common.cuh"

namespace kcg {

namespace {

constexpr int TR_THREADS = 256;

// 16 bytes of T, moved as one vector.
template <typename T>
union Pack16 {
  uint4 v;
  T e[16 / sizeof(T)];
};

// TT = tile edge in elements: 256 bytes of a row (64 fp32, 128 bf16), so that both the reads along
// rows of X and the writes along rows of Y move 256-byte segments.
template <typename T, int TT>
__global__ void __launch_bounds__(TR_THREADS) transpose_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                               long long rows, long long cols, int tiles_c,
                                                               long long tiles_r, long long tiles_per_mat,
                                                               long long total_tiles, int vec_ok) {
  constexpr int VW = 16 / sizeof(T);        // elements per 16-byte vector
  constexpr int PAD = 4 / sizeof(T);        // one 32-bit word of padding: odd pitch in words
  constexpr int PASSES = TT / 16;           // 16 threads cover a row segment, 16 rows per pass
  static_assert(TT / VW == 16, "a row segment is 16 vectors");
  extern __shared__ __align__(16) unsigned char tr_smem[];
  T(*tile)[TT + PAD] = reinterpret_cast<T(*)[TT + PAD]>(tr_smem);
  const int tr = threadIdx.x >> 4;          // 0..15: row within a 16-row pass
  const int tc = (threadIdx.x & 15) * VW;   // first of this thread's VW columns
  // where tile t lies, and whether it takes the vector path
  auto locate = [&](long long t, const T*& xb, T*& yb, long long& i0, long long& j0) -> bool {
    const long long b = t / tiles_per_mat;
    const long long r = t - b * tiles_per_mat;
    // Tiles are walked in bands of 8 tile rows, column by column inside a band, so the CTAs that
    // run at the same time cover 8 x 8-ish blocks of tiles: their reads (along rows of X) and
    // their writes (along rows of Y) both fall on runs of neighbouring 256-byte segments.
    const long long band = r / (8ll * tiles_c);
    const long long in_band = r - band * 8ll * tiles_c;
    const long long band_rows = min(8ll, tiles_r - band * 8);
    i0 = (band * 8 + in_band % band_rows) * TT;
    j0 = (in_band / band_rows) * TT;
    xb = x + b * rows * cols;
    yb = y + b * rows * cols;
    return vec_ok && i0 + TT <= rows && j0 + TT <= cols;
  };
  auto fetch = [&](const T* xb, long long i0, long long j0, uint4 (&v)[PASSES]) {
#pragma unroll
    for (int p = 0; p < PASSES; ++p)
      v[p] = __ldg(reinterpret_cast<const uint4*>(xb + (i0 + tr + 16 * p) * cols + j0 + tc));
  };
  // The loads of a CTA's next tile are issued before the stores of the current one, so reads
  // and writes of one CTA overlap instead of alternating.
  uint4 nxt[PASSES];
  {
    const T* xb;
    T* yb;
    long long i0, j0;
    if (blockIdx.x < total_tiles && locate(blockIdx.x, xb, yb, i0, j0)) fetch(xb, i0, j0, nxt);
  }
  for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const T* xb;
    T* yb;
    long long i0, j0;
    const bool full = locate(t, xb, yb, i0, j0);
    if (full) {
#pragma unroll
      for (int p = 0; p < PASSES; ++p) {
        Pack16<T> v;
        v.v = nxt[p];
#pragma unroll
        for (int k = 0; k < VW; ++k) tile[tr + 16 * p][tc + k] = v.e[k];
      }
    } else {
      for (int idx = threadIdx.x; idx < TT * TT; idx += TR_THREADS) {
        const int i = idx / TT, j = idx % TT;
        if (i0 + i < rows && j0 + j < cols) tile[i][j] = xb[(i0 + i) * cols + j0 + j];
      }
    }
    __syncthreads();
    {
      const T* xn;
      T* yn;
      long long in0, jn0;
      if (t + gridDim.x < total_tiles && locate(t + gridDim.x, xn, yn, in0, jn0)) fetch(xn, in0, jn0, nxt);
    }
    if (full) {
#pragma unroll
      for (int p = 0; p < PASSES; ++p) {
        const int j = tr + 16 * p;          // row of Y inside the tile = column of X
        Pack16<T> v;
#pragma unroll
        for (int k = 0; k < VW; ++k) v.e[k] = tile[tc + k][j];
        *reinterpret_cast<uint4*>(yb + (j0 + j) * rows + i0 + tc) = v.v;
      }
    } else {
      for (int idx = threadIdx.x; idx < TT * TT; idx += TR_THREADS) {
        const int j = idx / TT, i = idx % TT;
        if (i0 + i < rows && j0 + j < cols) yb[(j0 + j) * rows + i0 + i] = tile[i][j];
      }
    }
    __syncthreads();
  }
}

// 16-bit elements: the same walk over 128 x 128 tiles, but the tile sits in shared memory as 32-bit
// words (two neighbouring columns of X per word), so shared memory moves whole words in both
// phases instead of 2-byte halves (which cost the element-wise form 28 % of the bandwidth).  A
// word's column is XOR-ed with its row group (rows / 8) instead of padding the pitch.  A
// thread of the write phase owns a column pair (2 jw, 2 jw + 1) and eight consecutive rows of X:
// eight word loads give it both columns, two byte permutes per word pair sort them into the two
// rows of Y, and each row leaves as one 16-byte store.
__global__ void __launch_bounds__(TR_THREADS) transpose16_kernel(const uint16_t* x, uint16_t* y, long long rows,
                                                                 long long cols, int tiles_c, long long tiles_r,
                                                                 long long tiles_per_mat, long long total_tiles,
                                                                 int vec_ok) {
  constexpr int TT = 128;                   // tile edge in elements (256 bytes)
  constexpr int TW = TT / 2;                // words per tile row
  constexpr int PITCH = TW;                 // no padding: word (i, w) sits in column w ^ ((i >> 3) & 15) ^ ((i & 1) << 1)
  extern __shared__ __align__(16) unsigned char tr_smem[];
  uint32_t(*tile)[PITCH] = reinterpret_cast<uint32_t(*)[PITCH]>(tr_smem);
  const int tr = threadIdx.x >> 4;          // read phase: row within a 16-row pass
  const int tw = (threadIdx.x & 15) * 4;    // read phase: first of this thread's 4 words (8 columns)
  auto locate = [&](long long t, const uint16_t*& xb, uint16_t*& yb, long long& i0, long long& j0) -> bool {
    const long long b = t / tiles_per_mat;
    const long long r = t - b * tiles_per_mat;
    const long long band = r / (8ll * tiles_c);      // bands of 8 tile rows, column by column inside a band
    const long long in_band = r - band * 8ll * tiles_c;
    const long long band_rows = min(8ll, tiles_r - band * 8);
    i0 = (band * 8 + in_band % band_rows) * TT;
    j0 = (in_band / band_rows) * TT;
    xb = x + b * rows * cols;
    yb = y + b * rows * cols;
    return vec_ok && i0 + TT <= rows && j0 + TT <= cols;
  };
  constexpr int PASSES = TT / 16;
  auto fetch = [&](const uint16_t* xb, long long i0, long long j0, uint4 (&v)[PASSES]) {
#pragma unroll
    for (int p = 0; p < PASSES; ++p)
      v[p] = __ldg(reinterpret_cast<const uint4*>(xb + (i0 + tr + 16 * p) * cols + j0 + 2 * tw));
  };
  uint4 nxt[PASSES];
  {
    const uint16_t* xb;
    uint16_t* yb;
    long long i0, j0;
    if (blockIdx.x < total_tiles && locate(blockIdx.x, xb, yb, i0, j0)) fetch(xb, i0, j0, nxt);
  }
  uint16_t* tile16 = reinterpret_cast<uint16_t*>(tr_smem);   // element view for ragged tiles: [i][j] at i * 2 * PITCH + j
  for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const uint16_t* xb;
    uint16_t* yb;
    long long i0, j0;
    const bool full = locate(t, xb, yb, i0, j0);
    if (full) {
#pragma unroll
      for (int p = 0; p < PASSES; ++p) {
        const int r = tr + 16 * p;
        uint32_t* row = tile[r];
        const int sw = ((r >> 3) & 15) ^ ((r & 1) << 1);   // odd rows two columns over: the warp's two rows miss each other
        row[(tw + 0) ^ sw] = nxt[p].x;
        row[(tw + 1) ^ sw] = nxt[p].y;
        row[(tw + 2) ^ sw] = nxt[p].z;
        row[(tw + 3) ^ sw] = nxt[p].w;
      }
    } else {
      for (int idx = threadIdx.x; idx < TT * TT; idx += TR_THREADS) {
        const int i = idx / TT, j = idx % TT;
        if (i0 + i < rows && j0 + j < cols) tile16[i * 2 * PITCH + j] = xb[(i0 + i) * cols + j0 + j];
      }
    }
    __syncthreads();
    {
      const uint16_t* xn;
      uint16_t* yn;
      long long in0, jn0;
      if (t + gridDim.x < total_tiles && locate(t + gridDim.x, xn, yn, in0, jn0)) fetch(xn, in0, jn0, nxt);
    }
    if (full) {
      // 64 column pairs x 16 groups of eight rows = 1024 tasks, 256 per pass.  16 lanes take the 16
      // row groups of one column pair (256 contiguous bytes of a row of Y); the two column pairs
      // of a warp differ by 16, so with the column swizzle the 32 lanes read 32 different banks.
      const int ig = threadIdx.x & 15;                      // rows 8 ig .. 8 ig + 7 of X
      const int i8 = ig * 8;
      const int jsel = (threadIdx.x >> 4) & 1;
      const int wq = threadIdx.x >> 5;                      // warp 0..7
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int u = p * 8 + wq;                           // 0..31
        const int jw = (u & 15) + 16 * jsel + 32 * (u >> 4);   // column pair 0..63
        uint32_t w[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) w[k] = tile[i8 + k][jw ^ ig ^ ((k & 1) << 1)];
        uint4 lo, hi;
        lo.x = __byte_perm(w[0], w[1], 0x5410);
        lo.y = __byte_perm(w[2], w[3], 0x5410);
        lo.z = __byte_perm(w[4], w[5], 0x5410);
        lo.w = __byte_perm(w[6], w[7], 0x5410);
        hi.x = __byte_perm(w[0], w[1], 0x7632);
        hi.y = __byte_perm(w[2], w[3], 0x7632);
        hi.z = __byte_perm(w[4], w[5], 0x7632);
        hi.w = __byte_perm(w[6], w[7], 0x7632);
        *reinterpret_cast<uint4*>(yb + (j0 + 2 * jw) * rows + i0 + i8) = lo;
        *reinterpret_cast<uint4*>(yb + (j0 + 2 * jw + 1) * rows + i0 + i8) = hi;
      }
    } else {
      for (int idx = threadIdx.x; idx < TT * TT; idx += TR_THREADS) {
        const int j = idx / TT, i = idx % TT;
        if (i0 + i < rows && j0 + j < cols) yb[(j0 + j) * rows + i0 + i] = tile16[i * 2 * PITCH + j];
      }
    }
    __syncthreads();
  }
}

template <typename T, int TT>
kcg_status_t launch_transpose(int64_t batch, int64_t rows, int64_t cols, const void* x, void* y, cudaStream_t stream) {
  const long long tiles_r = (rows + TT - 1) / TT, tiles_c = (cols + TT - 1) / TT;
  if (tiles_c > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  const long long per_mat = tiles_r * tiles_c;
  const long long total = per_mat * batch;
  constexpr int VW = 16 / sizeof(T);
  // vector path: rows and columns multiples of a 16-byte vector and 16-byte-aligned bases
  const int vec_ok = (rows % VW == 0) && (cols % VW == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(y) % 16 == 0);
  constexpr int smem = TT * (TT + 4 / static_cast<int>(sizeof(T))) * static_cast<int>(sizeof(T));
  auto kern = transpose_kernel<T, TT>;
  KCG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int per_sm = 0;   // resident CTAs per SM: the persistent grid is exactly one resident wave
  KCG_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, TR_THREADS, smem));
  if (per_sm < 1) per_sm = 1;
  const long long cap = static_cast<long long>(device_sm_count()) * per_sm;
  const int grid = static_cast<int>(total < cap ? total : cap);
  kern<<<grid, TR_THREADS, smem, stream>>>(static_cast<const T*>(x), static_cast<T*>(y), rows, cols,
                                           static_cast<int>(tiles_c), tiles_r, per_mat, total, vec_ok);
  g_launches.fetch_add(1);
  KCG_CUDA_TRY(cudaGetLastError());
  return KCG_OK;
}

kcg_status_t launch_transpose16(int64_t batch, int64_t rows, int64_t cols, const void* x, void* y, cudaStream_t stream) {
  constexpr int TT = 128;
  const long long tiles_r = (rows + TT - 1) / TT, tiles_c = (cols + TT - 1) / TT;
  if (tiles_c > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  const long long per_mat = tiles_r * tiles_c;
  const long long total = per_mat * batch;
  const int vec_ok = (rows % 8 == 0) && (cols % 8 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(y) % 16 == 0);
  constexpr int smem = TT * (TT / 2) * 4;
  KCG_CUDA_TRY(cudaFuncSetAttribute(transpose16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int per_sm = 0;   // resident CTAs per SM: the persistent grid is exactly one resident wave
  KCG_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, transpose16_kernel, TR_THREADS, smem));
  if (per_sm < 1) per_sm = 1;
  const long long cap = static_cast<long long>(device_sm_count()) * per_sm;
  const int grid = static_cast<int>(total < cap ? total : cap);
  transpose16_kernel<<<grid, TR_THREADS, smem, stream>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(y), rows,
                                                         cols, static_cast<int>(tiles_c), tiles_r, per_mat, total, vec_ok);
  g_launches.fetch_add(1);
  KCG_CUDA_TRY(cudaGetLastError());
  return KCG_OK;
}

}  // namespace

kcg_status_t transpose_launch_impl(int64_t batch, int64_t rows, int64_t cols, int dtype, const void* x, void* y,
                                   cudaStream_t stream) {
  if (!x || !y) return KCG_BAD_ARGUMENT;
  if (x == y) return KCG_UNSUPPORTED;   // out of place only
  if (batch <= 0 || rows <= 0 || cols <= 0) return KCG_BAD_SHAPE;
  if (dtype == KCG_F32) return launch_transpose<float, 64>(batch, rows, cols, x, y, stream);
  if (dtype == KCG_BF16) return launch_transpose16(batch, rows, cols, x, y, stream);
  return KCG_UNSUPPORTED;
}

}  // namespace kcg
