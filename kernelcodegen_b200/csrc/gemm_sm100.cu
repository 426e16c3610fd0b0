// C[M,N] = epilogue(A[M,K] . B) on the 5th-generation tensor cores of sm_100a.
//
// The computation is the loop nest Matmul::build emits in the reference
// (src/Frontend/Operators.cc:140-173: C[i,j] = sum_k A[i,k]*B[k,j], fp32) followed by the
// elementwise max(0, x) of Relu::build (src/Frontend/Operators.cc:232-244), fused into the
// epilogue.  The reference schedules that nest for CUDA cores (128x128x8 CTA tile, 8x8 thread
// tile, src/Optimizer/Optimizer.cc:383-548); here the same roles are played by hardware units:
//
//   warp 0      TMA producer : global -> 128B-swizzled shared memory, STAGES-deep mbarrier ring
//   warp 1      UMMA issuer  : tcgen05.mma 128 x BN x (32 bytes of K), accumulators in TMEM,
//                              two accumulator buffers so tile i+1 starts while tile i drains
//   warps 2..5  epilogue of the tiles in accumulator buffer 0 } tcgen05.ld -> ReLU -> (bf16 pack)
//   warps 6..9  epilogue of the tiles in accumulator buffer 1 } -> global stores (and, for the
//                              fused all-gather, the same stores to peer GPUs).  Two groups, so
//                              that a drain (up to eight copies of the tile) may take as long as
//                              two main loops before it holds up the issuer.
//
// The grid is persistent (one CTA per SM); tiles are walked in groups of `group_m` row blocks
// so that concurrently running CTAs share A and B panels in L2.
//
// Precisions (KIND): 0 = bf16 inputs, 1 = single TF32 product of fp32 inputs,
// 2 = 3xTF32: four operand tiles per stage (A_hi, A_lo, B_hi, B_lo) and three UMMA passes
//     a_lo*b_hi + a_hi*b_lo + a_hi*b_hi accumulated in fp32.
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace kcg {

namespace {

// Scratch of the entry point that allocates nothing (kcg_gemm_launch_static): the hi/lo split
// copies of A and B live here instead of in a caller-provided workspace.  Every device that
// loads the library holds these bytes until the process exits.  In host code this name is only
// a stand-in for the symbol; the device address is looked up with cudaGetSymbolAddress.
constexpr size_t STATIC_SCRATCH_BYTES = KCG_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int BM = 128;
constexpr int GEMM_THREADS = 192;         // CTA-pair kernel: producer, issuer, 4 epilogue warps
constexpr int GEMM1_THREADS = 320;        // single-CTA kernel: producer, issuer, 2 x 4 epilogue warps
constexpr int SMEM_LIMIT = 232448;  // 227 KB opt-in limit per CTA

struct GemmParams {
  void* C;
  int M, N, K;
  long long ldc;
  int tiles_m, tiles_n, group_m;
  int relu;
  // Long-K fp32 products run as several launches over K ranges (see gemm_batched_launch_impl): a
  // launch with `accum` adds its tile to what C already holds (fp32, round-to-nearest, in the
  // epilogue's write loop) and applies ReLU afterwards when `relu_late` is set.
  int accum, relu_late;
  int* status;
  uint32_t spin;
  // bounds-checking build: bytes of C (all batch entries) and of the shared-K scratch, and where a
  // failed check leaves its offset; unused in the normal build
  unsigned long long c_extent, sk_extent;
  unsigned long long* bounds_detail;
  // Batched product: `batch` independent M x N x K products; tile index = batch entry major.  The
  // operands are 3-D tensor maps {k, rows, batch}; an operand shared by all entries has batch
  // extent 1 (a_bz / b_bz = 0: its batch coordinate stays 0).  C of entry b starts c_bstride
  // elements after that of entry b - 1.
  int batch, a_bz, b_bz;
  long long c_bstride;
  int n_peers;
  void* peers[8];
  // Multicast form of the fused all-gather: when set, full 128-byte row segments are stored once
  // to this address (NVSwitch multicast mapping of C at this rank's rows) instead of to C and
  // to each peer.
  void* mc;
  // Completion flags: the CTA that finishes last stores `flag_value` (release, system scope) to
  // each of these words, after every CTA's stores of C.  `done_counter` counts finished CTAs.
  int n_flags;
  uint32_t flag_value;
  uint32_t* flags[9];
  int* done_counter;
  // Shared-K tail (CTA-pair kernel): the last `sk_tiles` tiles do not fill a wave of the
  // persistent grid, so their k-blocks, laid end to end (`sk_span` >= num_kb positions per tile;
  // positions past num_kb are padding that makes a tile a whole number of ranges), are cut into
  // `sk_units` ranges of `sk_share` positions, one per pair; partial accumulators meet in
  // `sk_partial`.
  int sk_tiles, sk_units, sk_share, sk_span, sk_maxc;
  float* sk_partial;
  int* sk_count;   // one arrival counter per (tile, CTA of the pair, epilogue warp); zero between launches
};

// One piece of work of a persistent CTA (pair): k-blocks [kb0, kb1) of output tile t.
struct WorkItem {
  int t, kb0, kb1;
};

// Walks a pair's work: its range of the shared-K tiles (which may end one tile and begin the
// next), then whole tiles pair, pair + stride, ... below `dp_tiles`.
struct WorkIter {
  int t_next, stride, dp_tiles, num_kb, span, lin0, lin1;
  __device__ __forceinline__ WorkIter(const GemmParams& p, int unit, int units, int num_tiles, int nkb)
      : t_next(unit), stride(units), dp_tiles(num_tiles - p.sk_tiles), num_kb(nkb), span(p.sk_span), lin0(0), lin1(0) {
    if (p.sk_tiles > 0 && unit < p.sk_units) {
      const int total = p.sk_tiles * span;
      lin0 = min(total, unit * p.sk_share);
      lin1 = min(total, lin0 + p.sk_share);
    }
  }
  __device__ __forceinline__ bool next(WorkItem& w) {
    // The shared-K range comes first: adding up the partial accumulators takes a few L2 round
    // trips, and done first it runs beside the main loop of the whole tiles that follow
    // (the accumulators are double buffered) instead of at the very end of the kernel.
    while (lin0 < lin1) {
      const int ti = lin0 / span;
      const int off = lin0 - ti * span;
      const int end = min(span, off + (lin1 - lin0));
      lin0 += end - off;
      if (off < num_kb) {   // not all padding
        w.t = dp_tiles + ti;
        w.kb0 = off;
        w.kb1 = min(num_kb, end);
        return true;
      }
    }
    if (t_next < dp_tiles) {
      w.t = t_next;
      w.kb0 = 0;
      w.kb1 = num_kb;
      t_next += stride;
      return true;
    }
    return false;
  }
};

template <int KIND, int BN>
struct GemmCfg {
  static constexpr int ES = (KIND == 0) ? 2 : 4;     // bytes per input element
  static constexpr int BK = 128 / ES;                // one 128-byte swizzle row of K
  static constexpr int UK = 32 / ES;                 // K per UMMA instruction
  static constexpr int NOPS = (KIND == 2) ? 2 : 1;   // hi/lo copies per operand
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = NOPS * (A_BYTES + B_BYTES);
  static constexpr int CTRL_BYTES = 1024;            // barriers, TMEM pointer, abort flag
  static constexpr int EPI_BYTES = 8 * 4096;         // one 32-row x 128-byte staging slab per epilogue warp
  static constexpr int MAX_STAGES = (SMEM_LIMIT - CTRL_BYTES - EPI_BYTES - 1024) / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;           // two accumulator buffers (256 or 512)
};

// Epilogue of one accumulator tile for one warp: TMEM rows [32 lanes] x BN columns -> ReLU ->
// OutT -> global rows row0.. (and the same rows of every peer copy of C).
//
// With `sk_src` set, the tile is the sum of `sk_n` partial accumulators of this warp's slab: slot
// `sk_own` is the one in TMEM, the others lie in global memory (slot s at sk_src + s * 32 * BN
// floats, laid out as write_partial leaves them).  They are added in slot order, so the result
// does not depend on which contributor happens to finish last.
template <int BN, typename OutT>
__device__ __forceinline__ void drain_tile(const GemmParams& p, uint32_t t_row, int row0, int col0, long long c_off,
                                           uint8_t* epi_stage, int lane, const float* sk_src = nullptr,
                                           int sk_n = 0, int sk_own = 0) {
      // Each pass handles CW columns = 128 bytes of output per row: thread t (row t of the
      // slab) packs its part into the warp's staging slab [32 rows x 128 B] (16-byte chunks
      // XOR-swizzled by row against bank conflicts); the warp then writes the slab out with
      // 8 lanes per row, so every store instruction covers four full 128-byte row segments.
      constexpr int CW = 128 / static_cast<int>(sizeof(OutT));   // 64 bf16 or 32 fp32 columns
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CW) {
        const int col = col0 + c0;
        if (col >= p.N) break;
        const bool full = (col + CW <= p.N);
#pragma unroll
        for (int sub = 0; sub < CW / 32; ++sub) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c0 + sub * 32, r);
          if (sk_src != nullptr) {
            // the first foreign slot is fetched while the TMEM load is in flight (one L2 round trip
            // per chunk for two contributors); any further ones one after the other
            const float4* src = reinterpret_cast<const float4*>(sk_src) + ((c0 / 32 + sub) * 8) * 32 + lane;
            const int f0 = sk_own == 0 ? 1 : 0;
            float4 v0[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v0[j] = __ldcg(src + static_cast<size_t>(f0) * (8 * BN) + j * 32);
            tmem_ld_wait();
            float acc[32];
            for (int sl = 0; sl < sk_n; ++sl) {
              if (sl == sk_own) {
                if (sl == 0) {
#pragma unroll
                  for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(r[i]);
                } else {
#pragma unroll
                  for (int i = 0; i < 32; ++i) acc[i] += __uint_as_float(r[i]);
                }
              } else {
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  v[j] = (sl == f0) ? v0[j] : __ldcg(src + static_cast<size_t>(sl) * (8 * BN) + j * 32);
                if (sl == 0) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    acc[4 * j] = v[j].x;
                    acc[4 * j + 1] = v[j].y;
                    acc[4 * j + 2] = v[j].z;
                    acc[4 * j + 3] = v[j].w;
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    acc[4 * j] += v[j].x;
                    acc[4 * j + 1] += v[j].y;
                    acc[4 * j + 2] += v[j].z;
                    acc[4 * j + 3] += v[j].w;
                  }
                }
              }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(acc[i]);
          } else {
            tmem_ld_wait();
          }
          if (p.relu) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = (r[i] & 0x80000000u) ? 0u : r[i];
          }
          if (full) {
            uint8_t* srow = epi_stage + lane * 128;
            if (sizeof(OutT) == 2) {
#pragma unroll
              for (int ch = 0; ch < 4; ++ch) {  // 8 bf16 per 16-byte chunk
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                *reinterpret_cast<uint4*>(srow + (((sub * 4 + ch) ^ (lane & 7)) << 4)) = v;
              }
            } else {
#pragma unroll
              for (int ch = 0; ch < 8; ++ch)    // 4 fp32 per 16-byte chunk
                *reinterpret_cast<uint4*>(srow + ((ch ^ (lane & 7)) << 4)) =
                    make_uint4(r[4 * ch], r[4 * ch + 1], r[4 * ch + 2], r[4 * ch + 3]);
            }
          } else if (row0 + lane < p.M) {
            // ragged right edge: element-wise, this thread's row
            const long long off = c_off + static_cast<long long>(row0 + lane) * p.ldc + col + sub * 32;
            for (int dst = 0; dst <= p.n_peers; ++dst) {
              OutT* cp = static_cast<OutT*>(dst == 0 ? p.C : p.peers[dst - 1]) + off;
              for (int i = 0; i < 32; ++i) {
                if (col + sub * 32 + i < p.N &&
                    bounds_ok((off + i) * sizeof(OutT), sizeof(OutT), p.c_extent, p.status, p.bounds_detail)) {
                  if (sizeof(OutT) == 2) {
                    reinterpret_cast<__nv_bfloat16*>(cp)[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
                  } else if (p.accum) {
                    float v = reinterpret_cast<float*>(cp)[i] + __uint_as_float(r[i]);
                    if (p.relu_late) v = v > 0.f ? v : 0.f;
                    reinterpret_cast<float*>(cp)[i] = v;
                  } else {
                    reinterpret_cast<uint32_t*>(cp)[i] = r[i];
                  }
                }
              }
            }
          }
        }
        if (full) {
          __syncwarp();
          const int rr = lane >> 3, ch = lane & 7;
          if (p.mc != nullptr) {
            // one store per 16 bytes, replicated by the switch to every rank's C (this one's too)
            uint8_t* cbase = static_cast<uint8_t*>(p.mc);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rloc = i * 4 + rr;
              const int grow = row0 + rloc;
              if (grow < p.M &&
                  bounds_ok((c_off + static_cast<long long>(grow) * p.ldc + col) * sizeof(OutT) + ch * 16, 16, p.c_extent,
                            p.status, p.bounds_detail)) {
                const uint4 v = *reinterpret_cast<const uint4*>(epi_stage + rloc * 128 +
                                                                 ((ch ^ (rloc & 7)) << 4));
                multimem_st_v4(cbase + (c_off + static_cast<long long>(grow) * p.ldc + col) *
                                           static_cast<long long>(sizeof(OutT)) +
                                   ch * 16, v);
              }
            }
          }
          for (int dst = (p.mc != nullptr ? 1 : 0); dst <= p.n_peers; ++dst) {
            uint8_t* cbase = static_cast<uint8_t*>(dst == 0 ? p.C : p.peers[dst - 1]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rloc = i * 4 + rr;
              const int grow = row0 + rloc;
              if (grow < p.M &&
                  bounds_ok((c_off + static_cast<long long>(grow) * p.ldc + col) * sizeof(OutT) + ch * 16, 16, p.c_extent,
                            p.status, p.bounds_detail)) {
                uint4 v = *reinterpret_cast<const uint4*>(epi_stage + rloc * 128 +
                                                           ((ch ^ (rloc & 7)) << 4));
                uint4* out = reinterpret_cast<uint4*>(cbase + (c_off + static_cast<long long>(grow) * p.ldc + col) *
                                                                  static_cast<long long>(sizeof(OutT)) +
                                                      ch * 16);
                if (sizeof(OutT) == 4 && p.accum) {
                  const uint4 old = *out;
                  float4 f = make_float4(__uint_as_float(old.x) + __uint_as_float(v.x), __uint_as_float(old.y) + __uint_as_float(v.y),
                                         __uint_as_float(old.z) + __uint_as_float(v.z), __uint_as_float(old.w) + __uint_as_float(v.w));
                  if (p.relu_late) {
                    f.x = f.x > 0.f ? f.x : 0.f;
                    f.y = f.y > 0.f ? f.y : 0.f;
                    f.z = f.z > 0.f ? f.z : 0.f;
                    f.w = f.w > 0.f ? f.w : 0.f;
                  }
                  v = make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w));
                }
                *out = v;
              }
            }
          }
          __syncwarp();
        }
      }
}

// One warp's 32 x BN slab of a partial accumulator, TMEM -> global.  Float4 j of 32-column chunk
// c of row `lane` goes to float4 index (c * 8 + j) * 32 + lane: every store instruction of the
// warp covers 512 contiguous bytes, and the reader uses the same mapping.
template <int BN>
__device__ __forceinline__ void write_partial(const GemmParams& p, uint32_t t_row, float* dst, int lane) {
  // the whole 32 x BN slab of this warp must lie inside the scratch the host set aside
  if (!bounds_ok(reinterpret_cast<const uint8_t*>(dst) - reinterpret_cast<const uint8_t*>(p.sk_partial),
                 32ull * BN * sizeof(float), p.sk_extent, p.status, p.bounds_detail))
    return;
  float4* out = reinterpret_cast<float4*>(dst) + lane;
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(t_row + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      __stcg(out + (c * 8 + j) * 32, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
  }
}

// End of a launch that carries completion flags.  Every thread that stored C has executed a
// system-scope fence after its last store and the CTA has synchronised; one thread per CTA counts
// the CTA in, and the CTA that finds all the others counted publishes `flag_value` to every flag
// word (this rank's own and, through their peer mappings, the other ranks').  A consumer that
// reads the value with an acquire load therefore sees all of this launch's C.
__device__ __forceinline__ void signal_completion(const GemmParams& p) {
  if (p.n_flags <= 0) return;
  __threadfence_system();
  const int seen = atom_add_acq_rel_gpu(p.done_counter, 1);
  if (seen == static_cast<int>(gridDim.x) - 1) {
    *p.done_counter = 0;   // ready for the next launch that is handed this counter
    __threadfence_system();
    for (int i = 0; i < p.n_flags; ++i) st_release_sys_u32(p.flags[i], p.flag_value);
  }
}

template <int KIND, int BN, int STAGES, bool B_KMAJOR, typename OutT>
__global__ void __launch_bounds__(GEMM1_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
            const GemmParams p) {
  using Cfg = GemmCfg<KIND, BN>;
  constexpr int ES = Cfg::ES, BK = Cfg::BK, UK = Cfg::UK;
  constexpr int A_BYTES = Cfg::A_BYTES, B_BYTES = Cfg::B_BYTES;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
  constexpr uint32_t FMT = (KIND == 0) ? UMMA_FMT_BF16 : UMMA_FMT_TF32;
  constexpr uint32_t IDESC = make_idesc(FMT, BM, BN, 0, B_KMAJOR ? 0 : 1);
  // B in [K,N] row-major form is "MN-major": shared memory holds BN/(BK) column groups, each
  // BK k-rows of 128 bytes; successive groups are B_GROUP bytes apart.
  constexpr int B_NGROUP = 128 / ES;                 // n-elements per 128-byte row
  constexpr int B_GROUP = BK * 128;                  // bytes of one [BK x 128B] group
  constexpr uint32_t B_LBO = B_KMAJOR ? 16 : B_GROUP;
  constexpr uint32_t B_KSTEP = B_KMAJOR ? 32 : UK * 128;
  // fp32 operands stored along N use the 32-byte-atom swizzle (4-row period).
  constexpr bool B_ATOM32 = (!B_KMAJOR) && ES == 4;
  constexpr uint32_t B_SBO = B_ATOM32 ? 512 : 1024;
  constexpr uint32_t B_LAYOUT = B_ATOM32 ? SMEM_LAYOUT_SW128_ATOM32 : SMEM_LAYOUT_SW128;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;      // swizzle atoms need 1024-byte alignment
  uint8_t* ctrl = smem_raw + (base - raw) + STAGES * STAGE_BYTES;
  const uint32_t ctrl_u = base + STAGES * STAGE_BYTES;
  // control block: full[STAGES] | empty[STAGES] | tmem_full[2] | tmem_empty[2] | tmem ptr | abort
  const uint32_t bar_full = ctrl_u;
  const uint32_t bar_empty = ctrl_u + 8 * STAGES;
  const uint32_t bar_tfull = ctrl_u + 16 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(ctrl + 16 * STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 16 * STAGES + 36);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (KIND == 2) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int tiles_per_entry = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_entry * p.batch;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_per_group = p.group_m * p.tiles_n;

  auto tile_coord = [&](int t, int& mb, int& nb, int& bt) {
    bt = t / tiles_per_entry;
    t -= bt * tiles_per_entry;
    const int g = t / tiles_per_group;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, p.tiles_m - first_m);
    const int r = t - g * tiles_per_group;
    mb = first_m + r % gm;
    nb = r / gm;
  };

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // the residual arrays come from the launch just before this one; everything above ran
      // beside its tail (programmatic dependent launch)
      if (KIND == 2) griddep_wait();
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb, bt;
        tile_coord(t, mb, nb, bt);
        const int m0 = mb * BM, n0 = nb * BN;
        const int za = bt * p.a_bz, zb = bt * p.b_bz;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status,
                         DEV_TIMEOUT_PRODUCER, p.spin);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sA = base + stage * STAGE_BYTES;
          const uint32_t sB = sA + Cfg::NOPS * A_BYTES;
          mbar_expect_tx(full, STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_3d(sA, &tmA, full, k0, m0, za);
          if (KIND == 2) tma_load_3d(sA + A_BYTES, &tmA2, full, k0, m0, za);
          if (B_KMAJOR) {
            tma_load_3d(sB, &tmB, full, k0, n0, zb);
            if (KIND == 2) tma_load_3d(sB + B_BYTES, &tmB2, full, k0, n0, zb);
          } else {
#pragma unroll
            for (int j = 0; j < BN / B_NGROUP; ++j) {
              tma_load_3d(sB + j * B_GROUP, &tmB, full, n0 + j * B_NGROUP, k0, zb);
              if (KIND == 2)
                tma_load_3d(sB + B_BYTES + j * B_GROUP, &tmB2, full, n0 + j * B_NGROUP, k0, zb);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Unwinding: let copies already in flight land before the CTA's shared memory goes
        // away.  Stages before `stage` were armed in the current phase, the others in the
        // previous one (a never-armed barrier passes a wait on parity 1 at once).
        for (int s = 0; s < STAGES; ++s) {
          const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
          for (uint32_t it = 0; it < 4096u; ++it)
            if (mbar_try_wait(bar_full + 8 * s, par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer ---------------------------------------------
    // The whole warp walks the loop and waits on the barriers; one elected lane issues, so
    // descriptors and addresses stay warp-uniform (see elect_one()).
    {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      const uint64_t a_desc0 = make_smem_desc(base, 16, 1024);
      const uint64_t b_desc0 = make_smem_desc(base + Cfg::NOPS * A_BYTES, B_LBO, B_SBO, B_LAYOUT);
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status,
                                               DEV_TIMEOUT_MMA_TMEM, p.spin));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status,
                                                 DEV_TIMEOUT_MMA_FULL, p.spin));
          if (!ok) break;
          tc_fence_after();
          // start-address field (16-byte units) of this stage's operand tiles
          const uint64_t ad0 = a_desc0 + static_cast<uint64_t>((stage * STAGE_BYTES) >> 4);
          const uint64_t bd0 = b_desc0 + static_cast<uint64_t>((stage * STAGE_BYTES) >> 4);
          if (elect_one()) {
            if (KIND == 2) {
              // small terms first: a_lo*b_hi, a_hi*b_lo, then a_hi*b_hi
#pragma unroll
              for (int pass = 0; pass < 3; ++pass) {
                const uint64_t a_off = (pass == 0) ? (A_BYTES >> 4) : 0;
                const uint64_t b_off = (pass == 1) ? (B_BYTES >> 4) : 0;
#pragma unroll
                for (int k = 0; k < BK / UK; ++k)
                  umma_tf32_ss(d_tmem, ad0 + a_off + ((k * 32) >> 4), bd0 + b_off + ((k * B_KSTEP) >> 4), IDESC,
                               (kb | pass | k) ? 1u : 0u);
              }
            } else {
#pragma unroll
              for (int k = 0; k < BK / UK; ++k) {
                const uint64_t ad = ad0 + ((k * 32) >> 4);
                const uint64_t bd = bd0 + ((k * B_KSTEP) >> 4);
                if (KIND == 0)
                  umma_bf16_ss(d_tmem, ad, bd, IDESC, (kb | k) ? 1u : 0u);
                else
                  umma_tf32_ss(d_tmem, ad, bd, IDESC, (kb | k) ? 1u : 0u);
              }
            }
            umma_commit(bar_empty + 8 * stage);  // stage reusable once these UMMAs have read it
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          if (elect_one()) umma_commit(bar_tfull + 8 * acc);
          __syncwarp();
        }
      }
      if (!ok) {
        // Unwinding: UMMAs already issued still read shared memory and write TMEM.  One more
        // commit arrives on this stage's `empty` barrier when all of them have finished; wait for
        // it (bounded) before TMEM is freed.  The barrier has completed as many phases as this
        // stage was passed, so the new arrival completes the phase of parity `phase`.
        if (elect_one()) umma_commit(bar_empty + 8 * stage);
        __syncwarp();
        for (uint32_t it = 0; it < 65536u; ++it)
          if (mbar_try_wait(bar_empty + 8 * stage, phase)) break;
      }
    }
  } else {
    // ------------------------------- epilogue (2 groups of 4 warps) --------------------------
    const int q = warp & 3;               // TMEM lane quarter this warp may read
    const int grp = (warp - 2) >> 2;      // group g drains the tiles that land in accumulator buffer g
    uint8_t* epi_stage = ctrl + Cfg::CTRL_BYTES + (grp * 4 + q) * 4096;  // this warp's 32 x 128 B slab
    int local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
      const int acc = local & 1;
      if (acc != grp) continue;
      int mb, nb, bt;
      tile_coord(t, mb, nb, bt);
      const uint32_t acc_phase = (local >> 1) & 1u;
      ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE,
                     p.spin);
      if (!ok) break;
      tc_fence_after();
      const int row0 = mb * BM + q * 32;           // first row of this warp's 32-row slab
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      drain_tile<BN, OutT>(p, t_row, row0, nb * BN, bt * p.c_bstride, epi_stage, lane);
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
    }
    if (p.n_flags > 0) __threadfence_system();   // this thread's stores of C, before the flags
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag == 0) signal_completion(p);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}


// ---- CTA-pair variant (cluster of 2, tcgen05 cta_group::2) ------------------------------------
// Two CTAs on neighbouring SMs share one 256 x BN output tile: each loads its own 128 rows of A
// and only HALF of the B tile (BN/2 columns); one UMMA issued by the leader CTA drives both
// tensor cores, each reading its local A and both halves of B, and each CTA's TMEM receives its
// 128 x BN accumulator.  Per SM this halves the B bytes fetched from L2 and read from shared
// memory per flop (96 -> 64 B/clk at BN = 256), which is what limits the single-CTA kernel.
// Protocol: `full` barriers live in the leader (it expects the bytes of both CTAs' TMA loads,
// the peer's loads signal it through its cluster address); `empty` and `tmem_full` barriers are
// per CTA and the leader commits to both; `tmem_empty` lives in the leader and collects the 256
// epilogue threads of both CTAs.  Every TMA load is a plain per-CTA load.
template <int KIND, int BN>
struct PairCfg {
  static constexpr int ES = (KIND == 0) ? 2 : 4;
  static constexpr int BK = 128 / ES;
  static constexpr int UK = 32 / ES;
  static constexpr int NOPS = (KIND == 2) ? 2 : 1;
  static constexpr int A_BYTES = BM * 128;
  static constexpr int BNL = BN / 2;                 // B columns held by one CTA
  static constexpr int B_BYTES = BNL * 128;
  static constexpr int STAGE_BYTES = NOPS * (A_BYTES + B_BYTES);
  static constexpr int CTRL_BYTES = 1024;
  static constexpr int EPI_BYTES = 4 * 4096;
  static constexpr int MAX_STAGES = (SMEM_LIMIT - CTRL_BYTES - EPI_BYTES - 1024) / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
};

template <int KIND, int BN, int STAGES, bool B_KMAJOR, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                 const GemmParams p) {
  using Cfg = PairCfg<KIND, BN>;
  constexpr int ES = Cfg::ES, BK = Cfg::BK, UK = Cfg::UK, BNL = Cfg::BNL;
  constexpr int A_BYTES = Cfg::A_BYTES, B_BYTES = Cfg::B_BYTES;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
  constexpr uint32_t FMT = (KIND == 0) ? UMMA_FMT_BF16 : UMMA_FMT_TF32;
  constexpr uint32_t IDESC = make_idesc(FMT, 2 * BM, BN, 0, B_KMAJOR ? 0 : 1);
  constexpr int B_NGROUP = 128 / ES;
  constexpr int B_GROUP = BK * 128;
  constexpr uint32_t B_LBO = B_KMAJOR ? 16 : B_GROUP;
  constexpr uint32_t B_KSTEP = B_KMAJOR ? 32 : UK * 128;
  constexpr bool B_ATOM32 = (!B_KMAJOR) && ES == 4;
  constexpr uint32_t B_SBO = B_ATOM32 ? 512 : 1024;
  constexpr uint32_t B_LAYOUT = B_ATOM32 ? SMEM_LAYOUT_SW128_ATOM32 : SMEM_LAYOUT_SW128;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* ctrl = smem_raw + (base - raw) + STAGES * STAGE_BYTES;
  const uint32_t ctrl_u = base + STAGES * STAGE_BYTES;
  const uint32_t bar_full = ctrl_u;                  // used in the leader only
  const uint32_t bar_empty = ctrl_u + 8 * STAGES;    // per CTA
  const uint32_t bar_tfull = ctrl_u + 16 * STAGES;   // per CTA
  const uint32_t bar_tempty = bar_tfull + 16;        // used in the leader only
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(ctrl + 16 * STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 16 * STAGES + 36);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (KIND == 2) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 256);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_holder), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();    // both CTAs' barriers are initialised and both TMEM allocations exist
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int tiles_m2 = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_per_entry = tiles_m2 * p.tiles_n;
  const int num_tiles = tiles_per_entry * p.batch;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_per_group = p.group_m * p.tiles_n;
  auto tile_coord = [&](int t, int& mb, int& nb, int& bt) {
    bt = t / tiles_per_entry;
    t -= bt * tiles_per_entry;
    const int g = t / tiles_per_group;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, tiles_m2 - first_m);
    const int r = t - g * tiles_per_group;
    mb = first_m + r % gm;
    nb = r / gm;
  };

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (KIND == 2) griddep_wait();   // the residual arrays come from the launch just before
      WorkIter it(p, pair, num_pairs, num_tiles, num_kb);
      WorkItem w;
      while (ok && it.next(w)) {
        int mb, nb, bt;
        tile_coord(w.t, mb, nb, bt);
        const int m0 = mb * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = nb * BN + static_cast<int>(rank) * BNL;
        const int za = bt * p.a_bz, zb = bt * p.b_bz;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER, p.spin);
          if (!ok) break;
          const uint32_t full = mapa_shared(bar_full + 8 * stage, 0);   // the leader's barrier
          const uint32_t sA = base + stage * STAGE_BYTES;
          const uint32_t sB = sA + Cfg::NOPS * A_BYTES;
          if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_3d_pair(sA, &tmA, full, k0, m0, za);
          if (KIND == 2) tma_load_3d_pair(sA + A_BYTES, &tmA2, full, k0, m0, za);
          if (B_KMAJOR) {
            tma_load_3d_pair(sB, &tmB, full, k0, n0, zb);
            if (KIND == 2) tma_load_3d_pair(sB + B_BYTES, &tmB2, full, k0, n0, zb);
          } else {
#pragma unroll
            for (int j = 0; j < BNL / B_NGROUP; ++j) {
              tma_load_3d_pair(sB + j * B_GROUP, &tmB, full, n0 + j * B_NGROUP, k0, zb);
              if (KIND == 2) tma_load_3d_pair(sB + B_BYTES + j * B_GROUP, &tmB2, full, n0 + j * B_NGROUP, k0, zb);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        // Unwinding after a wait ran out somewhere in the pair: copies already requested must land
        // before either CTA's shared memory goes away.  The leader's `full` barriers collect the
        // bytes of BOTH CTAs' loads, so the leader polls them (bounded) for every stage that was
        // armed: stages before `stage` in the current phase, the others in the previous one (a
        // barrier that was never armed passes a wait on parity 1 at once).  The peer CTA cannot
        // see those barriers complete from its side; it stays resident until the cluster-wide
        // synchronisation below, which the leader reaches only after this loop.
        if (rank == 0) {
          for (int s = 0; s < STAGES; ++s) {
            const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
            for (uint32_t it = 0; it < 4096u; ++it)
              if (mbar_try_wait(bar_full + 8 * s, par)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer (leader CTA only) --------------------------
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      const uint64_t a_desc0 = make_smem_desc(base, 16, 1024);
      const uint64_t b_desc0 = make_smem_desc(base + Cfg::NOPS * A_BYTES, B_LBO, B_SBO, B_LAYOUT);
      WorkIter it(p, pair, num_pairs, num_tiles, num_kb);
      WorkItem w;
      for (; ok && it.next(w); ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status,
                                               DEV_TIMEOUT_MMA_TMEM, p.spin));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status,
                                                 DEV_TIMEOUT_MMA_FULL, p.spin));
          if (!ok) break;
          tc_fence_after();
          const uint64_t ad0 = a_desc0 + static_cast<uint64_t>((stage * STAGE_BYTES) >> 4);
          const uint64_t bd0 = b_desc0 + static_cast<uint64_t>((stage * STAGE_BYTES) >> 4);
          if (elect_one()) {
            if (KIND == 2) {
#pragma unroll
              for (int pass = 0; pass < 3; ++pass) {
                const uint64_t a_off = (pass == 0) ? (A_BYTES >> 4) : 0;
                const uint64_t b_off = (pass == 1) ? (B_BYTES >> 4) : 0;
#pragma unroll
                for (int k = 0; k < BK / UK; ++k)
                  umma_tf32_ss_pair(d_tmem, ad0 + a_off + ((k * 32) >> 4), bd0 + b_off + ((k * B_KSTEP) >> 4),
                                    IDESC, ((kb - w.kb0) | pass | k) ? 1u : 0u);
              }
            } else {
#pragma unroll
              for (int k = 0; k < BK / UK; ++k) {
                const uint64_t ad = ad0 + ((k * 32) >> 4);
                const uint64_t bd = bd0 + ((k * B_KSTEP) >> 4);
                if (KIND == 0)
                  umma_bf16_ss_pair(d_tmem, ad, bd, IDESC, ((kb - w.kb0) | k) ? 1u : 0u);
                else
                  umma_tf32_ss_pair(d_tmem, ad, bd, IDESC, ((kb - w.kb0) | k) ? 1u : 0u);
              }
            }
            // the stage is free in both CTAs once these UMMAs have read it
            umma_commit_pair(bar_empty + 8 * stage);
            umma_commit_pair(mapa_shared(bar_empty + 8 * stage, 1));
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          if (elect_one()) {
            umma_commit_pair(bar_tfull + 8 * acc);
            umma_commit_pair(mapa_shared(bar_tfull + 8 * acc, 1));
          }
          __syncwarp();
        }
      }
      if (!ok) {
        // Unwinding: UMMAs already issued still read shared memory and write TMEM of both CTAs.
        // One more commit arrives on a stage barrier when all of them have finished; wait for it
        // (bounded) before the pair synchronises and frees TMEM.  `empty` of `stage` last saw the
        // commit of the k-block issued STAGES blocks ago, so the new arrival completes the phase a
        // producer waiting for that stage would wait on.
        if (elect_one()) umma_commit_pair(bar_empty + 8 * stage);
        __syncwarp();
        for (uint32_t it = 0; it < 65536u; ++it)
          if (mbar_try_wait(bar_empty + 8 * stage, phase)) break;
      }
    }
  } else {
    // ------------------------------- epilogue (4 warps, both CTAs) ---------------------------
    const int q = warp & 3;
    uint8_t* epi_stage = ctrl + Cfg::CTRL_BYTES + q * 4096;
    const uint32_t tempty_leader = mapa_shared(bar_tempty, 0);
    int local = 0;
    bool ok = true;
    WorkIter it(p, pair, num_pairs, num_tiles, num_kb);
    WorkItem w;
    for (; ok && it.next(w); ++local) {
      int mb, nb, bt;
      tile_coord(w.t, mb, nb, bt);
      const long long c_off = bt * p.c_bstride;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE, p.spin);
      if (!ok) break;
      tc_fence_after();
      const int row0 = mb * 2 * BM + static_cast<int>(rank) * BM + q * 32;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (w.kb1 - w.kb0 == num_kb) {
        drain_tile<BN, OutT>(p, t_row, row0, nb * BN, c_off, epi_stage, lane);
      } else {
        // Part of a tile's K range.  Every contributor leaves its partial slab in global memory and
        // counts itself in; nobody waits: whoever finds all the others already counted adds the
        // slabs up (in slot order) and writes the tile.
        const int ti = w.t - (num_tiles - p.sk_tiles);
        const int first = (ti * p.sk_span) / p.sk_share;
        const int last = min(p.sk_units - 1, (ti * p.sk_span + num_kb - 1) / p.sk_share);
        const int n_contrib = last - first + 1;
        const int slab = (ti * 2 + static_cast<int>(rank)) * 4 + q;
        float* slab_base = p.sk_partial + static_cast<size_t>(slab) * p.sk_maxc * (32 * BN);
        write_partial<BN>(p, t_row, slab_base + static_cast<size_t>(pair - first) * (32 * BN), lane);
        __syncwarp();
        // release the warp's slab and learn how many contributors came before, in one atomic
        int seen = 0;
        if (lane == 0) seen = atom_add_acq_rel_gpu(p.sk_count + slab, 1);
        seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
        if (seen == n_contrib - 1) {
          drain_tile<BN, OutT>(p, t_row, row0, nb * BN, c_off, epi_stage, lane, slab_base, n_contrib, pair - first);
          if (lane == 0) p.sk_count[slab] = 0;   // ready for the next launch
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(tempty_leader + 8 * acc);
    }
    if (p.n_flags > 0) __threadfence_system();   // this thread's stores of C, before the flags
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag == 0) signal_completion(p);
  cluster_sync_all();    // the peer may still signal barriers in this CTA's shared memory until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

// Residuals for the 3xTF32 product: lo = x - hi with hi = x with the 13 low mantissa bits cleared
// (exact in fp32).  The tensor core itself truncates fp32 operands to TF32 (measured: 1 + 2^-11 +
// 2^-12 multiplies as 1.0), so the original arrays serve as the hi operands and only the
// residuals are materialised.  One launch covers both operands; outputs are compact [rows, cols].
struct SplitArgs {
  const float* src;
  float* lo;
  long long rows;     // rows of all batch entries together (batch * rows per entry)
  int cols4;
  long long ld;
  long long rows_per_entry;
  long long entry_stride;   // elements between the first rows of successive entries in src
};
__device__ __forceinline__ float4 tf32_residual(const float4 v) {
  float4 l;
  l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
  l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
  l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
  l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
  return l;
}
__global__ void __launch_bounds__(256) split_lo_kernel(SplitArgs a, SplitArgs b) {
  griddep_launch_dependents();   // the GEMM may move in and set itself up while this runs
  const long long na = a.rows * a.cols4, nb = b.rows * b.cols4, n = na + nb;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  auto src_of = [&](long long i) -> const float4* {
    const bool second = i >= na;
    const SplitArgs& s = second ? b : a;
    const long long k = second ? i - na : i;
    const long long r = k / s.cols4;
    const long long e = r / s.rows_per_entry;
    return reinterpret_cast<const float4*>(s.src + e * s.entry_stride + (r - e * s.rows_per_entry) * s.ld +
                                           4ll * (k - r * s.cols4));
  };
  auto dst_of = [&](long long i) -> float4* {
    return i >= na ? reinterpret_cast<float4*>(b.lo) + (i - na) : reinterpret_cast<float4*>(a.lo) + i;
  };
  // four independent 16-byte loads in flight per thread before the first store
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < n; i += 4 * stride) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldg(src_of(i + u * stride));
#pragma unroll
    for (int u = 0; u < 4; ++u) *dst_of(i + u * stride) = tf32_residual(v[u]);
  }
  for (; i < n; i += stride) *dst_of(i) = tf32_residual(__ldg(src_of(i)));
}

inline size_t pad256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// Arrival counters of the shared-K tail.  A launch uses one row; rows are handed out round robin,
// so launches that overlap on one device (different streams) do not share counters unless
// SK_ROWS of them are in flight at once.  The kernel leaves every counter it used at zero.
constexpr int SK_ROWS = 32;
constexpr int SK_MAX_TILES = 80;                       // tail tiles: fewer than the pairs of one wave
constexpr int SK_ROW_INTS = SK_MAX_TILES * 8;          // tile x CTA of the pair x epilogue warp
static __device__ int g_sk_counters[SK_ROWS * SK_ROW_INTS];
std::atomic<unsigned> g_sk_row{0};

static kcg_status_t sk_counters_ptr(int** out) {
  static std::mutex mu;
  static int* cache[64] = {};
  int dev = 0;
  KCG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return KCG_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* q = nullptr;
    KCG_CUDA_TRY(cudaGetSymbolAddress(&q, g_sk_counters));
    if (!q) return KCG_CUDA_ERROR;
    cache[dev] = static_cast<int*>(q);
  }
  *out = cache[dev];
  return KCG_OK;
}

// Counters of finished CTAs for launches that publish completion flags: one per launch, handed
// out round robin (launches that overlap on a device use different ones unless DONE_ROWS of them
// are in flight), each on its own 128-byte line, left at zero by the launch that used it.
constexpr int DONE_ROWS = 32;
constexpr int DONE_STRIDE = 32;
static __device__ int g_done_counters[DONE_ROWS * DONE_STRIDE];
std::atomic<unsigned> g_done_row{0};

static kcg_status_t done_counters_ptr(int** out) {
  static std::mutex mu;
  static int* cache[64] = {};
  int dev = 0;
  KCG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return KCG_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* q = nullptr;
    KCG_CUDA_TRY(cudaGetSymbolAddress(&q, g_done_counters));
    if (!q) return KCG_CUDA_ERROR;
    cache[dev] = static_cast<int*>(q);
  }
  *out = cache[dev];
  return KCG_OK;
}

// Plan of the shared-K tail for `tiles` pair tiles of `num_kb` k-blocks on `pairs` CTA pairs.
struct SkPlan {
  int tiles = 0, units = 0, share = 0, span = 0, maxc = 0;
  size_t bytes = 0;    // partial accumulators
};
inline SkPlan plan_shared_k(int tiles, int num_kb, int pairs, int bn) {
  SkPlan pl;
  if (pairs <= 1 || tiles % pairs == 0) return pl;
  const int r = tiles % pairs;
  if (r > SK_MAX_TILES) return pl;
  constexpr int MIN_SHARE = 8;   // k-blocks: a few microseconds of tensor work per range
  int share, span;
  if (pairs / r >= 2) {
    // every left-over tile is cut into g equal ranges: g contributors per tile, none shared
    int g = std::min(pairs / r, 4);
    while (g > 1 && ((num_kb + g - 1) / g < MIN_SHARE || (g - 1) * ((num_kb + g - 1) / g) >= num_kb)) --g;
    if (g < 2) return pl;
    share = (num_kb + g - 1) / g;
    span = g * share;
  } else {
    // more left-over tiles than half the pairs: equal ranges of the k-blocks laid end to end; a
    // range may end one tile and begin the next (at most 3 contributors per tile)
    const long long total = static_cast<long long>(r) * num_kb;
    long long sh = (total + pairs - 1) / pairs;
    sh = std::max<long long>(sh, MIN_SHARE);
    sh = std::max<long long>(sh, (num_kb + 1) / 2);
    if (sh * 5 > static_cast<long long>(num_kb) * 4) return pl;   // tail less than a fifth shorter
    share = static_cast<int>(sh);
    span = num_kb;
  }
  const long long total = static_cast<long long>(r) * span;
  const int units = static_cast<int>((total + share - 1) / share);
  int maxc = 1;
  for (int t = 0; t < r; ++t) {
    const long long first = (static_cast<long long>(t) * span) / share;
    const long long last = std::min<long long>(units - 1, (static_cast<long long>(t) * span + num_kb - 1) / share);
    maxc = std::max(maxc, static_cast<int>(last - first + 1));
  }
  pl.tiles = r;
  pl.units = units;
  pl.share = share;
  pl.span = span;
  pl.maxc = maxc;
  pl.bytes = static_cast<size_t>(r) * 8 * maxc * 32 * bn * sizeof(float);
  return pl;
}

template <int KIND, int BN, bool B_KMAJOR, typename OutT>
kcg_status_t launch_instance(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
                             const CUtensorMap& tB2, const GemmParams& p, int stages_req,
                             cudaStream_t stream) {
  using Cfg = GemmCfg<KIND, BN>;
  constexpr int STAGES = Cfg::MAX_STAGES > 8 ? 8 : Cfg::MAX_STAGES;
  static_assert(STAGES >= 2, "need at least two pipeline stages");
  if (stages_req != 0 && stages_req != STAGES) return KCG_UNSUPPORTED;
  auto kern = gemm_kernel<KIND, BN, STAGES, B_KMAJOR, OutT>;
  constexpr int smem = STAGES * Cfg::STAGE_BYTES + Cfg::CTRL_BYTES + Cfg::EPI_BYTES + 1024;
  static_assert(smem <= SMEM_LIMIT, "shared memory budget");
  KCG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int sms = device_sm_count();
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batch;
  const int grid = tiles < sms ? static_cast<int>(tiles) : sms;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(GEMM1_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  // 3xTF32: overlap the set-up with the residual pass before it (not for a launch that adds to
  // the C the launch before it wrote)
  cfg.numAttrs = (KIND == 2 && !p.accum) ? 1 : 0;
  KCG_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tA, tB, tA2, tB2, p));
  g_launches.fetch_add(1);
  return KCG_OK;
}

template <int KIND, typename OutT>
kcg_status_t dispatch_shape(int bn, bool b_kmajor, const CUtensorMap& tA, const CUtensorMap& tB,
                            const CUtensorMap& tA2, const CUtensorMap& tB2, const GemmParams& p,
                            int stages, cudaStream_t s) {
  if (bn == 256) {
    return b_kmajor ? launch_instance<KIND, 256, true, OutT>(tA, tB, tA2, tB2, p, stages, s)
                    : launch_instance<KIND, 256, false, OutT>(tA, tB, tA2, tB2, p, stages, s);
  }
  if (bn == 128) {
    return b_kmajor ? launch_instance<KIND, 128, true, OutT>(tA, tB, tA2, tB2, p, stages, s)
                    : launch_instance<KIND, 128, false, OutT>(tA, tB, tA2, tB2, p, stages, s);
  }
  return KCG_UNSUPPORTED;
}


template <int KIND, int BN, bool B_KMAJOR, typename OutT>
kcg_status_t launch_pair_instance(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
                                  const CUtensorMap& tB2, const GemmParams& p_in, int stages_req,
                                  cudaStream_t stream, void* sk_ws, size_t sk_ws_bytes) {
  GemmParams p = p_in;
  using Cfg = PairCfg<KIND, BN>;
  constexpr int STAGES = Cfg::MAX_STAGES > 8 ? 8 : Cfg::MAX_STAGES;
  static_assert(STAGES >= 2, "need at least two pipeline stages");
  if (stages_req != 0 && stages_req != STAGES) return KCG_UNSUPPORTED;
  auto kern = gemm_pair_kernel<KIND, BN, STAGES, B_KMAJOR, OutT>;
  constexpr int smem = STAGES * Cfg::STAGE_BYTES + Cfg::CTRL_BYTES + Cfg::EPI_BYTES + 1024;
  static_assert(smem <= SMEM_LIMIT, "shared memory budget");
  KCG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * p.tiles_n * p.batch;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(2);
  int max_clusters = 0;
  KCG_CUDA_TRY(cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg));
  if (max_clusters <= 0) return KCG_UNSUPPORTED;
  int pairs = tiles < max_clusters ? tiles : max_clusters;
  // shared-K tail, when the caller's workspace has room for the partial accumulators
  const SkPlan pl = plan_shared_k(tiles, (p.K + Cfg::BK - 1) / Cfg::BK, max_clusters, BN);
  if (pl.tiles > 0 && sk_ws && sk_ws_bytes >= pl.bytes) {
    int* counters = nullptr;
    const kcg_status_t st = sk_counters_ptr(&counters);
    if (st != KCG_OK) return st;
    p.sk_tiles = pl.tiles;
    p.sk_units = pl.units;
    p.sk_share = pl.share;
    p.sk_span = pl.span;
    p.sk_maxc = pl.maxc;
    p.sk_partial = static_cast<float*>(sk_ws);
    p.sk_extent = pl.bytes;
    p.sk_count = counters + (g_sk_row.fetch_add(1) % SK_ROWS) * SK_ROW_INTS;
    pairs = tiles >= max_clusters ? max_clusters : pl.units;
  }
  cfg.gridDim = dim3(2 * pairs);
  cfg.numAttrs = (KIND == 2 && !p.accum) ? 2 : 1;   // 3xTF32: overlap the set-up with the residual pass before it
  KCG_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tA, tB, tA2, tB2, p));
  g_launches.fetch_add(1);
  return KCG_OK;
}

template <int KIND, typename OutT>
kcg_status_t dispatch_pair_shape(int bn, bool b_kmajor, const CUtensorMap& tA, const CUtensorMap& tB,
                                 const CUtensorMap& tA2, const CUtensorMap& tB2, const GemmParams& p,
                                 int stages, cudaStream_t s, void* sk_ws, size_t sk_bytes) {
  if (bn == 256) {
    return b_kmajor ? launch_pair_instance<KIND, 256, true, OutT>(tA, tB, tA2, tB2, p, stages, s, sk_ws, sk_bytes)
                    : launch_pair_instance<KIND, 256, false, OutT>(tA, tB, tA2, tB2, p, stages, s, sk_ws, sk_bytes);
  }
  if (bn == 128) {
    return b_kmajor ? launch_pair_instance<KIND, 128, true, OutT>(tA, tB, tA2, tB2, p, stages, s, sk_ws, sk_bytes)
                    : launch_pair_instance<KIND, 128, false, OutT>(tA, tB, tA2, tB2, p, stages, s, sk_ws, sk_bytes);
  }
  return KCG_UNSUPPORTED;
}

}  // namespace

// Kernel variant and tile width for a descriptor.  Defaults, from interleaved measurements on one
// B200 under its 1000 W power cap:
//  - short launches (< ~4 TFLOP of work) run faster on CTA pairs (bf16 4096^3 +8 %, 8192^3 +4 %;
//    3xTF32 with 128-wide tiles +15..30 % on 4096x2048x1024 and 4096^3);
//  - long launches are power-limited, and there the pair kernel sustains lower clocks
//    (bf16 16384^3 -3.5 %, 32768^3 -19 %), so single CTAs with 256-wide tiles are used.
static void resolve_variant(const kcg_gemm_desc* d, int* bn, bool* pair_mode, long long batch = 1) {
  const double work = 2.0 * static_cast<double>(d->M) * static_cast<double>(d->N) * static_cast<double>(d->K) *
                      static_cast<double>(batch);
  const bool small_job = work < 4e12;
  *bn = d->tile_n;
  if (*bn == 0) *bn = (d->precision == KCG_PREC_3XTF32 && small_job) ? 128 : 256;
  *pair_mode = d->cta_group == 2 || (d->cta_group == 0 && d->M > BM && small_job);
  // Products of at most one wave of 128 x 128 tiles (bf16 / TF32): single CTAs on those tiles put
  // one tile on every SM at once; wider tiles or CTA pairs leave most SMs idle and lengthen the
  // one main loop there is (bf16, cold L2: 1024^3 14.3 us against 23.4, 1536^3 17.2 against 26.6,
  // 512^3 11.0 against 14.2; at 2048^3, two waves, the wider pair tiles win again).  The 3xTF32
  // path keeps its pairs: there the shared-K split of the few tiles is what fills the SMs.
  if (d->tile_n == 0 && d->cta_group == 0 && d->precision != KCG_PREC_3XTF32) {
    const long long t128 = ((d->M + BM - 1) / BM) * ((d->N + 127) / 128) * batch;
    if (t128 <= 148) {
      *bn = 128;
      *pair_mode = false;
    }
  }
}

// The plan itself, for tests: out = {tail tiles, units, share, span, max contributors per tile}.
void gemm_shared_k_plan_impl(int tiles, int num_kb, int pairs, int bn, int* out) {
  const SkPlan pl = plan_shared_k(tiles, num_kb, pairs, bn);
  out[0] = pl.tiles;
  out[1] = pl.units;
  out[2] = pl.share;
  out[3] = pl.span;
  out[4] = pl.maxc;
}

// Zeroes the arrival counters on the current device (after a launch that ended on a bounded wait;
// the device is idle when this is called).
void gemm_reset_shared_k_counters() {
  int* counters = nullptr;
  if (sk_counters_ptr(&counters) == KCG_OK) cudaMemset(counters, 0, sizeof(int) * SK_ROWS * SK_ROW_INTS);
  if (done_counters_ptr(&counters) == KCG_OK) cudaMemset(counters, 0, sizeof(int) * DONE_ROWS * DONE_STRIDE);
}

// Tail tiles the shared-K plan covers for this descriptor on 74 CTA pairs (0 = no shared-K tail).
int gemm_shared_k_tiles_impl(const kcg_gemm_desc* d) {
  if (!d || d->M <= 0 || d->N <= 0 || d->K <= 0) return 0;
  if (d->M > 0x7FFFFFFF || d->N > 0x7FFFFFFF || d->K > 0x7FFFFFFF) return 0;
  int bn = 0;
  bool pair_mode = false;
  resolve_variant(d, &bn, &pair_mode);
  if (!pair_mode || (bn != 128 && bn != 256)) return 0;
  const int bk = d->precision == KCG_PREC_BF16 ? 64 : 32;
  const long long tiles = ((d->M + 2 * BM - 1) / (2 * BM)) * ((d->N + bn - 1) / bn);
  if (tiles > 0x7FFFFFFF) return 0;
  return plan_shared_k(static_cast<int>(tiles), static_cast<int>((d->K + bk - 1) / bk), 74, bn).tiles;
}

// Launch geometry for a descriptor on a B200 (148 SMs / 74 CTA pairs):
// out = {grid, threads per CTA, cluster size, tile rows, tile columns, output tiles}.
kcg_status_t gemm_launch_geometry_impl(const kcg_gemm_desc* d, int* out) {
  if (!d || !out) return KCG_BAD_ARGUMENT;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0 || d->M > 0x7FFFFFFF || d->N > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  int bn = 0;
  bool pair_mode = false;
  resolve_variant(d, &bn, &pair_mode);
  if (bn != 128 && bn != 256) return KCG_UNSUPPORTED;
  const int tile_m = pair_mode ? 2 * BM : BM;
  const long long tiles = ((d->M + tile_m - 1) / tile_m) * ((d->N + bn - 1) / bn);
  if (tiles > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  const int units = pair_mode ? 74 : 148;
  long long resident = tiles < units ? tiles : units;
  if (pair_mode && tiles < units) {
    // fewer tiles than pairs: the shared-K plan may spread them over more pairs
    const int bk = d->precision == KCG_PREC_BF16 ? 64 : 32;
    const SkPlan pl = plan_shared_k(static_cast<int>(tiles), static_cast<int>((d->K + bk - 1) / bk), units, bn);
    if (pl.tiles > 0 && pl.units > resident) resident = pl.units;
  }
  out[0] = static_cast<int>(pair_mode ? 2 * resident : resident);
  out[1] = pair_mode ? GEMM_THREADS : GEMM1_THREADS;
  out[2] = pair_mode ? 2 : 1;
  out[3] = tile_m;
  out[4] = bn;
  out[5] = static_cast<int>(tiles);
  return KCG_OK;
}

// bytes of the 3xTF32 residual arrays at the head of the workspace
static size_t gemm_lo_bytes(const kcg_gemm_desc* d) {
  if (d->precision != KCG_PREC_3XTF32) return 0;
  return pad256(static_cast<size_t>(d->M) * d->K * 4) + pad256(static_cast<size_t>(d->K) * d->N * 4);
}

size_t gemm_workspace_impl(const kcg_gemm_desc* d) {
  if (!d) return 0;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return 0;
  if (d->M > 0x7FFFFFFF || d->N > 0x7FFFFFFF || d->K > 0x7FFFFFFF) return 0;
  size_t need = gemm_lo_bytes(d);
  // room for the partial accumulators of the shared-K tail, planned for the 74 CTA pairs of a
  // B200 (the launch plans again for the device it runs on and goes without if this is too small)
  int bn = 0;
  bool pair_mode = false;
  resolve_variant(d, &bn, &pair_mode);
  if (pair_mode && (bn == 128 || bn == 256)) {
    const int bk = d->precision == KCG_PREC_BF16 ? 64 : 32;
    const long long tiles = ((d->M + 2 * BM - 1) / (2 * BM)) * ((d->N + bn - 1) / bn);
    if (tiles <= 0x7FFFFFFF)
      need += plan_shared_k(static_cast<int>(tiles), static_cast<int>((d->K + bk - 1) / bk), 74, bn).bytes;
  }
  return need;
}

// bytes of the residual arrays of a batched 3xTF32 product: an operand shared by all entries
// (stride 0) is split once
static size_t batched_lo_bytes(const kcg_gemm_desc* d, long long batch, long long stride_a, long long stride_b) {
  if (d->precision != KCG_PREC_3XTF32) return 0;
  const size_t ea = stride_a == 0 ? 1 : static_cast<size_t>(batch), eb = stride_b == 0 ? 1 : static_cast<size_t>(batch);
  return pad256(ea * d->M * d->K * 4) + pad256(eb * d->K * d->N * 4);
}

size_t gemm_batched_workspace_impl(const kcg_gemm_desc* d, long long batch, long long stride_a, long long stride_b) {
  if (!d || batch <= 0) return 0;
  if (batch == 1) return gemm_workspace_impl(d);
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return 0;
  if (d->M > 0x7FFFFFFF || d->N > 0x7FFFFFFF || d->K > 0x7FFFFFFF) return 0;
  size_t need = batched_lo_bytes(d, batch, stride_a, stride_b);
  int bn = 0;
  bool pair_mode = false;
  resolve_variant(d, &bn, &pair_mode, batch);
  if (pair_mode && (bn == 128 || bn == 256)) {
    const int bk = d->precision == KCG_PREC_BF16 ? 64 : 32;
    const long long tiles = ((d->M + 2 * BM - 1) / (2 * BM)) * ((d->N + bn - 1) / bn) * batch;
    if (tiles <= 0x7FFFFFFF)
      need += plan_shared_k(static_cast<int>(tiles), static_cast<int>((d->K + bk - 1) / bk), 74, bn).bytes;
  }
  return need;
}

// `batch` independent products described by `d`; operand i at base + i * stride (elements; 0 = the
// operand is shared).  One launch: the batch entry is the outermost part of the tile index and the
// third coordinate of the tensor maps, so a tile never runs into the next entry's rows and ragged
// shapes are zero-filled per entry.
kcg_status_t gemm_batched_launch_impl(const kcg_gemm_desc* d, long long batch, long long stride_a, long long stride_b,
                                      long long stride_c, const void* A, const void* B, void* C, void* ws,
                                      size_t ws_bytes, cudaStream_t stream) {
  if (!d || !A || !B || !C) return KCG_BAD_ARGUMENT;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return KCG_BAD_SHAPE;
  if (d->M > 0x7FFFFFFF || d->N > 0x7FFFFFFF || d->K > 0x7FFFFFFF) return KCG_BAD_SHAPE;
  if (batch <= 0 || batch > 0x7FFFFFFF || stride_a < 0 || stride_b < 0 || stride_c < 0) return KCG_BAD_SHAPE;
  const bool b_kmajor = d->b_layout == KCG_COL_MAJOR;
  if (d->b_layout != KCG_ROW_MAJOR && d->b_layout != KCG_COL_MAJOR) return KCG_UNSUPPORTED;
  if (d->lda < d->K || d->ldc < d->N || d->ldb < (b_kmajor ? d->K : d->N)) return KCG_BAD_SHAPE;
  int kind;
  if (d->precision == KCG_PREC_BF16) {
    if (d->dtype_in != KCG_BF16) return KCG_UNSUPPORTED;
    if (d->dtype_out != KCG_BF16 && d->dtype_out != KCG_F32) return KCG_UNSUPPORTED;
    kind = 0;
  } else if (d->precision == KCG_PREC_TF32 || d->precision == KCG_PREC_3XTF32) {
    if (d->dtype_in != KCG_F32 || d->dtype_out != KCG_F32) return KCG_UNSUPPORTED;
    kind = d->precision == KCG_PREC_TF32 ? 1 : 2;
  } else {
    return KCG_UNSUPPORTED;
  }
  if (d->epilogue != KCG_EPI_NONE && d->epilogue != KCG_EPI_RELU) return KCG_UNSUPPORTED;
  if (d->n_peers < 0 || d->n_peers > 8) return KCG_BAD_ARGUMENT;
  const int es = kind == 0 ? 2 : 4;
  const int os = d->dtype_out == KCG_BF16 ? 2 : 4;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return KCG_BAD_ALIGN;
  if ((d->lda * es) % 16 || (d->ldb * es) % 16 || (d->ldc * os) % 16) return KCG_BAD_ALIGN;
  if (batch > 1) {
    if ((stride_a * es) % 16 || (stride_b * es) % 16 || (stride_c * os) % 16) return KCG_BAD_ALIGN;
    if (stride_c == 0) return KCG_BAD_SHAPE;      // every entry needs its own C
  }
  const long long batch_a = (batch > 1 && stride_a != 0) ? batch : 1;
  const long long batch_b = (batch > 1 && stride_b != 0) ? batch : 1;
  for (int i = 0; i < d->n_peers; ++i)
    if (!d->peer_c[i] || !aligned16(d->peer_c[i])) return KCG_BAD_ALIGN;
  if (d->mc_c) {
    // the multicast path stores whole 128-byte row segments only
    if (!aligned16(d->mc_c) || (d->N * os) % 128) return KCG_BAD_ALIGN;
  }
  if (d->n_done_flags < 0 || d->n_done_flags > 9) return KCG_BAD_ARGUMENT;
  for (int i = 0; i < d->n_done_flags; ++i)
    if (!d->done_flags[i] || (reinterpret_cast<uintptr_t>(d->done_flags[i]) & 3u)) return KCG_BAD_ALIGN;
  int bn = 0;
  bool pair_mode = false;
  resolve_variant(d, &bn, &pair_mode, batch);
  if (bn != 128 && bn != 256) return KCG_UNSUPPORTED;
  if (d->cta_group != 0 && d->cta_group != 1 && d->cta_group != 2) return KCG_UNSUPPORTED;
  {
    const long long tm = pair_mode ? (d->M + 2 * BM - 1) / (2 * BM) : (d->M + BM - 1) / BM;
    if (tm * ((d->N + bn - 1) / bn) * batch > 0x7FFFFFFFll) return KCG_BAD_SHAPE;
  }

  const void* pa = A;
  const void* pb = B;
  const void* pa2 = A;
  const void* pb2 = B;
  long long lda = d->lda, ldb = d->ldb;
  long long lda2 = d->lda, ldb2 = d->ldb;  // leading dimensions of the residual arrays
  long long sa_elems = stride_a, sb_elems = stride_b;      // entry strides of the operands ...
  long long sa2_elems = stride_a, sb2_elems = stride_b;    // ... and of the residual arrays
  const size_t lo_bytes = batched_lo_bytes(d, batch, batch_a == 1 ? 0 : stride_a, batch_b == 1 ? 0 : stride_b);
  if (kind == 2) {
    const size_t need = lo_bytes;
    if (!ws || ws_bytes < need || !aligned16(ws)) return KCG_BAD_WORKSPACE;
    if ((d->K % 4) || (d->N % 4)) return KCG_BAD_ALIGN;
    const size_t a = pad256(static_cast<size_t>(batch_a) * d->M * d->K * 4);
    float* a_lo = static_cast<float*>(ws);
    float* b_lo = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + a);
    const int sms = device_sm_count();
    const long long b_rows = b_kmajor ? d->N : d->K;
    const long long b_cols = b_kmajor ? d->K : d->N;
    SplitArgs sa{static_cast<const float*>(A), a_lo, batch_a * d->M, static_cast<int>(d->K / 4), d->lda, d->M, stride_a};
    SplitArgs sb{static_cast<const float*>(B), b_lo, batch_b * b_rows, static_cast<int>(b_cols / 4), d->ldb, b_rows, stride_b};
    split_lo_kernel<<<sms * 4, 256, 0, stream>>>(sa, sb);
    g_launches.fetch_add(1);
    KCG_CUDA_TRY(cudaGetLastError());
    pa2 = a_lo;
    pb2 = b_lo;
    lda2 = d->K;
    ldb2 = b_cols;
    sa2_elems = d->M * d->K;
    sb2_elems = b_rows * b_cols;
  }
  // entry strides of the tensor maps (any valid value when the operand has a single entry)
  if (batch_a == 1) sa_elems = sa2_elems = d->M * lda;
  if (batch_b == 1) sb_elems = sb2_elems = (b_kmajor ? d->N : d->K) * ldb;

  // One launch over the K range [k0, k0 + kc): the tensor maps start k0 elements into the operands.
  auto launch_range = [&](long long k0, long long kc, int accum, bool relu_now, bool relu_late) -> kcg_status_t {
    using Cfg0 = GemmCfg<0, 128>;
    (void)sizeof(Cfg0);
    const CUtensorMapDataType dt =
        kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const uint32_t bk = 128 / es;
    CUtensorMap tA, tB, tA2, tB2;
    {
      const uint64_t dims[3] = {static_cast<uint64_t>(kc), static_cast<uint64_t>(d->M), static_cast<uint64_t>(batch_a)};
      const uint64_t strides[2] = {static_cast<uint64_t>(lda) * es, static_cast<uint64_t>(sa_elems) * es};
      const uint64_t strides2[2] = {static_cast<uint64_t>(lda2) * es, static_cast<uint64_t>(sa2_elems) * es};
      const uint32_t box[3] = {bk, BM, 1};
      kcg_status_t st = encode_tmap(&tA, dt, 3, static_cast<const uint8_t*>(pa) + k0 * es, dims, strides, box);
      if (st != KCG_OK) return st;
      st = encode_tmap(&tA2, dt, 3, static_cast<const uint8_t*>(pa2) + k0 * es, dims, strides2, box);
      if (st != KCG_OK) return st;
    }
    {
      uint64_t dims[3];
      uint32_t box[3];
      dims[2] = static_cast<uint64_t>(batch_b);
      box[2] = 1;
      if (b_kmajor) {  // B stored [N, K]
        dims[0] = static_cast<uint64_t>(kc);
        dims[1] = d->N;
        box[0] = bk;
        box[1] = pair_mode ? bn / 2 : bn;
      } else {  // B stored [K, N]
        dims[0] = d->N;
        dims[1] = static_cast<uint64_t>(kc);
        box[0] = 128 / es;
        box[1] = bk;
      }
      const uint64_t strides[2] = {static_cast<uint64_t>(ldb) * es, static_cast<uint64_t>(sb_elems) * es};
      const CUtensorMapSwizzle sw = (!b_kmajor && es == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                           : CU_TENSOR_MAP_SWIZZLE_128B;
      const uint64_t strides2[2] = {static_cast<uint64_t>(ldb2) * es, static_cast<uint64_t>(sb2_elems) * es};
      kcg_status_t st = encode_tmap(&tB, dt, 3, static_cast<const uint8_t*>(pb) + (b_kmajor ? k0 : k0 * ldb) * es, dims, strides, box, sw);
      if (st != KCG_OK) return st;
      st = encode_tmap(&tB2, dt, 3, static_cast<const uint8_t*>(pb2) + (b_kmajor ? k0 : k0 * ldb2) * es, dims, strides2, box, sw);
      if (st != KCG_OK) return st;
    }

  #ifdef KCG_DEBUG_BOUNDS
    // Every tensor-map coordinate the kernels will issue, checked on the host: the innermost
    // coordinate times the element size must be a multiple of 16 bytes (nothing checks that before
    // the copy runs, and a violation loses the context), no coordinate is negative, and the tiles
    // cover the whole problem.  Coordinates beyond an extent are legal for loads (zero fill).
    {
      const long long tm = pair_mode ? 2 * BM : BM;
      const long long tiles_m = (d->M + tm - 1) / tm, tiles_n = (d->N + bn - 1) / bn, kbs = (kc + bk - 1) / bk;
      bool ok = tiles_m * tm >= d->M && tiles_n * bn >= d->N && kbs * bk >= kc;
      ok = ok && (static_cast<long long>(bk) * es) % 16 == 0;            // k0 = kb * bk for the K-major operands
      if (!b_kmajor) {
        const long long group = 128 / es;                                 // x = n0 + j * group for row-major B
        ok = ok && (static_cast<long long>(bn) * es) % 16 == 0 && (group * es) % 16 == 0 &&
             ((pair_mode ? bn / 2 : bn) * static_cast<long long>(es)) % 16 == 0;
      }
      if (!ok) {
        std::fprintf(stderr, "kcg: bounds build: tile / tensor-map coordinate self-check failed\n");
        return KCG_BAD_ALIGN;
      }
    }
  #endif
    GemmParams p;
    p.C = C;
    p.M = static_cast<int>(d->M);
    p.N = static_cast<int>(d->N);
    p.K = static_cast<int>(kc);
    p.ldc = d->ldc;
    p.batch = static_cast<int>(batch);
    p.a_bz = batch_a > 1 ? 1 : 0;
    p.b_bz = batch_b > 1 ? 1 : 0;
    p.c_bstride = batch > 1 ? stride_c : 0;
    // extent of C for the bounds-checking build: up to the last element of the last entry's last row
    p.c_extent = (static_cast<unsigned long long>(batch - 1) * (batch > 1 ? stride_c : 0) +
                  static_cast<unsigned long long>(d->M - 1) * d->ldc + d->N) * os;
    if (const unsigned long long cap = debug_extent_limit()) p.c_extent = p.c_extent < cap ? p.c_extent : cap;
    p.sk_extent = 0;
    p.bounds_detail = nullptr;
    debug_bounds_detail_ptr(&p.bounds_detail);
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.N + bn - 1) / bn;
    p.group_m = d->group_m > 0 ? d->group_m : 16;
    p.relu = relu_now ? 1 : 0;
    p.accum = accum;
    p.relu_late = relu_late ? 1 : 0;
    kcg_status_t st = device_status_ptr(&p.status);
    if (st != KCG_OK) return st;
    const uint32_t spin = g_spin_limit.load();
    p.spin = spin ? spin : KCG_SPIN_LIMIT;
    p.n_peers = d->n_peers;
    for (int i = 0; i < 8; ++i) p.peers[i] = i < d->n_peers ? d->peer_c[i] : nullptr;
    p.mc = d->mc_c;
    p.n_flags = d->n_done_flags;
    p.flag_value = d->done_value;
    for (int i = 0; i < 9; ++i) p.flags[i] = i < d->n_done_flags ? static_cast<uint32_t*>(d->done_flags[i]) : nullptr;
    p.done_counter = nullptr;
    if (p.n_flags > 0) {
      int* counters = nullptr;
      st = done_counters_ptr(&counters);
      if (st != KCG_OK) return st;
      p.done_counter = counters + (g_done_row.fetch_add(1) % DONE_ROWS) * DONE_STRIDE;
    }
    p.sk_tiles = p.sk_units = p.sk_share = p.sk_span = p.sk_maxc = 0;
    p.sk_partial = nullptr;
    p.sk_count = nullptr;

    if (pair_mode) {
      // what follows the residual arrays in the workspace is free for the shared-K tail
      void* sk_ws = (ws && aligned16(ws) && ws_bytes > lo_bytes) ? static_cast<uint8_t*>(ws) + lo_bytes : nullptr;
      const size_t sk_bytes = sk_ws ? ws_bytes - lo_bytes : 0;
      if (kind == 0) {
        if (d->dtype_out == KCG_BF16)
          return dispatch_pair_shape<0, __nv_bfloat16>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages, stream, sk_ws,
                                                       sk_bytes);
        return dispatch_pair_shape<0, float>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages, stream, sk_ws, sk_bytes);
      }
      if (kind == 1)
        return dispatch_pair_shape<1, float>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages, stream, sk_ws, sk_bytes);
      return dispatch_pair_shape<2, float>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages, stream, sk_ws, sk_bytes);
    }
    if (kind == 0) {
      if (d->dtype_out == KCG_BF16)
        return dispatch_shape<0, __nv_bfloat16>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages,
                                                stream);
      return dispatch_shape<0, float>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages, stream);
    }
    if (kind == 1) return dispatch_shape<1, float>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages, stream);
    return dispatch_shape<2, float>(bn, b_kmajor, tA, tB, tA2, tB2, p, d->stages, stream);
  };

  // The tensor core adds into its fp32 accumulator with truncation, so the 3xTF32 result drifts from
  // the exact product in proportion to K (about 1.8e-5 of max|C| per 2048 of K with uniform inputs)
  // and would leave the 1e-4 contract near K = 12000.  Longer products are therefore run as
  // several launches over K ranges of 4096; each launch after the first adds its tile to C in the
  // epilogue with round-to-nearest fp32 adds (ReLU on the last one), which resets the drift per
  // range.  Costs one extra read and write of C per range.
  constexpr long long K_RANGE = 4096, K_WHOLE = 8192;
  const bool relu = d->epilogue == KCG_EPI_RELU;
  if (kind == 2 && batch == 1 && d->K > K_WHOLE && d->n_peers == 0 && !d->mc_c && d->n_done_flags == 0) {
    const long long ranges = (d->K + K_RANGE - 1) / K_RANGE;
    for (long long r = 0; r < ranges; ++r) {
      const long long k0 = r * K_RANGE, kc = std::min<long long>(K_RANGE, d->K - k0);
      const bool last = r + 1 == ranges;
      const kcg_status_t st = launch_range(k0, kc, r > 0 ? 1 : 0, false, last && relu && r > 0);
      if (st != KCG_OK) return st;
    }
    return KCG_OK;
  }
  return launch_range(0, d->K, 0, relu, false);
}

kcg_status_t gemm_launch_impl(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                              void* ws, size_t ws_bytes, cudaStream_t stream) {
  return gemm_batched_launch_impl(d, 1, 0, 0, 0, A, B, C, ws, ws_bytes, stream);
}

// Device address of g_static_scratch on the current device.  Looked up once per device, with
// that device current (the symbol has one instance per device).
static kcg_status_t static_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* cache[64] = {};
  int dev = 0;
  KCG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return KCG_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    KCG_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    if (!p) return KCG_CUDA_ERROR;
    cache[dev] = p;
  }
  *out = cache[dev];
  return KCG_OK;
}

kcg_status_t gemm_launch_static_impl(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                                     cudaStream_t stream) {
  if (!d) return KCG_BAD_ARGUMENT;
  if (d->precision != KCG_PREC_3XTF32) return KCG_UNSUPPORTED;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return KCG_BAD_SHAPE;
  const size_t need = gemm_lo_bytes(d);
  if (need > STATIC_SCRATCH_BYTES) {
    std::fprintf(stderr,
                 "kcg: kcg_gemm_launch_static: %lld x %lld x %lld needs %zu bytes of scratch, the "
                 "built-in scratch holds %zu; use kcg_gemm_launch with a workspace\n",
                 static_cast<long long>(d->M), static_cast<long long>(d->N),
                 static_cast<long long>(d->K), need, STATIC_SCRATCH_BYTES);
    return KCG_TOO_LARGE;
  }
  void* scratch = nullptr;
  kcg_status_t st = static_scratch_ptr(&scratch);
  if (st != KCG_OK) return st;
  // The split pass overwrites every byte of scratch the GEMM then reads, so nothing left by an
  // earlier call is ever consumed and nothing has to be cleared.
  // Exactly the residual arrays are handed on, so the shared-K tail (which would use the rest of
  // the scratch for partial accumulators) stays off on this entry.
  return gemm_launch_impl(d, A, B, C, scratch, need, stream);
}

}  // namespace kcg
