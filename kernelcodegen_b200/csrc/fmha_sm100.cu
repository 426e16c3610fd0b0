// O = softmax(scale * Q.K^T [causal]) . V on sm_100a; one CTA per (batch*head, 256 queries).
//
// The computation is the reference's three-operator graph (test/test.cc:88-90):
// BatchedMatmul(Q, K colMajor) (src/Frontend/Operators.cc:353-414), Softmax over the last axis
// (:474-536) and BatchedMatmul(P, V).  The reference's FMHAOptimizer fuses that chain into a
// FlashAttention-2 style kernel with scalar FFMA outer products and shuffle reductions
// (src/Optimizer/Optimizer.cc:1079-1333); here both contractions run on tcgen05 tensor cores
// and the online softmax works on rows read straight out of TMEM.
//
// A CTA owns two 128-query tiles that share every K_j / V_j block (128 keys) it loads:
//
//   warp 0        TMA producer : Q tiles once, then K_j / V_j through 2-stage rings
//   warp 1        UMMA issuer  : per block j and tile t: S_t = Q_t.K_j^T -> TMEM, then, once the
//                                softmax warps have turned S_t into P_t in place (bf16, same
//                                TMEM columns), PV_t = P_t.V_j -> TMEM with P_t as the TMEM
//                                operand.  Issue order PV_0(j), S_0(j+1), PV_1(j), S_1(j+1) keeps
//                                the tensor core busy with one tile while the other tile's
//                                softmax runs.
//   warps 4..7    softmax, tile 0 } thread t owns query row t of its tile: tcgen05.ld of its S
//   warps 8..11   softmax, tile 1 } row (pass 1: running max; pass 2: exp2 -> P), running sum,
//                                   O += rescaled PV_t in registers, final O / l -> global.
//
// Row max / row sum are thread-local (one TMEM lane = one query row), so no cross-lane step
// exists.  Registers are re-balanced with setmaxnreg: the softmax warpgroups hold an O row of D
// floats per thread, the producer/issuer warpgroup needs next to nothing.
//
// fp32 inputs with head dimension 64 (TF = true) run both contractions as TF32 products straight
// from the fp32 tiles: Q and K as K-major 128B-swizzled panels of 32 floats, V as an MN-major
// operand in the 32-byte-atom swizzle, P written back over S as fp32 (the tensor core truncates
// fp32 operands to TF32 itself).  No conversion pass, and three more mantissa bits than bf16.
// Other fp32 shapes are rounded to bf16 by a separate pass into the workspace first.
//
// Online softmax: m_j = max(m_{j-1}, rowmax(S_j)), alpha_j = exp(scale*(m_{j-1}-m_j)),
// l_j = alpha_j*l_{j-1} + rowsum(P_j), O_j = alpha_j*O_{j-1} + P_j.V_j, out = O_n / l_n --
// mathematically the reference's exp(x)/sum(exp(x)) (no max subtraction there), evaluated
// without overflow.
#include "common.cuh"
#include "ptx.cuh"

namespace kcg {

namespace {

constexpr int FM_THREADS = 384;
constexpr int BQ = 128;        // query rows per tile
constexpr int QTILES = 2;      // tiles per CTA
constexpr int BKV = 128;       // keys per block

struct FmhaParams {
  void* O;
  int Sq, Skv;
  int causal;
  int out_bf16;
  float scale_log2;  // scale * log2(e)
  int* status;
  uint32_t spin;
  int after_cast;    // the inputs come from the cast launch just before (programmatic dependent launch)
  int n_qp;          // 256-query tile pairs per (batch, head)
  int bh_total;      // batch * heads
  int bh_group;      // (batch, head) pairs walked together, see the block-index mapping in the kernel
  int bh_small;      // how many of the groups (the first ones) hold one pair fewer
  unsigned long long o_extent;          // bounds-checking build: bytes of O
  unsigned long long* bounds_detail;
};

template <int D, bool TF>
struct FmhaCfg {
  static constexpr int ES = TF ? 4 : 2;               // bytes per operand element
  static constexpr int TILE_BYTES = 128 * D * ES;     // Q_t, K_j, V_j tile: 128 rows x D elements
  static constexpr int PANEL_BYTES = 128 * 128;       // 128 rows x 128 bytes (one swizzle panel)
  static constexpr int PANEL_ELEMS = 128 / ES;        // 64 bf16 or 32 fp32 per panel row
  static constexpr int DPANELS = D / PANEL_ELEMS;
  static constexpr int UMMA_K = 32 / ES;              // elements of K per UMMA: 16 bf16 or 8 fp32
  static constexpr int SMEM_DATA = QTILES * TILE_BYTES + 2 * TILE_BYTES /*K*/ + 2 * TILE_BYTES /*V*/;
  static constexpr int SMEM_TOTAL = SMEM_DATA + 1024 /*ctrl*/ + 1024 /*align slack*/;
  static constexpr int TMEM_COLS = 512;               // S0 | S1 | PV0 | PV1
};

// Register re-balancing.  The CTA is launched with 384 threads x 168 registers = 64512; the
// pool never grows, so after the change the three warpgroups must still fit in 64512:
// 128 x 96 + 256 x 200 = 63488.  (The producer / issuer warps spill below 96 registers -- at 56
// they cost 8 % -- and the softmax warps need fewer than 190.  setmaxnreg.inc waits, unbounded,
// for registers to be released: a budget that does not add up hangs the CTA.)
static_assert(128 * 96 + 256 * 200 <= 384 * 168, "setmaxnreg budget must fit the launch allocation");
__device__ __forceinline__ void reg_dealloc_96() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 96;" ::: "memory");
}
__device__ __forceinline__ void reg_alloc_200() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 200;" ::: "memory");
}

// 2^x of a pair; POLY eighths of the pairs (a fixed pattern over the pair index, so that the two
// kinds of instruction interleave) take it from the FMA-pipe cubic, the rest from the MUFU unit.
// Measured: with head dimension 64 in bf16 the tensor core needs half as long per block as the
// MUFU unit and a share of 3/8 gains 9 %; with head dimension 128, or TF32 operands, the two
// are level and any share costs 1-9 %.
template <int POLY>
__device__ __forceinline__ float2 exp2_pair(int g, int pi, float2 x) {
  if (((pi * 5 + g * 3) & 7) < POLY) {
    x.x = fmaxf(x.x, -125.f);   // masked keys (-inf) and far tails end as 2^-125, nothing in the sums
    x.y = fmaxf(x.y, -125.f);
    return ex2_poly2(x);
  }
  x.x = ex2_approx(x.x);
  x.y = ex2_approx(x.y);
  return x;
}

template <int D, bool TF>
__global__ void __launch_bounds__(FM_THREADS, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FmhaParams p) {
  using Cfg = FmhaCfg<D, TF>;
  constexpr int TILE = Cfg::TILE_BYTES;
  constexpr int PANEL = Cfg::PANEL_BYTES;
  constexpr int DPANELS = Cfg::DPANELS;
  constexpr int PW = Cfg::PANEL_ELEMS;
  constexpr int UK = Cfg::UMMA_K;
  constexpr int POLY = (!TF && D == 64) ? 3 : 0;     // eighths of the exponentials on the FMA pipe
  constexpr uint32_t FMT = TF ? UMMA_FMT_TF32 : UMMA_FMT_BF16;
  constexpr uint32_t IDESC_S = make_idesc(FMT, BQ, BKV, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc(FMT, BQ, D, 0, 1);
  constexpr uint32_t TM_S = 0, TM_O = 256;            // + 128 * tile

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t sQ = base;                           // [QTILES]
  const uint32_t sK = sQ + QTILES * TILE;             // [2]
  const uint32_t sV = sK + 2 * TILE;                  // [2]
  const uint32_t ctrl_u = sV + 2 * TILE;
  uint8_t* ctrl = gen_base + Cfg::SMEM_DATA;
  const uint32_t bar_q = ctrl_u;             // [2] one per tile
  const uint32_t bar_kfull = ctrl_u + 16;    // [2]
  const uint32_t bar_kempty = ctrl_u + 32;   // [2]
  const uint32_t bar_vfull = ctrl_u + 48;    // [2]
  const uint32_t bar_vempty = ctrl_u + 64;   // [2]
  const uint32_t bar_sfull = ctrl_u + 80;    // [2] per tile: S_t(j) complete in TMEM
  const uint32_t bar_pfull = ctrl_u + 96;    // [2] per tile: P_t(j) written, PV_t(j-1) consumed
  const uint32_t bar_pvfull = ctrl_u + 112;  // [2] per tile: PV_t(j) complete in TMEM
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(ctrl + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 132);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Block index -> (batch*head, query tile pair).  CTAs are handed to the SMs in index order as
  // earlier ones retire, so the order of the indices is the schedule.  Causal tile pairs differ
  // 32-fold in length at S = 8192: the (batch, head) pairs are walked in groups of `bh_group`, and
  // within a group the tile pairs of all its heads go longest first, so the launch ends on the
  // short ones (heads one after the other leave the long tile pairs of the last head to start
  // when most SMs are already idle: 86 % of the SM-time used at 32 heads, 98 % in groups of 8).
  // A group's K and V (bh_group heads) stay in L2 while its tile pairs run.
  // groups are of equal size up to one head: the first `bh_small` groups hold bh_group - 1 heads
  int idx = blockIdx.x, gsz = p.bh_group - 1, g0 = 0;
  const int small_items = p.bh_small * gsz * p.n_qp;
  if (idx >= small_items) {
    idx -= small_items;
    gsz = p.bh_group;
    g0 = p.bh_small * (p.bh_group - 1);
  }
  const int grp = idx / (gsz * p.n_qp);
  g0 += grp * gsz;
  const int rem = idx - grp * gsz * p.n_qp;
  const int bh = g0 + rem % gsz;
  const int qpair = p.causal ? (p.n_qp - 1 - rem / gsz) : (rem / gsz);
  const int q0 = qpair * (QTILES * BQ);
  const int shift = p.Skv - p.Sq;  // causal: query i sees keys j <= i + shift
  // number of key blocks tile t needs (0 when the tile starts beyond Sq)
  int n_kv_t[QTILES];
#pragma unroll
  for (int t = 0; t < QTILES; ++t) {
    int kv_end = p.Skv;
    if (p.causal) {
      const int lim = q0 + (t + 1) * BQ + shift;  // exclusive bound for the last row of the tile
      kv_end = lim < kv_end ? lim : kv_end;
      if (kv_end < 0) kv_end = 0;
    }
    n_kv_t[t] = (q0 + t * BQ < p.Sq) ? (kv_end + BKV - 1) / BKV : 0;
  }
  const int n_kv = n_kv_t[0] > n_kv_t[1] ? n_kv_t[0] : n_kv_t[1];

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q + 8 * i, 1);
      mbar_init(bar_kfull + 8 * i, 1);
      mbar_init(bar_kempty + 8 * i, 1);
      mbar_init(bar_vfull + 8 * i, 1);
      mbar_init(bar_vempty + 8 * i, 1);
      mbar_init(bar_sfull + 8 * i, 1);
      mbar_init(bar_pfull + 8 * i, 128);
      mbar_init(bar_pvfull + 8 * i, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    // This thread is also the TMA producer: the Q tiles and the first K / V block go out now and
    // are in flight while TMEM is allocated and the CTA synchronises.
    if (n_kv > 0) {
      // fp32 inputs, head dimension 128: the bf16 copies come from the launch just before this one
      if (p.after_cast) griddep_wait();
#pragma unroll
      for (int t = 0; t < QTILES; ++t) {
        if (n_kv_t[t] == 0) continue;
        mbar_expect_tx(bar_q + 8 * t, TILE);
#pragma unroll
        for (int dp = 0; dp < DPANELS; ++dp)
          tma_load_3d(sQ + t * TILE + dp * PANEL, &tmQ, bar_q + 8 * t, dp * PW, q0 + t * BQ, bh);
      }
      mbar_expect_tx(bar_kfull, TILE);
#pragma unroll
      for (int dp = 0; dp < DPANELS; ++dp) tma_load_3d(sK + dp * PANEL, &tmK, bar_kfull, dp * PW, 0, bh);
      mbar_expect_tx(bar_vfull, TILE);
#pragma unroll
      for (int dp = 0; dp < DPANELS; ++dp) tma_load_3d(sV + dp * PANEL, &tmV, bar_vfull, dp * PW, 0, bh);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
    reg_dealloc_96();
    if (warp == 0 && lane == 0 && n_kv > 0) {
      // ------------------------------- TMA producer -----------------------------------------
      // (block 0 and the Q tiles were issued before the CTA-wide synchronisation above)
      bool ok = true;
      for (int j = 1; j < n_kv && ok; ++j) {
        const int b = j & 1;
        const uint32_t par = ((j >> 1) & 1u) ^ 1u;
        ok = mbar_wait(bar_kempty + 8 * b, par, abort_flag, p.status, DEV_TIMEOUT_PRODUCER, p.spin);
        if (!ok) break;
        mbar_expect_tx(bar_kfull + 8 * b, TILE);
#pragma unroll
        for (int dp = 0; dp < DPANELS; ++dp)
          tma_load_3d(sK + b * TILE + dp * PANEL, &tmK, bar_kfull + 8 * b, dp * PW, j * BKV, bh);
        ok = mbar_wait(bar_vempty + 8 * b, par, abort_flag, p.status, DEV_TIMEOUT_PRODUCER, p.spin);
        if (!ok) break;
        mbar_expect_tx(bar_vfull + 8 * b, TILE);
#pragma unroll
        for (int dp = 0; dp < DPANELS; ++dp)
          tma_load_3d(sV + b * TILE + dp * PANEL, &tmV, bar_vfull + 8 * b, dp * PW, j * BKV, bh);
      }
      if (!ok) {
        // give copies already in flight time to land before shared memory is released
        for (int i = 0; i < 2; ++i)
          for (uint32_t it = 0; it < 4096u; ++it) {
            if (mbar_try_wait(bar_q + 8 * i, 0) & mbar_try_wait(bar_kfull + 8 * i, 0) &
                mbar_try_wait(bar_vfull + 8 * i, 0))
              break;
          }
      }
    } else if (warp == 1 && n_kv > 0) {
      // ------------------------------- UMMA issuer -------------------------------------------
      // all 32 lanes walk the loop and wait on the barriers; one elected lane issues
      bool ok = true;
      auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
        return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag, p.status, code, p.spin));
      };
      // The issuing thread has ~64 tensor-core clocks per UMMA to stay ahead of the pipe, so the
      // descriptors are built once; per instruction only the 16-byte-unit start address (low 14
      // bits of the descriptor, never overflowing: shared memory is < 256 KB) is advanced.
      const uint64_t q_desc0 = make_smem_desc(sQ, 16, 1024);
      const uint64_t k_desc0 = make_smem_desc(sK, 16, 1024);
      // V is the MN-major operand (head dimension contiguous): fp32 tiles use the 32-byte-atom
      // form of the 128B swizzle (4-row period, stride-byte-offset 512)
      const uint64_t v_desc0 = TF ? make_smem_desc(sV, PANEL, 512, SMEM_LAYOUT_SW128_ATOM32)
                                  : make_smem_desc(sV, PANEL, 1024);
      constexpr uint64_t TILE16 = TILE >> 4;
      auto issue_s = [&](int t, int j) {
        // S_t(j) = Q_t . K_j^T; the caller has waited for K_j and for the S_t buffer
        const uint64_t qd = q_desc0 + t * TILE16, kd = k_desc0 + (j & 1) * TILE16;
        const uint32_t d_tmem = tmem_base + TM_S + t * BKV;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / UK; ++ks) {   // 32 bytes of K per instruction, 4 per panel
            const uint64_t off = static_cast<uint64_t>(((ks >> 2) * PANEL + (ks & 3) * 32) >> 4);
            if (TF)
              umma_tf32_ss(d_tmem, qd + off, kd + off, IDESC_S, ks ? 1u : 0u);
            else
              umma_bf16_ss(d_tmem, qd + off, kd + off, IDESC_S, ks ? 1u : 0u);
          }
          umma_commit(bar_sfull + 8 * t);
        }
        __syncwarp();
      };
      auto issue_pv = [&](int t, int j) {
        // O_t (+)= P_t(j) . V_j with P_t in the TMEM columns of S_t (one instruction takes 8
        // columns: 16 bf16 keys, two per column, or 8 fp32 keys); the accumulator stays in TMEM
        // across blocks, the softmax warps rescale it in place when the row maximum moves.
        // V tile: groups of [128 keys x 128 bytes]; one instruction's keys are UK * 128 bytes.
        const uint64_t vd = v_desc0 + (j & 1) * TILE16;
        const uint32_t d_tmem = tmem_base + TM_O + t * 128;
        const uint32_t a_tmem = tmem_base + TM_S + t * BKV;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < BKV / UK; ++ks) {
            const uint64_t vk = vd + static_cast<uint64_t>((ks * UK * 128) >> 4);
            if (TF)
              umma_tf32_ts(d_tmem, a_tmem + ks * 8, vk, IDESC_PV, (j | ks) ? 1u : 0u);
            else
              umma_bf16_ts(d_tmem, a_tmem + ks * 8, vk, IDESC_PV, (j | ks) ? 1u : 0u);
          }
          umma_commit(bar_pvfull + 8 * t);
        }
        __syncwarp();
      };
      // prologue: S_0(0), S_1(0)
#pragma unroll
      for (int t = 0; t < QTILES && ok; ++t) {
        if (n_kv_t[t] == 0) continue;
        ok = wait_all(bar_q + 8 * t, 0, DEV_TIMEOUT_Q);
        if (ok && t == 0)
          ok = wait_all(bar_kfull, 0, DEV_TIMEOUT_MMA_FULL);
        if (ok && t == 1 && n_kv_t[0] == 0)
          ok = wait_all(bar_kfull, 0, DEV_TIMEOUT_MMA_FULL);
        if (!ok) break;
        tc_fence_after();
        issue_s(t, 0);
      }
      if (ok && elect_one()) umma_commit(bar_kempty);  // K_0 is free once S_0(0), S_1(0) have read it
      __syncwarp();
      for (int j = 0; j < n_kv && ok; ++j) {
        const int b = j & 1;
        const uint32_t par = (j >> 1) & 1u;
        const bool next = j + 1 < n_kv;
        bool k_next_ready = false;
#pragma unroll
        for (int t = 0; t < QTILES && ok; ++t) {
          if (j < n_kv_t[t]) {
            if (t == 0 || j >= n_kv_t[0]) {
              ok = wait_all(bar_vfull + 8 * b, par, DEV_TIMEOUT_MMA_FULL);
              if (!ok) break;
            }
            ok = wait_all(bar_pfull + 8 * t, j & 1u, DEV_TIMEOUT_P);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, j);
          }
          if (next && j + 1 < n_kv_t[t]) {
            if (!k_next_ready) {
              ok = wait_all(bar_kfull + 8 * (b ^ 1), ((j + 1) >> 1) & 1u, DEV_TIMEOUT_MMA_FULL);
              if (!ok) break;
              k_next_ready = true;
              tc_fence_after();
            }
            issue_s(t, j + 1);
          }
        }
        if (!ok) break;
        if (elect_one()) {
          umma_commit(bar_vempty + 8 * b);
          if (next) umma_commit(bar_kempty + 8 * (b ^ 1));
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------- softmax / output (2 x 4 warps) --------------------------
    reg_alloc_200();
    const int t = (warp >> 2) - 1;        // tile of this warpgroup
    const int q = warp & 3;               // TMEM lane quarter this warp may access
    const int r = q * 32 + lane;          // row inside the tile == TMEM lane
    const int row = q0 + t * BQ + r;      // query index
    const uint32_t t_lane = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_s = tmem_base + TM_S + t * BKV + t_lane;
    const uint32_t t_o = tmem_base + TM_O + t * 128 + t_lane;
    const float c = p.scale_log2;
    const int my_n_kv = n_kv_t[t];
    int limit = p.Skv;                    // keys [0, limit) are visible to this row
    if (p.causal) {
      const int l2 = row + shift + 1;
      limit = l2 < limit ? l2 : limit;
    }
    // m = the row maximum the exponentials are currently taken against (raw S units).  It is
    // only raised when the true maximum has grown by more than 2^RESCALE_LOG2 (lazy rescale);
    // until then P may exceed 1 by at most that factor, harmless in bf16/fp32, and O and l stay
    // consistent because both are scaled against the same m.
    constexpr float RESCALE_LOG2 = 8.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_n_kv && ok; ++j) {
      ok = mbar_wait(bar_sfull + 8 * t, j & 1u, abort_flag, p.status, DEV_TIMEOUT_SOFTMAX, p.spin);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * BKV;
      const bool need_mask = kv0 + BKV > limit;
      // the whole S row of this thread: 128 fp32 in registers
      uint32_t sr[4][32];
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld_32x32(t_s + 32 * g, sr[g]);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!(kv0 + 32 * g + i < limit)) sr[g][i] = 0xFF800000u;  // -inf
      }
      // four independent chains keep the max reduction off the critical path
      float mxg[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        mxg[g] = fmax3(__uint_as_float(sr[g][0]), __uint_as_float(sr[g][1]), __uint_as_float(sr[g][2]));
#pragma unroll
        for (int i = 3; i < 31; i += 2) mxg[g] = fmax3(mxg[g], __uint_as_float(sr[g][i]), __uint_as_float(sr[g][i + 1]));
        mxg[g] = fmaxf(mxg[g], __uint_as_float(sr[g][31]));
      }
      const float mx = fmaxf(fmaxf(mxg[0], mxg[1]), fmaxf(mxg[2], mxg[3]));
      // lazy rescale (warp-uniform decision: the TMEM accesses below are warp-collective)
      const bool grow = (mx - m) * c > RESCALE_LOG2 || (m == -INFINITY && mx != -INFINITY);
      if (__any_sync(0xFFFFFFFFu, grow)) {
        const float m_new = grow ? mx : m;
        const float alpha = (m == -INFINITY) ? 0.f : ex2_approx((m - m_new) * c);
        l *= alpha;
        m = m_new;
        if (j > 0) {
          // O_t must be at rest: PV_t(j-1) complete (it is, in steady state: S_t(j) came after it)
          ok = mbar_wait(bar_pvfull + 8 * t, (j - 1) & 1u, abort_flag, p.status, DEV_TIMEOUT_PV, p.spin);
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32(t_o + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(t_o + c0, v);
          }
        }
      }
      // P = exp2(c*s - c*m) as bf16, written over the first 64 columns of this S buffer
      const float mc = (m == -INFINITY) ? 0.f : m * c;
      // (the MUFU unit, 16 exp2 per clock per SM, needs as long for a 128x128 block as the tensor
      // core needs for its two contractions at head dimension 128: see exp2_pair)
      float2 rsg[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) rsg[g] = make_float2(0.f, 0.f);
      if (TF) {
        // P stays fp32 (the tensor core reads it as TF32), over all 128 columns of this S buffer
#pragma unroll
        for (int g = 0; g < 4; ++g) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float2 x = fma2(make_float2(__uint_as_float(sr[g][i]), __uint_as_float(sr[g][i + 1])), make_float2(c, c),
                            make_float2(-mc, -mc));
            x = exp2_pair<POLY>(g, i >> 1, x);
            rsg[(i >> 1) & 3] = add2(rsg[(i >> 1) & 3], x);
            sr[g][i] = __float_as_uint(x.x);
            sr[g][i + 1] = __float_as_uint(x.y);
          }
          tmem_st_32x32(t_s + 32 * g, sr[g]);
        }
      } else {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t pk[32];
#pragma unroll
          for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float2 x = fma2(make_float2(__uint_as_float(sr[2 * hh + g][i]), __uint_as_float(sr[2 * hh + g][i + 1])),
                              make_float2(c, c), make_float2(-mc, -mc));
              x = exp2_pair<POLY>(2 * hh + g, i >> 1, x);
              rsg[(i >> 1) & 3] = add2(rsg[(i >> 1) & 3], x);
              pk[16 * g + (i >> 1)] = pack_bf16x2(x.x, x.y);
            }
          tmem_st_32x32(t_s + 32 * hh, pk);
        }
      }
      const float2 rs2 = add2(add2(rsg[0], rsg[1]), add2(rsg[2], rsg[3]));
      tmem_st_wait();
      l += rs2.x + rs2.y;
      tc_fence_before();
      mbar_arrive(bar_pfull + 8 * t);
    }
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    if (ok && my_n_kv > 0) {
      ok = mbar_wait(bar_pvfull + 8 * t, (my_n_kv - 1) & 1u, abort_flag, p.status, DEV_TIMEOUT_PV, p.spin);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c0 + i] = __uint_as_float(v[i]);
        }
        tc_fence_before();
      }
    }
    const size_t off = (static_cast<size_t>(bh) * p.Sq + row) * D;
    if (ok && row < p.Sq &&
        bounds_ok(off * (p.out_bf16 ? 2 : 4), static_cast<unsigned long long>(D) * (p.out_bf16 ? 2 : 4), p.o_extent,
                  p.status, p.bounds_detail)) {
      const float inv = l > 1e-30f ? 1.f / l : 0.f;   // a row with no visible key sums to < 2^-100
      if (p.out_bf16) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.O) + off);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          uint4 pk;
          pk.x = pack_bf16x2(o[8 * i + 0] * inv, o[8 * i + 1] * inv);
          pk.y = pack_bf16x2(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
          pk.z = pack_bf16x2(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
          pk.w = pack_bf16x2(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
          dst[i] = pk;
        }
      } else {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.O) + off);
#pragma unroll
        for (int i = 0; i < D / 4; ++i)
          dst[i] = make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv,
                               o[4 * i + 3] * inv);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// fp32 -> bf16 (round to nearest even) of Q, K and V in one launch; counts in float4 units
struct CastArgs {
  const float4* src[3];
  uint2* dst[3];
  long long n4[3];
};
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(CastArgs a) {
  griddep_launch_dependents();   // the attention kernel may move in as SMs become free
  const long long n01 = a.n4[0] + a.n4[1], total = n01 + a.n4[2];
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // element i of the concatenation Q | K | V -> its source and destination (selects, so that
  // the argument arrays are never indexed by a run-time value)
  auto locate = [&](long long i, const float4*& src, uint2*& dst) {
    if (i < a.n4[0]) {
      src = a.src[0] + i;
      dst = a.dst[0] + i;
    } else if (i < n01) {
      src = a.src[1] + (i - a.n4[0]);
      dst = a.dst[1] + (i - a.n4[0]);
    } else {
      src = a.src[2] + (i - n01);
      dst = a.dst[2] + (i - n01);
    }
  };
  auto convert = [](const float4 v) { return make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w)); };
  // four independent 16-byte loads in flight per thread before the first store
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < total; i += 4 * stride) {
    float4 v[4];
    uint2* dst[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float4* src;
      locate(i + u * stride, src, dst[u]);
      v[u] = __ldg(src);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) *dst[u] = convert(v[u]);
  }
  for (; i < total; i += stride) {
    const float4* src;
    uint2* dst;
    locate(i, src, dst);
    *dst = convert(__ldg(src));
  }
}

inline size_t pad256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

template <int D, bool TF = false>
kcg_status_t launch_fmha(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const FmhaParams& p, int bh, cudaStream_t stream, bool after_cast) {
  using Cfg = FmhaCfg<D, TF>;
  static_assert(Cfg::SMEM_TOTAL <= 232448, "shared memory budget");
  auto kern = fmha_fwd_kernel<D, TF>;
  KCG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_TOTAL));
  FmhaParams pp = p;
  pp.after_cast = after_cast ? 1 : 0;
  pp.n_qp = (p.Sq + QTILES * BQ - 1) / (QTILES * BQ);
  pp.bh_total = bh;
  // heads per group: enough tile pairs for two waves of the SMs, at least 8 heads, and K + V of
  // a group within a third of the L2 (head dimension D, Skv keys, 2 or 4 bytes per element)
  {
    const long long kv_bytes = 2ll * p.Skv * D * (TF ? 4 : 2);
    const long long l2_heads = (40ll << 20) / (kv_bytes > 0 ? kv_bytes : 1);
    long long g = (2ll * device_sm_count() + pp.n_qp - 1) / pp.n_qp;
    if (g < 8) g = 8;
    if (g > l2_heads) g = l2_heads;
    if (g < 1) g = 1;
    if (g > bh) g = bh;
    // equal groups: a short last group would start its longest tile pairs when the launch is
    // nearly over
    const long long n_groups = (bh + g - 1) / g;
    g = (bh + n_groups - 1) / n_groups;
    pp.bh_group = static_cast<int>(g);
    pp.bh_small = static_cast<int>(g * n_groups - bh);
  }
  const long long items = static_cast<long long>(pp.n_qp) * bh;
  if (items > 0x7FFFFFFFll) return KCG_BAD_SHAPE;
  dim3 grid(static_cast<unsigned>(items));
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = grid;
  cfg.blockDim = dim3(FM_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_TOTAL;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = after_cast ? 1 : 0;
  KCG_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, pp));
  g_launches.fetch_add(1);
  return KCG_OK;
}

}  // namespace

// out = {grid, threads per CTA, queries per CTA, keys per block}
kcg_status_t fmha_launch_geometry_impl(const kcg_fmha_desc* d, int* out) {
  if (!d || !out) return KCG_BAD_ARGUMENT;
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Skv <= 0) return KCG_BAD_SHAPE;
  const long long items = static_cast<long long>((d->Sq + QTILES * BQ - 1) / (QTILES * BQ)) * d->B * d->H;
  if (items > 0x7FFFFFFFll) return KCG_BAD_SHAPE;
  out[0] = static_cast<int>(items);
  out[1] = FM_THREADS;
  out[2] = QTILES * BQ;
  out[3] = BKV;
  return KCG_OK;
}

size_t fmha_workspace_impl(const kcg_fmha_desc* d) {
  if (!d || d->dtype_in != KCG_F32) return 0;
  if (d->D == 64) return 0;   // TF32 contractions straight from the fp32 tiles
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Skv <= 0 || d->D <= 0) return 0;
  const size_t bh = static_cast<size_t>(d->B) * d->H;
  return pad256(bh * d->Sq * d->D * 2) + 2 * pad256(bh * d->Skv * d->D * 2);
}

kcg_status_t fmha_launch_impl(const kcg_fmha_desc* d, const void* Q, const void* K, const void* V,
                              void* O, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (!d || !Q || !K || !V || !O) return KCG_BAD_ARGUMENT;
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Skv <= 0) return KCG_BAD_SHAPE;
  if (d->D != 64 && d->D != 128) return KCG_BAD_SHAPE;
  if (static_cast<long long>(d->B) * d->H > 0x7FFFFFll) return KCG_BAD_SHAPE;
  if (d->dtype_in != KCG_F32 && d->dtype_in != KCG_BF16) return KCG_UNSUPPORTED;
  if (d->dtype_out != KCG_F32 && d->dtype_out != KCG_BF16) return KCG_UNSUPPORTED;
  if (!(d->scale > 0.f)) return KCG_BAD_ARGUMENT;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return KCG_BAD_ALIGN;
  const int bh = d->B * d->H;
  const size_t q_elems = static_cast<size_t>(bh) * d->Sq * d->D;
  const size_t kv_elems = static_cast<size_t>(bh) * d->Skv * d->D;
  const void* q = Q;
  const void* k = K;
  const void* v = V;
  const bool tf = d->dtype_in == KCG_F32 && d->D == 64;   // TF32 contractions on the fp32 tiles
  if (d->dtype_in == KCG_F32 && !tf) {
    const size_t need = fmha_workspace_impl(d);
    if (!ws || ws_bytes < need || !aligned16(ws)) return KCG_BAD_WORKSPACE;
    uint8_t* w = static_cast<uint8_t*>(ws);
    void* qb = w;
    void* kb = w + pad256(q_elems * 2);
    void* vb = w + pad256(q_elems * 2) + pad256(kv_elems * 2);
    const int blocks = device_sm_count() * 4;
    CastArgs ca;
    ca.src[0] = static_cast<const float4*>(Q);
    ca.src[1] = static_cast<const float4*>(K);
    ca.src[2] = static_cast<const float4*>(V);
    ca.dst[0] = static_cast<uint2*>(qb);
    ca.dst[1] = static_cast<uint2*>(kb);
    ca.dst[2] = static_cast<uint2*>(vb);
    ca.n4[0] = static_cast<long long>(q_elems / 4);
    ca.n4[1] = ca.n4[2] = static_cast<long long>(kv_elems / 4);
    f32_to_bf16_kernel<<<blocks, 256, 0, stream>>>(ca);
    g_launches.fetch_add(1);
    KCG_CUDA_TRY(cudaGetLastError());
    q = qb;
    k = kb;
    v = vb;
  }
  CUtensorMap tq, tk, tv;
  // one 128-byte swizzle panel of a tile per copy: 64 bf16 or 32 fp32 wide, 128 rows
  const uint32_t box[3] = {tf ? 32u : 64u, 128, 1};
  const CUtensorMapDataType dt = tf ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t es = tf ? 4 : 2;
  // fp32 V is an MN-major operand: 32-byte-atom form of the 128B swizzle
  const CUtensorMapSwizzle sw_v = tf ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(d->D), static_cast<uint64_t>(d->Sq),
                              static_cast<uint64_t>(bh)};
    const uint64_t strides[2] = {static_cast<uint64_t>(d->D) * es,
                                 static_cast<uint64_t>(d->Sq) * d->D * es};
    kcg_status_t st = encode_tmap(&tq, dt, 3, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != KCG_OK) return st;
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(d->D), static_cast<uint64_t>(d->Skv),
                              static_cast<uint64_t>(bh)};
    const uint64_t strides[2] = {static_cast<uint64_t>(d->D) * es,
                                 static_cast<uint64_t>(d->Skv) * d->D * es};
    kcg_status_t st = encode_tmap(&tk, dt, 3, k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != KCG_OK) return st;
    st = encode_tmap(&tv, dt, 3, v, dims, strides, box, sw_v);
    if (st != KCG_OK) return st;
  }
  FmhaParams p;
  p.O = O;
  p.Sq = d->Sq;
  p.Skv = d->Skv;
  p.causal = d->causal ? 1 : 0;
  p.out_bf16 = d->dtype_out == KCG_BF16;
  p.scale_log2 = d->scale * 1.4426950408889634f;
  p.o_extent = static_cast<unsigned long long>(q_elems) * (d->dtype_out == KCG_BF16 ? 2 : 4);
  if (const unsigned long long cap = debug_extent_limit()) p.o_extent = p.o_extent < cap ? p.o_extent : cap;
  p.bounds_detail = nullptr;
  debug_bounds_detail_ptr(&p.bounds_detail);
  kcg_status_t st = device_status_ptr(&p.status);
  if (st != KCG_OK) return st;
  const uint32_t spin = g_spin_limit.load();
  p.spin = spin ? spin : KCG_SPIN_LIMIT;
  if (tf) return launch_fmha<64, true>(tq, tk, tv, p, bh, stream, false);
  if (d->D == 64) return launch_fmha<64>(tq, tk, tv, p, bh, stream, false);
  return launch_fmha<128>(tq, tk, tv, p, bh, stream, d->dtype_in == KCG_F32);
}

}  // namespace kcg
