/*
 * kcg_capi.h -- C-ABI launch layer of the B200 (sm_100a) backend.
 *
 * The reference project (yao-jiashu/KernelCodeGen) has no FFI of its own: its Backend returns
 * CUDA source text (src/Backend/CUDA.cc:878-890) whose kernels take flat row-major device
 * pointers in first-touch order -- (A, B, C) for matmul, (Q, K, V, O) for attention
 * (src/Backend/CUDA.cc:217-266, 795-801) -- and an out-of-tree harness compiled and launched
 * that text (test/test.cc:26-34).  The entry points below take the place of that
 * "emit text, compile, launch" step: same pointer order, same row-major layouts, but the
 * kernels are hand-written for sm_100a and are launched directly.
 *
 * Conventions
 *   - every pointer is caller-owned DEVICE memory unless the name says host;
 *   - launches are asynchronous on `stream` (a cudaStream_t passed as void*; NULL = default);
 *   - nothing here allocates device memory unless documented; scratch is passed in;
 *   - no exceptions cross this boundary; every call returns a kcg_status_t;
 *   - there is no CPU fallback: without an sm_100 device the launch calls fail with
 *     KCG_UNSUPPORTED / KCG_CUDA_ERROR.
 */
#ifndef KCG_CAPI_H_
#define KCG_CAPI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum kcg_status_t {
  KCG_OK = 0,
  KCG_BAD_SHAPE = 1,      /* non-positive extent, K mismatch, head_dim not supported ...   */
  KCG_BAD_ALIGN = 2,      /* pointer not 16-byte aligned or leading dimension not 16 bytes  */
  KCG_UNSUPPORTED = 3,    /* dtype / precision / tile combination with no kernel            */
  KCG_CUDA_ERROR = 4,     /* a CUDA runtime/driver call failed                              */
  KCG_DEVICE_TIMEOUT = 5, /* a bounded device-side wait ran out (see kcg_last_device_status)*/
  KCG_PEER_TIMEOUT = 6,   /* a rank did not arrive: host-side check-in, or kcg_peer_wait_launch */
  /* 7 is not used: the library itself makes no NCCL call */
  KCG_BAD_WORKSPACE = 8,  /* workspace NULL or smaller than kcg_*_workspace_bytes()         */
  KCG_BAD_ARGUMENT = 9,   /* NULL descriptor / NULL tensor pointer                          */
  KCG_TOO_LARGE = 10      /* problem needs more scratch than kcg_gemm_launch_static holds   */
} kcg_status_t;

typedef enum kcg_dtype_t { KCG_F32 = 0, KCG_BF16 = 1 } kcg_dtype_t;

/* How an fp32 contraction is carried out on the tensor cores.
 *   3XTF32: a = a_hi + a_lo, C = a_lo*b_hi + a_hi*b_lo + a_hi*b_hi, fp32 accumulate --
 *           keeps the reference's fp32 contract (src/Frontend/Operators.cc:163-164) to ~1e-6.
 *   TF32  : one TF32 product (10-bit mantissa inputs).
 *   BF16  : inputs are bf16 in memory. */
typedef enum kcg_precision_t {
  KCG_PREC_3XTF32 = 0,
  KCG_PREC_TF32 = 1,
  KCG_PREC_BF16 = 2
} kcg_precision_t;

typedef enum kcg_epilogue_t { KCG_EPI_NONE = 0, KCG_EPI_RELU = 1 } kcg_epilogue_t;

/* Layout of the B operand, named after the reference's enum Layout (include/enum.h:24-27):
 * ROW_MAJOR = B stored [K, N]; COL_MAJOR = B stored [N, K] (the QK^T case,
 * src/Frontend/Operators.cc:301-307). A and C are always row-major. */
typedef enum kcg_layout_t { KCG_ROW_MAJOR = 0, KCG_COL_MAJOR = 1 } kcg_layout_t;

/* C[M,N] = epilogue(A[M,K] . B), replaces the kernel generated from Matmul::build
 * (src/Frontend/Operators.cc:77-179) + Relu::build (:182-250) by MatmulOptimizer
 * (src/Optimizer/Optimizer.cc:383-548).  Leading dimensions are in ELEMENTS.
 * tile_n / stages / group_m are the schedule knobs (0 = library default):
 *   tile_n  <- BLOCK_SIZE_N (128 or 256; default 256, 128 for short 3xTF32 launches),
 *              tile_m is fixed at 128 (one UMMA M) per CTA,
 *   stages  <- depth of the TMA->UMMA shared-memory ring,
 *   group_m <- GROUP_SIZE_M: how many row-blocks are walked before moving to the next
 *              column-block (L2 reuse of the B panel). */
typedef struct kcg_gemm_desc {
  int64_t M, N, K;
  int64_t lda, ldb, ldc;
  int32_t dtype_in;  /* kcg_dtype_t of A and B  */
  int32_t dtype_out; /* kcg_dtype_t of C        */
  int32_t precision; /* kcg_precision_t         */
  int32_t epilogue;  /* kcg_epilogue_t          */
  int32_t b_layout;  /* kcg_layout_t            */
  int32_t tile_n;
  int32_t stages;
  int32_t group_m;
  /* Fused all-gather (optional): when n_peers > 0 every finished C tile is also stored to
   * peer_c[i] + the same offset, i = 0..n_peers-1 (peer-mapped device pointers of the other
   * ranks' C buffers, already offset to this rank's row block). Plain unicast stores. */
  int32_t n_peers;
  /* 1: one CTA per 128 x tile_n tile.  2: CTA pairs (tcgen05 cta_group::2) share a
   * 256 x tile_n tile, each CTA loading half of the B tile.  0: library default (pairs for launches
   * below ~4 TFLOP of work, single CTAs for long, power-limited ones). */
  int32_t cta_group;
  void* peer_c[8];
  /* Fused all-gather through an NVSwitch multicast mapping (optional; NULL = off): the multicast
   * address of C at this rank's first row.  Every finished 128-byte row segment is then stored
   * ONCE (multimem.st) and the switch delivers it to all ranks bound to the mapping, this one
   * included; neither C nor peer_c is written for those segments.  The local C pointer must be
   * this rank's unicast view of the same memory.  Needs N * sizeof(element of C) % 128 == 0.
   * The mapping comes from the caller (CUDA multicast objects, e.g. torch symmetric memory). */
  void* mc_c;
  /* Completion flags (optional; 0 = none): when the last CTA of the launch has finished, and
   * after all of the launch's stores of C, done_value is stored (release, system scope) to each
   * of the n_done_flags 32-bit words -- normally this rank's slot in every rank's flag array
   * (peer-mapped addresses) -- so that a consumer on any rank can wait for this rank's row
   * block with kcg_peer_wait_launch instead of a collective. */
  int32_t n_done_flags;
  uint32_t done_value;
  void* done_flags[9];
} kcg_gemm_desc;

/* O[B,H,Sq,D] = softmax(scale * Q.K^T [+ causal mask]) . V, tensors [B,H,S,D] contiguous
 * (test/test.cc:71-90).  Replaces the kernel FMHAOptimizer builds from the
 * BatchedMatmul -> Softmax -> BatchedMatmul chain (src/Optimizer/Optimizer.cc:1079-1333).
 * scale = 1 and causal = 0 reproduce the reference's graph exactly
 * (src/Frontend/Operators.cc:504-534 has neither scale nor mask). */
typedef struct kcg_fmha_desc {
  int32_t B, H;
  int32_t Sq, Skv;
  int32_t D;          /* head dim: 64 or 128 */
  int32_t dtype_in;   /* kcg_dtype_t of Q, K, V (F32: TF32 products for D = 64, rounded to bf16 for D = 128) */
  int32_t dtype_out;  /* kcg_dtype_t of O */
  int32_t causal;     /* 0 / 1 : query i sees keys j <= i + (Skv - Sq) */
  float scale;        /* multiplies the logits before exp */
  int32_t reserved;
} kcg_fmha_desc;

/* Scratch the launch can use (bytes; may be 0).
 * GEMM: (1) required for 3xTF32: the fp32 residuals (x minus its TF32 truncation) of A and B,
 * 4*(M*K + K*N) bytes, each array rounded up to 256; (2) optional, behind (1), for launches on
 * CTA pairs whose tile count does not fill the last wave of the persistent grid: room for the
 * partial accumulators of the shared-K tail (the k-blocks of the left-over tiles are divided
 * between all CTA pairs, and the partial sums meet in the workspace).  A launch given only (1),
 * or no workspace for bf16/TF32, runs without the shared-K tail: same result up to fp32
 * summation order, a little slower when the last wave is poorly filled.
 * FMHA with f32 inputs and head dimension 128: bf16 copies of Q, K, V (head dimension 64 runs TF32
 * contractions on the fp32 arrays and needs none). */
size_t kcg_gemm_workspace_bytes(const kcg_gemm_desc* d);
size_t kcg_fmha_workspace_bytes(const kcg_fmha_desc* d);

/* Introspection (no counterpart in the reference): how many left-over tiles the shared-K tail
 * covers for this descriptor on a B200's 74 CTA pairs; 0 = the launch has no shared-K tail. */
int kcg_gemm_shared_k_tiles(const kcg_gemm_desc* d);

/* Introspection for tests (no counterpart in the reference): the shared-K plan for `tiles` pair
 * tiles of `num_kb` k-blocks on `pairs` CTA pairs; out5 = {tail tiles, ranges, k-block positions
 * per range, positions per tile (>= num_kb: the surplus is padding), most contributors per tile};
 * all zero when the launch has no shared-K tail.  Range u covers positions [u*share, (u+1)*share)
 * of the tail tiles laid end to end, `span` positions per tile. */
void kcg_gemm_shared_k_plan(int32_t tiles, int32_t num_kb, int32_t pairs, int32_t tile_n, int32_t* out5);

/* The launch geometry the library will use for a descriptor on a B200 (148 SMs): takes the place
 * of the `// grid dims:(..), block dims:(..)` comment the reference prints above each kernel
 * (src/Backend/CUDA.cc:786-791), and is what the generated launcher text quotes.
 * GEMM  out6 = {CTAs in the grid, threads per CTA, cluster size (2 = CTA pairs), rows and columns
 *               of one output tile, number of output tiles};
 * FMHA  out4 = {CTAs in the grid, threads per CTA, queries per CTA, keys per block}. */
kcg_status_t kcg_gemm_launch_geometry(const kcg_gemm_desc* d, int32_t* out6);
kcg_status_t kcg_fmha_launch_geometry(const kcg_fmha_desc* d, int32_t* out4);

/* Replaces: launch of `<graph>::kernel0(A, B, C)` emitted by CUDAGen
 * (src/Backend/CUDA.cc:773-857) for the scheduled Matmul func, with Relu fused. */
kcg_status_t kcg_gemm_launch(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Same fp32-contract (3xTF32) matmul(+ReLU) as kcg_gemm_launch, for callers that cannot hand
 * over a workspace because they cannot allocate device memory at all: a plug-in running inside
 * a host whose allocator has reserved the whole GPU up front (a cudaMalloc there fails or
 * fragments the host's pool), or a latency-critical loop where an allocation's implicit
 * device synchronisation is not acceptable.  The TF32 residuals of A and B go into a
 * fixed array that is part of the library image, KCG_STATIC_SCRATCH_BYTES (32 MiB) on every
 * GPU that loads the library, held until the process exits.  This call performs no
 * cudaMalloc/cudaFree and calls nothing that allocates.
 *   - Limit: the residual arrays must fit KCG_STATIC_SCRATCH_BYTES, i.e.
 *     4*(M*K + K*N) bytes (each term rounded up to 256) -- e.g. up to 1024 x N x 1024 with
 *     N <= 7168, or 2048 x 2048 x 2048.  Larger problems return KCG_TOO_LARGE (and say so on
 *     stderr).
 *   - Only precision KCG_PREC_3XTF32 (the one path that needs scratch); others:
 *     KCG_UNSUPPORTED -- use kcg_gemm_launch with a NULL workspace for those.
 *   - The first call on each device looks up the array's device address; make that first
 *     call before starting any stream capture on that device.  With lazy module loading it is
 *     also this first call (or any earlier GEMM launch of this library on the device) that
 *     loads the module and with it reserves the 32 MiB: in a host that reserves the rest of
 *     the GPU's memory for itself, make it before the host does so, or it can fail.
 *   - All calls on a device share the one array.  Nothing in it has to be cleared between
 *     calls (each call rewrites every byte it later reads), but two calls whose kernels
 *     overlap on the GPU (different streams, no ordering between them) race on it: keep
 *     calls to this entry point ordered on one stream, or serialise them yourself.
 * This entry point has no counterpart in the reference. */
#define KCG_STATIC_SCRATCH_BYTES (32u << 20)
kcg_status_t kcg_gemm_launch_static(const kcg_gemm_desc* d, const void* A, const void* B, void* C,
                                    void* stream);

/* Replaces: launch of `Fused_Multi_Head_Attention_*::kernel0(Q, K, V, O)`
 * (src/Optimizer/Optimizer.cc:1101-1111, src/Backend/CUDA.cc:773-857). */
kcg_status_t kcg_fmha_fwd_launch(const kcg_fmha_desc* d, const void* Q, const void* K,
                                 const void* V, void* O, void* workspace, size_t workspace_bytes,
                                 void* stream);

/* The reference's Softmax operator on its own (src/Frontend/Operators.cc:474-536): last-axis
 * exp(x)/sum(exp(x)) over a [rows, cols] fp32 array, in place when y == x.  Used for graphs
 * where Softmax is not part of an attention chain (there it is fused into the FMHA kernel). */
kcg_status_t kcg_softmax_launch(int64_t rows, int64_t cols, const void* x, void* y, void* stream);

/* The reference's Transpose operator (include/Frontend/Operators.h:100-102; its build has no body,
 * src/Frontend/Operators.cc:422-423): y[b, j, i] = x[b, i, j] for `batch` contiguous row-major
 * [rows, cols] matrices of KCG_F32 or KCG_BF16 elements; out of place (x != y). */
kcg_status_t kcg_transpose_launch(int64_t batch, int64_t rows, int64_t cols, int32_t dtype, const void* x, void* y,
                                  void* stream);

/* The reference's BatchedMatmul operator on its own (src/Frontend/Operators.cc:253-420): `batch`
 * independent products described by `d`, operand i at base + i * stride (strides in elements, each
 * a multiple of 16 bytes; 0 shares an operand between all entries).  Layout::colMajor B =
 * d->b_layout KCG_COL_MAJOR.  ONE launch: the batch entry is the outermost part of the persistent
 * tile index and the third coordinate of the tensor maps, so tiles of all entries fill the SMs
 * together and a ragged entry is zero-filled at its own edge.  For 3xTF32 the residual pass
 * covers all entries in the same single launch, and a shared operand is split once; the
 * workspace is sized by kcg_batched_gemm_workspace_bytes. */
kcg_status_t kcg_batched_gemm_launch(const kcg_gemm_desc* d, int64_t batch, int64_t stride_a, int64_t stride_b,
                                     int64_t stride_c, const void* A, const void* B, void* C, void* workspace,
                                     size_t workspace_bytes, void* stream);
size_t kcg_batched_gemm_workspace_bytes(const kcg_gemm_desc* d, int64_t batch, int64_t stride_a, int64_t stride_b);

/* Host-buffer forms (what the reference's absent harness did around the kernel: cudaMalloc, H2D,
 * launch, D2H -- performance/output.log:6-13).  They allocate device buffers, copy, launch, copy
 * back and synchronise.  kcg_gemm_host runs the schedule of kcg_gemm_host_staged below. */
kcg_status_t kcg_gemm_host(const kcg_gemm_desc* d, const void* hA, const void* hB, void* hC);

/* The same host-to-host product with the PCIe copies overlapped with the kernel, on device buffers
 * the caller owns (no allocation here).  hA/hB/hC are host arrays laid out as `d` says (pinned
 * memory for the copies to overlap; pageable memory works but serialises); dA/dB/dC are device
 * arrays of the same shapes and leading dimensions.  A is cut into row chunks and B into column
 * chunks (`chunks` of each, at most 16; 0 = about 2048 rows / columns per chunk), copied
 * alternately; the kernel runs on row chunk k x column chunks 0..k-1 as soon as row chunk k has
 * landed and on row chunks 0..k x column chunk k as soon as column chunk k has, so every C tile
 * is computed once, as early as its operands allow; finished strips of C return to the host while
 * later chunks are still arriving.  Copies and launches run on the library's own three streams per
 * device; they start after the work already queued on `stream`, and `stream` continues once the
 * last strip of C is on the host, so the caller only synchronises `stream`.  d->peer_c, when set,
 * receives every strip as in kcg_gemm_launch.  `workspace` as for kcg_gemm_launch with `d`.
 * hB may be NULL: B is then taken as already present in dB (a multi-GPU caller that copies 1/N of
 * B over its own PCIe link and gathers the rest from its peers over NVLink before this call);
 * only the row chunks of A and the strips of C move.
 * The device-side status is not read here: call kcg_last_device_status after synchronising. */
kcg_status_t kcg_gemm_host_staged(const kcg_gemm_desc* d, const void* hA, const void* hB, void* hC, void* dA,
                                  void* dB, void* dC, void* workspace, size_t workspace_bytes, int chunks,
                                  void* stream);
kcg_status_t kcg_fmha_fwd_host(const kcg_fmha_desc* d, const void* hQ, const void* hK,
                               const void* hV, void* hO);

/* Average device time of one launch (ms) on zero-filled scratch buffers the call allocates and
 * frees itself: the cost function behind KernelCodeGenerator::evaluate (a stub returning 0 in
 * the reference, include/KernelCodeGen.h:119-121).  KCG_CUDA_ERROR when no device is present. */
kcg_status_t kcg_gemm_time(const kcg_gemm_desc* d, int iters, float* ms_per_launch);
kcg_status_t kcg_fmha_time(const kcg_fmha_desc* d, int iters, float* ms_per_launch);

/* Buffers other ranks' kernels can store into (one process per GPU, same node).  The fused
 * all-gather of C needs every rank's C buffer mapped into every other rank:
 *   kcg_peer_alloc  allocates `bytes` of device memory and returns a 64-byte handle that can
 *                   be sent to the other processes (any byte transport);
 *   kcg_peer_open   maps a peer's handle into this process and returns a device pointer valid
 *                   for plain loads/stores from this GPU (peer access is enabled lazily);
 *   kcg_peer_close / kcg_peer_free undo them.
 * No counterpart in the reference, which has no multi-GPU path. */
kcg_status_t kcg_peer_alloc(size_t bytes, void** out_ptr, void* out_handle64);
kcg_status_t kcg_peer_open(const void* handle64, void** out_ptr);
kcg_status_t kcg_peer_close(void* ptr);
kcg_status_t kcg_peer_free(void* ptr);

/* Waits, on the device and in stream order, until each of the `n` 32-bit flag words
 * flags[i * stride_words] (i = 0..n-1, device memory of the current GPU that other ranks'
 * kernels store into, see kcg_gemm_desc.done_flags) has reached `value` (wrap-safe signed
 * comparison).  One small kernel, one thread per flag, acquire loads at system scope.  The wait
 * is bounded: after `max_polls` polls per flag (0 = about a second's worth) the kernel gives up,
 * records code 9 in the device status word and returns, so the stream continues and the context
 * stays usable; kcg_peer_wait_status then reports KCG_PEER_TIMEOUT.  No counterpart in the
 * reference, which has no multi-GPU path. */
kcg_status_t kcg_peer_wait_launch(const void* flags, int32_t n, int32_t stride_words, uint32_t value,
                                  uint32_t max_polls, void* stream);
/* Synchronises the device, reads and clears the status word: KCG_OK, KCG_PEER_TIMEOUT when a
 * kcg_peer_wait_launch gave up, KCG_DEVICE_TIMEOUT for any other bounded wait that ran out. */
kcg_status_t kcg_peer_wait_status(void);

/* Reads (and clears) the status word of the current device that a kernel sets when one of
 * its bounded waits runs out; 0 = no timeout.  Synchronises the device. */
int kcg_last_device_status(void);

/* Self-test of the bounded device-side wait: launches one thread that waits `iterations`
 * polls (1 .. 2^20) on a barrier nothing arrives on.  Returns KCG_DEVICE_TIMEOUT when the wait
 * gave up and reported it as designed (the expected outcome), KCG_OK if it did not time out.
 * The device stays usable afterwards.  No counterpart in the reference (it has no waits). */
kcg_status_t kcg_selftest_wait_timeout(uint32_t iterations);

/* Test hook: iteration cap of the device-side waits for subsequent launches (0 = default). */
void kcg_set_spin_limit(uint32_t iterations);

/* Bounds-checking build.  The library can be built a second time with -DKCG_DEBUG_BOUNDS
 * (libkcg_b200_bounds.so; kernelcodegen_b200.build.build_bounds()).  In that build every global
 * store of a result and every access to the shared-K scratch is checked against the byte extent
 * of its buffer, and the launch code checks every tensor-map coordinate it will issue for the
 * 16-byte rule; a failed device-side check records code 10 in the status word
 * (kcg_last_device_status) and the offending offset / extent (kcg_debug_bounds_detail), SKIPS the
 * access and lets the kernel finish: nothing traps and no memory outside the buffers is touched.
 * It takes the place of a memory sanitizer where none can be run.
 *   kcg_debug_bounds_enabled     1 in that build, 0 in the normal one;
 *   kcg_debug_set_extent_limit   test hook: caps the extents the kernels check against (0 = off),
 *                                so that the reporting path can be exercised on buffers that are in
 *                                fact large enough (no real out-of-bounds access is ever made);
 *   kcg_debug_bounds_detail      out2 = {byte offset of the first failed check, extent}.
 * No counterpart in the reference, whose generated kernels have no bounds checks at all. */
int kcg_debug_bounds_enabled(void);
void kcg_debug_set_extent_limit(uint64_t bytes);
kcg_status_t kcg_debug_bounds_detail(uint64_t* out2);

/* Number of kernel launches this library has issued since load (all threads). */
uint64_t kcg_launch_count(void);

const char* kcg_status_str(kcg_status_t s);
const char* kcg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KCG_CAPI_H_ */
