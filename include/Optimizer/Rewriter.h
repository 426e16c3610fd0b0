// Schedule primitives (reference: include/Optimizer/Rewriter.h:13-229).
//
// Every primitive of the reference exists under its name and signature and transforms the IR
// structurally, stage for stage as in the reference's README.md:28-1607 snapshots, so that a
// schedule written against the reference (src/Optimizer/Optimizer.cc:383-548) runs unchanged.
// The register / shared-memory choreography those later stages describe is done in hardware by
// the tcgen05 kernels (TMA, swizzled shared memory, TMEM); MatmulOptimizer therefore uses the
// short annotation forms of read / write / cache_* / pipeline (no map argument), which validate
// their arguments and leave a `kcg.<name>` record that the Backend turns into launch descriptor
// fields (e.g. pipeline depth -> stages).
#pragma once

#include <functional>
#include <string>
#include <vector>

#include "IR/IR.h"
#include "Optimizer/Analyzer.h"
#include "enum.h"

namespace KernelCodeGen {

struct Rewriter {
  Rewriter() = default;

  static mlir::OpBuilder getBuilder(mlir::AffineForOp op, Position pos);
  static std::vector<mlir::Value> getParallelIdx(mlir::AffineParallelOp parallelLevel) { return parallelLevel.getIVs(); }

  // One loop -> `num_output` nested loops.  `factors` are the tile sizes, any order; with
  // factors {8, 128} on `0 to 4096` the result is [0 to 4096 step 128, 0 to 128 step 8, 0 to 8]
  // (outer to inner) and every use of the old induction variable becomes the sum of the new ones.
  static std::vector<mlir::AffineForOp> split(mlir::AffineForOp forOp, uint64_t num_output,
                                              std::vector<int64_t>&& factors);

  // Turns the value carried by loops[0] (the k loop: iter_args) into a local buffer indexed by
  // the other loops of the vector; returns the buffer.  Handles in `loops` stay valid.
  static mlir::Value bufferizeLoopCarryVar(std::vector<mlir::AffineForOp>& loops);

  // Re-nests the given loops in the given order (outer to inner).  Operations that sit between
  // the loops (an accumulator initialisation before the k loop, the write-back after it) are
  // distributed into copies of the enclosing loops, as in README.md:148-187.
  static void reorder(const std::vector<mlir::AffineForOp>& forOp);

  // Up to three perfectly nested loops -> one affine.parallel (lower bound 0, step 1); the
  // first one created in a function is the grid level, a nested one the block level.
  static mlir::AffineParallelOp parallel(const std::vector<mlir::AffineForOp>& forOp);

  // memref.alloc at the top of `father`'s body.
  static mlir::Value alloc_buffer(mlir::Operation* father, MemorySpace ms, const std::vector<int64_t>& shape,
                                  mlir::Type dtype);
  static mlir::Value alloc_buffer(mlir::Operation* contextOp, Position pos, MemorySpace ms,
                                  const std::vector<int64_t>& shape, mlir::Type dtype);

  static mlir::gpu::BarrierOp barrier(mlir::AffineForOp compute_at, Position pos);

  // --- recorded (annotation-only) primitives --------------------------------------------------
  static mlir::Operation* read(mlir::Value src, mlir::Value dst, int64_t width, mlir::AffineForOp compute_at,
                               Position pos);
  static mlir::Operation* write(mlir::Value src, mlir::Value dst, int64_t width, mlir::AffineForOp compute_at,
                                Position pos);
  static void cache_read(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached);
  static void cache_write(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached);
  // The innermost copy loop `for i = 0 to n` over scalar loads / stores becomes `step width` over
  // affine.vector_load / affine.vector_store of `width` elements (README.md:723-802); the width
  // is also recorded on the loop (kcg.vectorize).  A loop that does not have that shape only
  // receives the attribute.
  static mlir::AffineForOp vectorize(mlir::AffineForOp readOrWrite, int64_t width);
  // double buffering of `buffer` around `compute_at`: `stages` buffers in flight
  static mlir::Operation* pipeline(mlir::Value buffer, mlir::AffineForOp compute_at, int64_t stages = 2);
  static void unrollAttribute(mlir::ModuleOp module, const std::function<bool(mlir::AffineForOp)>& unrollCheckFn);

  // Loops of `parallelLevel`'s body that store into `dst` (outer to inner per nest).
  static std::vector<std::vector<mlir::AffineForOp>> get_write(mlir::AffineParallelOp parallelLevel, mlir::Value dst);

  // --- the reference's structural forms (include/Optimizer/Rewriter.h:111-227 there): same names,
  // argument order and results, on the IR of include/IR/IR.h --------------------------------------
  // Copy loop src -> dst placed at `pos` of `compute_at`: `for iv = 0 to size(dst) / width` with
  // `vector_load src[map(operands..., iv)]` and `vector_store dst[iv * width]` (README.md:281-336).
  static mlir::AffineForOp read(mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                llvm::SmallVector<mlir::Value> operands, int64_t width, mlir::AffineForOp compute_at,
                                Position pos);
  static mlir::AffineForOp read(mlir::OpBuilder& builder, mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                llvm::SmallVector<mlir::Value> operands, int64_t width);
  // Copy loop src -> dst with the map on the destination: `vector_load src[iv * width]`,
  // `vector_store dst[map(operands..., iv)]`; a map with one more dimension gets an inner loop over
  // the `width` elements and stores them one by one (a transposed tile, README.md:338-405).
  static mlir::AffineForOp write(mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                 llvm::SmallVector<mlir::Value> operands, int64_t width, mlir::AffineForOp compute_at,
                                 Position pos);
  static mlir::AffineForOp write(mlir::OpBuilder& builder, mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                 llvm::SmallVector<mlir::Value> operands, int64_t width);
  // Inside `scope`: loads of `src` become loads of `cached[map(operands)]` (README.md:484-559);
  // stores to `src` keep their value and get the index `map(operands)` (README.md:561-640).
  static void cache_read(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached, mlir::AffineMap map,
                         llvm::SmallVector<mlir::Value> operands);
  static void cache_write(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached, mlir::AffineMap map,
                          llvm::SmallVector<mlir::Value> operands);
  // Double buffering of `buffer` (re-allocated with a leading extent 2; the reference to it is
  // updated) around `compute_at`: copies of `readBodys` with the induction variable at its first
  // value fill buffer[0] before the loop; inside, the bodies run one iteration ahead under
  // `affine.if (iv + 2 * step <= ub)` into buffer[(iv / step + 1) mod 2] while every other access
  // uses buffer[(iv / step) mod 2] (README.md:804-921).  Returns {copies before the loop, bodies
  // inside it}.
  static std::vector<std::vector<mlir::AffineForOp>> pipeline(std::vector<mlir::AffineForOp> readBodys,
                                                              mlir::Value& buffer, mlir::AffineForOp compute_at);
  // vector loads of `buffer` inside `scope` switch to the other half: x mod 2 -> (x + 1) mod 2
  static void change_double_buffer(mlir::AffineForOp scope, mlir::Value buffer);
  // The last iteration leaves the loop: upper bound - step, and a copy of the body with the
  // induction variable fixed to that value follows the loop (README.md:923-1063).
  static void detach_last_loop(mlir::AffineForOp forOp);
  // Moves `srcOp` before / after `dstOp`, or to the end of the loop `dstOp`.
  static void schedule(mlir::Operation* srcOp, mlir::Operation* dstOp, Position pos);
  // A copy of `srcOp` for iteration `iteration` of `forOp` is placed before `forOp`.
  static void extract_loop(mlir::Operation* srcOp, mlir::AffineForOp forOp, int64_t iteration);
  // affine.if whose condition holds (fails) for every value its operands take is replaced by its
  // body (erased).
  static void take_off_true_if(mlir::ModuleOp module);
  static void delete_false_if(mlir::ModuleOp module);
  // Full unrolling of the loops the predicate selects: one copy of the body per iteration with
  // the induction variable replaced by an index constant.
  static void unroll(mlir::ModuleOp module, mlir::function_ref<bool(mlir::AffineForOp)> unrollCheckFn);
  // Declared by the reference with an empty body (src/Optimizer/Rewriter.cc:1605-1612); here it
  // checks that the module verifies.  The CPU lowering of the Frontend's nests is test
  // infrastructure and not part of the product library.
  static void loweringAffineDialect(mlir::ModuleOp module);
  // tileC[i, j] += fragA[i] * fragB[j] as an m x n loop nest at the builder's position.
  static mlir::AffineForOp outer_product(mlir::OpBuilder& builder, mlir::Value tileC, mlir::Value fragA, mlir::Value fragB,
                                         int64_t m, int64_t n);

  static void set_buffer(mlir::OpBuilder& builder, mlir::Value mem, mlir::Value targetValue);
  static mlir::AffineForOp create_constant_loop(mlir::OpBuilder& builder, int64_t lowerBound, int64_t upperBound,
                                                int64_t step);
};

}  // namespace KernelCodeGen
