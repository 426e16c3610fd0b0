// Schedule primitives (reference: include/Optimizer/Rewriter.h:13-229).
//
// split / reorder / parallel / bufferizeLoopCarryVar / alloc_buffer / barrier transform the IR
// structurally, stage for stage as in the reference's README.md:28-190 snapshots.  The
// remaining primitives of the reference's SGEMM recipe (read, write, cache_read, cache_write,
// vectorize, pipeline, ...) describe register/shared-memory choreography that the tcgen05
// kernels do in hardware (TMA, swizzled shared memory, TMEM); here they validate their
// arguments and leave a `kcg.<name>` annotation in the IR, which the Backend turns into launch
// descriptor fields (e.g. pipeline depth -> stages).
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
  static mlir::Operation* vectorize(mlir::AffineForOp readOrWrite, int64_t width);
  // double buffering of `buffer` around `compute_at`: `stages` buffers in flight
  static mlir::Operation* pipeline(mlir::Value buffer, mlir::AffineForOp compute_at, int64_t stages = 2);
  static void unrollAttribute(mlir::ModuleOp module, const std::function<bool(mlir::AffineForOp)>& unrollCheckFn);

  // Loops of `parallelLevel`'s body that store into `dst` (outer to inner per nest).
  static std::vector<std::vector<mlir::AffineForOp>> get_write(mlir::AffineParallelOp parallelLevel, mlir::Value dst);

  static void set_buffer(mlir::OpBuilder& builder, mlir::Value mem, mlir::Value targetValue);
  static mlir::AffineForOp create_constant_loop(mlir::OpBuilder& builder, int64_t lowerBound, int64_t upperBound,
                                                int64_t step);
};

}  // namespace KernelCodeGen
