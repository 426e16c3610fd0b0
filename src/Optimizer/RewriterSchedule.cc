// The later stages of the reference's SGEMM recipe on the mini IR: copy loops through affine maps
// (read / write), cached accesses, vectorisation, double buffering and the loop surgery around
// it.  Each primitive reproduces the structure its README.md stage shows (citations in
// include/Optimizer/Rewriter.h); the reference's implementations are src/Optimizer/Rewriter.cc:
// 601-738 (read / write), 745-762 (cache_*), 786-807 (vectorize), 809-1180 (pipeline),
// 1182-1284 (detach_last_loop / schedule / extract_loop), 1359-1572 (if folding, unroll),
// 1614-1692 (change_double_buffer, outer_product).
#include <algorithm>
#include <cassert>
#include <iostream>

#include "Optimizer/Rewriter.h"

namespace KernelCodeGen {

using kcgir::AffineExpr;
using kcgir::IndexExpr;
using kcgir::OpKind;

namespace {

int64_t elementCount(mlir::Value memref) {
  const mlir::Type type = memref.getType();     // by value: getShape() refers into it
  int64_t n = 1;
  for (int64_t d : type.getShape()) n *= d;
  return n;
}

std::vector<AffineExpr> asExprs(const llvm::SmallVector<mlir::Value>& operands) {
  std::vector<AffineExpr> out;
  for (auto v : operands) out.push_back(AffineExpr::value(v));
  return out;
}

// the memref an access op reads or writes, or a null value
mlir::Value accessedMemref(mlir::Operation* op) {
  switch (op->kind) {
    case OpKind::Load:
    case OpKind::VectorLoad: return op->operands.at(0);
    case OpKind::Store:
    case OpKind::VectorStore: return op->operands.at(1);
    default: return mlir::Value();
  }
}

// switches an access to the general index form (no-op when it is already there)
void toGeneralForm(mlir::Operation* op) {
  if (!op->exprs.empty() || op->indices.empty()) return;
  for (auto& e : op->indices) op->exprs.push_back(AffineExpr::fromLinear(e));
  op->indices.clear();
}

// index of dimension d0 for a 1-D register buffer holding `width`-element groups
std::vector<AffineExpr> flatIndex(mlir::Value buffer, const AffineExpr& e) {
  assert(buffer.getType().getShape().size() == 1 && "copy loops stage through 1-D register buffers");
  (void)buffer;
  return {e};
}

}  // namespace

mlir::AffineForOp Rewriter::read(mlir::OpBuilder& builder, mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                 llvm::SmallVector<mlir::Value> operands, int64_t width) {
  assert(src && dst && src.getType().isMemRef() && dst.getType().isMemRef());
  assert(map.getNumDims() == operands.size() + 1 && "read: the map takes the operands and the copy index");
  assert(map.getNumResults() == src.getType().getShape().size() && "read: one result per source dimension");
  const int64_t n = elementCount(dst);
  assert(width > 0 && n % width == 0);
  mlir::AffineForOp loop = builder.createFor(0, n / width, 1);
  mlir::OpBuilder b(builder.getContext());
  b.setInsertionPointToEnd(loop.getBody());
  auto args = asExprs(operands);
  args.push_back(AffineExpr::value(loop.getInductionVar()));
  mlir::Value v = b.createVectorLoad(src, map.apply(args), width);
  b.createVectorStore(v, dst, flatIndex(dst, AffineExpr::value(loop.getInductionVar()) * width), width);
  return loop;
}

mlir::AffineForOp Rewriter::read(mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                 llvm::SmallVector<mlir::Value> operands, int64_t width, mlir::AffineForOp compute_at,
                                 Position pos) {
  mlir::OpBuilder b = getBuilder(compute_at, pos);
  return read(b, src, dst, map, std::move(operands), width);
}

mlir::AffineForOp Rewriter::write(mlir::OpBuilder& builder, mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                  llvm::SmallVector<mlir::Value> operands, int64_t width) {
  assert(src && dst && src.getType().isMemRef() && dst.getType().isMemRef());
  assert(map.getNumResults() == dst.getType().getShape().size() && "write: one result per destination dimension");
  const int64_t n = elementCount(src);
  assert(width > 0 && n % width == 0);
  const size_t extra = map.getNumDims() - operands.size();
  assert((extra == 1 || extra == 2) && "write: the map takes the operands, the copy index and optionally the element index");
  mlir::AffineForOp loop = builder.createFor(0, n / width, 1);
  mlir::OpBuilder b(builder.getContext());
  b.setInsertionPointToEnd(loop.getBody());
  auto args = asExprs(operands);
  const AffineExpr iv = AffineExpr::value(loop.getInductionVar());
  args.push_back(iv);
  if (extra == 1) {
    mlir::Value v = b.createVectorLoad(src, flatIndex(src, iv * width), width);
    b.createVectorStore(v, dst, map.apply(args), width);
  } else {
    // element by element (the tile is stored transposed)
    mlir::AffineForOp inner = b.createFor(0, width, 1);
    mlir::OpBuilder ib(builder.getContext());
    ib.setInsertionPointToEnd(inner.getBody());
    const AffineExpr e = AffineExpr::value(inner.getInductionVar());
    args.push_back(e);
    mlir::Value v = ib.createVectorLoad(src, flatIndex(src, iv * width + e), 1);
    ib.createVectorStore(v, dst, map.apply(args), 1);
  }
  return loop;
}

mlir::AffineForOp Rewriter::write(mlir::Value src, mlir::Value dst, mlir::AffineMap map,
                                  llvm::SmallVector<mlir::Value> operands, int64_t width, mlir::AffineForOp compute_at,
                                  Position pos) {
  mlir::OpBuilder b = getBuilder(compute_at, pos);
  return write(b, src, dst, map, std::move(operands), width);
}

void Rewriter::cache_read(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached, mlir::AffineMap map,
                          llvm::SmallVector<mlir::Value> operands) {
  assert(map.getNumDims() <= operands.size());
  assert(map.getNumResults() == cached.getType().getShape().size());
  const auto idx = map.apply(asExprs(operands));
  scope->walk([&](mlir::Operation* op) {
    if (op->kind != OpKind::Load || op->operands[0] != src) return;
    op->operands[0] = cached;
    op->indices.clear();
    op->exprs.clear();
    // a purely linear index stays in the linear form (prints as a plain affine.load)
    std::vector<IndexExpr> lin(idx.size());
    bool all = true;
    for (size_t i = 0; i < idx.size(); ++i) all = all && idx[i].toLinear(&lin[i]);
    if (all) op->indices = lin;
    else op->exprs = idx;
  });
}

void Rewriter::cache_write(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached, mlir::AffineMap map,
                           llvm::SmallVector<mlir::Value> operands) {
  assert(map.getNumDims() <= operands.size());
  assert(map.getNumResults() == src.getType().getShape().size());
  (void)cached;   // the stores already take their value from loads of the cached tile
  const auto idx = map.apply(asExprs(operands));
  scope->walk([&](mlir::Operation* op) {
    if (op->kind != OpKind::Store || op->operands[1] != src) return;
    op->indices.clear();
    op->exprs = idx;
  });
}

mlir::AffineForOp Rewriter::vectorize(mlir::AffineForOp loop, int64_t width) {
  assert(width == 1 || width == 2 || width == 4 || width == 8);
  loop->setAttr("kcg.vectorize", width);
  if (width == 1 || loop.getStep() != 1 || loop.getNumIterOperands() != 0) return loop;
  if ((loop.getConstantUpperBound() - loop.getConstantLowerBound()) % width != 0) return loop;
  // the body must be straight-line loads and stores whose innermost index advances by one with
  // the loop and whose other indices do not depend on it.  The indices may contain floordiv / mod
  // of other values, so the dependence is probed numerically: three valuations of the other
  // leaves, the loop variable at 0 .. width - 1.
  const mlir::Value iv = loop.getInductionVar();
  for (mlir::Operation* op : loop.getBody()->ops) {
    if (op->kind != OpKind::Load && op->kind != OpKind::Store) return loop;
    const size_t rank = op->indexRank();
    if (rank == 0) return loop;
    for (int trial = 0; trial < 3; ++trial) {
      for (size_t d = 0; d < rank; ++d) {
        const AffineExpr e = op->indexExpr(d);
        auto at = [&](int64_t t) {
          return e.evaluate([&](mlir::Value v) -> int64_t {
            if (v == iv) return t;
            return static_cast<int64_t>((reinterpret_cast<uintptr_t>(v.impl()) >> 4) * (trial + 3) % 61);
          });
        };
        for (int64_t t = 1; t < width; ++t)
          if (at(t) - at(0) != (d + 1 == rank ? t : 0)) return loop;
      }
    }
  }
  loop->step = width;
  for (mlir::Operation* op : loop.getBody()->ops) {
    toGeneralForm(op);
    op->kind = op->kind == OpKind::Load ? OpKind::VectorLoad : OpKind::VectorStore;
    op->width = width;
  }
  return loop;
}

}  // namespace KernelCodeGen
