// Schedule primitives on the mini IR.  The four structural ones reproduce, stage by stage, the
// loop structures of the reference's README.md:28-190 (split -> reorder -> parallel ->
// bufferize -> reorder -> split K); see include/Optimizer/Rewriter.h for the contract.
#include "Optimizer/Rewriter.h"

#include <algorithm>
#include <cassert>
#include <iostream>

namespace KernelCodeGen {

using kcgir::IndexExpr;
using kcgir::OpKind;

namespace {

mlir::Operation* rootOf(mlir::Operation* op) {
  while (op->getParentOp() && op->getParentOp()->kind != OpKind::Module) op = op->getParentOp();
  return op;
}

bool isAncestor(mlir::Operation* anc, mlir::Operation* op) {
  for (mlir::Operation* p = op->getParentOp(); p; p = p->getParentOp())
    if (p == anc) return true;
  return false;
}

// Moves every operation of `from` to the end of `to`.
void spliceBody(mlir::Block* from, mlir::Block* to) {
  for (mlir::Operation* op : from->ops) {
    op->parent = to;
    to->ops.push_back(op);
  }
  from->ops.clear();
}

mlir::Operation* enclosingParallel(mlir::Operation* op) {
  for (mlir::Operation* p = op->getParentOp(); p; p = p->getParentOp())
    if (p->kind == OpKind::Parallel) return p;
  return nullptr;
}

}  // namespace

mlir::OpBuilder Rewriter::getBuilder(mlir::AffineForOp op, Position pos) {
  mlir::OpBuilder b(op->getContext());
  switch (pos) {
    case Position::before: b.setInsertionPoint(op); break;
    case Position::after: b.setInsertionPointAfter(op); break;
    case Position::begin: b.setInsertionPointToStart(op.getBody()); break;
    case Position::end: b.setInsertionPointToEnd(op.getBody()); break;
  }
  return b;
}

std::vector<mlir::AffineForOp> Rewriter::split(mlir::AffineForOp forOp, uint64_t num_output,
                                               std::vector<int64_t>&& factors) {
  assert(forOp && forOp.getNumIterOperands() == 0 && "split: loops with iter_args are not splittable");
  assert(factors.size() + 1 == num_output && "split: need num_output - 1 tile sizes");
  std::sort(factors.begin(), factors.end(), std::greater<int64_t>());
  const int64_t lb = forOp.getConstantLowerBound(), ub = forOp.getConstantUpperBound();
  assert(forOp.getStep() == 1 && "split: unit-step loops only");
  int64_t span = ub - lb;
  for (int64_t f : factors) {
    assert(f > 0 && span % f == 0 && "split: tile sizes must divide evenly");
    span = f;
  }
  mlir::OpBuilder builder(forOp->getContext());
  builder.setInsertionPoint(forOp);
  std::vector<mlir::AffineForOp> loops;
  IndexExpr sum;
  for (uint64_t i = 0; i < num_output; ++i) {
    const int64_t l = i == 0 ? lb : 0;
    const int64_t u = i == 0 ? ub : factors[i - 1];
    const int64_t s = i + 1 < num_output ? factors[i] : 1;
    mlir::AffineForOp loop = builder.createFor(l, u, s);
    loops.push_back(loop);
    sum = sum + IndexExpr(loop.getInductionVar());
    builder.setInsertionPointToEnd(loop.getBody());
  }
  spliceBody(forOp.getBody(), loops.back().getBody());
  loops.back()->substituteIndex(forOp.getInductionVar(), sum);
  for (auto& kv : forOp->attrs) loops.front()->attrs[kv.first] = kv.second;
  forOp->erase();
  return loops;
}

mlir::Value Rewriter::bufferizeLoopCarryVar(std::vector<mlir::AffineForOp>& loops) {
  assert(!loops.empty());
  mlir::AffineForOp kLoop = loops[0];
  assert(kLoop.getNumIterOperands() == 1 && "bufferize: the first loop must carry exactly one value");
  std::vector<int64_t> shape;
  std::vector<IndexExpr> idx;
  for (size_t i = 1; i < loops.size(); ++i) {
    assert(loops[i].getConstantLowerBound() == 0 && loops[i].getStep() == 1);
    shape.push_back(loops[i].tripCount());
    idx.emplace_back(loops[i].getInductionVar());
  }
  if (shape.empty()) {
    shape.push_back(1);
    idx.push_back(IndexExpr::cst(0));
  }
  const mlir::Type elem = kLoop.getRegionIterArg(0).getType();
  // the buffer lives at the top of the enclosing parallel level (per-thread accumulator tile)
  mlir::Operation* scope = enclosingParallel(kLoop);
  if (!scope) scope = rootOf(kLoop);
  mlir::Value buf = alloc_buffer(scope, MemorySpace::local, shape, elem);

  mlir::OpBuilder b(kLoop->getContext());
  // init
  b.setInsertionPoint(kLoop);
  b.createStore(kLoop->operands[0], buf, idx);
  // body: load at the top replaces the carried value, the yield becomes a store
  mlir::Block* body = kLoop.getBody();
  b.setInsertionPointToStart(body);
  mlir::Value cur = b.createLoad(buf, idx);
  const mlir::Value carried = kLoop.getRegionIterArg(0);
  kLoop->replaceUsesOfWith(carried, cur);
  mlir::Operation* yield = body->ops.back();
  assert(yield->kind == OpKind::Yield);
  b.setInsertionPoint(yield);
  b.createStore(yield->operands[0], buf, idx);
  yield->erase();
  body->args.resize(1);
  // result
  b.setInsertionPointAfter(kLoop);
  mlir::Value fin = b.createLoad(buf, idx);
  const mlir::Value oldResult = kLoop.getResult(0);
  mlir::Operation* finDef = fin.getDefiningOp();
  rootOf(kLoop)->walk([&](mlir::Operation* op) {
    if (op == finDef) return;
    for (auto& v : op->operands) if (v == oldResult) v = fin;
  });
  kLoop->operands.clear();
  kLoop->results.clear();
  return buf;
}

void Rewriter::reorder(const std::vector<mlir::AffineForOp>& wanted) {
  const size_t n = wanted.size();
  if (n < 2) return;
  // current nesting order, outermost first
  std::vector<mlir::AffineForOp> cur = wanted;
  std::sort(cur.begin(), cur.end(), [](const mlir::AffineForOp& a, const mlir::AffineForOp& b) {
    return isAncestor(a, b);
  });
  // std::sort needs a strict weak order; ancestor-of is one on a chain, verify the chain
  for (size_t i = 0; i + 1 < n; ++i) {
    assert(cur[i + 1]->getParentOp() == cur[i].getOperation() && "reorder: loops must be directly nested");
    assert(cur[i].getNumIterOperands() == 0 && "reorder: loops with iter_args cannot be re-nested");
  }
  mlir::OpBuilder b(cur[0]->getContext());

  // 1. distribute operations that sit beside a nested loop into copies of the enclosing loops
  mlir::Operation* postAnchor = cur[0];
  auto makeChain = [&](size_t level, std::vector<mlir::Operation*>& ops, bool before) {
    // new loops equal to cur[0..level], holding `ops`
    if (before) b.setInsertionPoint(cur[0]);
    else b.setInsertionPointAfter(postAnchor);
    std::vector<mlir::AffineForOp> chain;
    for (size_t i = 0; i <= level; ++i) {
      mlir::AffineForOp l = b.createFor(cur[i].getConstantLowerBound(), cur[i].getConstantUpperBound(), cur[i].getStep());
      chain.push_back(l);
      b.setInsertionPointToEnd(l.getBody());
    }
    for (mlir::Operation* op : ops) {
      op->erase();
      op->parent = chain.back().getBody();
      chain.back().getBody()->ops.push_back(op);
    }
    for (size_t i = 0; i <= level; ++i)
      chain.back()->replaceUsesOfWith(cur[i].getInductionVar(), chain[i].getInductionVar());
    if (!before) postAnchor = chain.front();
  };
  for (size_t i = 0; i + 1 < n; ++i) {  // pre groups: outer levels first keeps program order
    std::vector<mlir::Operation*> pre;
    for (mlir::Operation* op : cur[i].getBody()->ops) {
      if (op == cur[i + 1].getOperation()) break;
      pre.push_back(op);
    }
    if (!pre.empty()) makeChain(i, pre, true);
  }
  for (size_t ii = n - 1; ii-- > 0;) {  // post groups: inner levels first
    std::vector<mlir::Operation*> post;
    bool seen = false;
    for (mlir::Operation* op : cur[ii].getBody()->ops) {
      if (seen) post.push_back(op);
      if (op == cur[ii + 1].getOperation()) seen = true;
    }
    if (!post.empty()) makeChain(ii, post, false);
  }

  // 2. the nest is perfect now: re-nest in the wanted order
  std::vector<mlir::Operation*> innerOps(cur[n - 1].getBody()->ops.begin(), cur[n - 1].getBody()->ops.end());
  cur[n - 1].getBody()->ops.clear();
  mlir::Block* outerBlock = cur[0]->parent;
  auto& outerOps = outerBlock->ops;
  auto pos = std::find(outerOps.begin(), outerOps.end(), cur[0].getOperation());
  pos = outerOps.erase(pos);
  cur[0]->parent = nullptr;
  for (size_t i = 1; i < n; ++i) {
    cur[i]->parent->ops.clear();
    cur[i]->parent = nullptr;
  }
  outerOps.insert(pos, wanted[0]);
  wanted[0]->parent = outerBlock;
  for (size_t i = 1; i < n; ++i) {
    wanted[i - 1].getBody()->ops.clear();
    wanted[i - 1].getBody()->ops.push_back(wanted[i]);
    wanted[i]->parent = wanted[i - 1].getBody();
  }
  mlir::Block* innermost = wanted[n - 1].getBody();
  innermost->ops.clear();
  for (mlir::Operation* op : innerOps) {
    op->parent = innermost;
    innermost->ops.push_back(op);
  }
}

mlir::AffineParallelOp Rewriter::parallel(const std::vector<mlir::AffineForOp>& loops) {
  assert(!loops.empty() && loops.size() <= 3 && "parallel: one to three loops");
  for (size_t i = 0; i + 1 < loops.size(); ++i) {
    assert(loops[i].getBody()->ops.size() == 1 && loops[i].getBody()->ops.front() == loops[i + 1].getOperation() &&
           "parallel: loops must be perfectly nested");
  }
  mlir::OpBuilder b(loops[0]->getContext());
  b.setInsertionPoint(loops[0]);
  std::vector<int64_t> extents;
  for (auto& l : loops) {
    assert(l.getNumIterOperands() == 0);
    extents.push_back(l.tripCount());
  }
  const std::string level = enclosingParallel(loops[0]) ? "block" : "grid";
  mlir::AffineParallelOp par = b.createParallel(extents, level);
  b.setInsertionPointToEnd(par.getBody());
  auto ivs = par.getIVs();
  mlir::Block* inner = loops.back().getBody();
  for (size_t i = 0; i < loops.size(); ++i) {
    const int64_t step = loops[i].getStep(), lb = loops[i].getConstantLowerBound();
    IndexExpr repl(ivs[i]);
    if (step != 1 || lb != 0) {
      IndexExpr e = IndexExpr(ivs[i]) * step + IndexExpr::cst(lb);
      repl = IndexExpr(b.createApply(e));
    }
    loops.back()->substituteIndex(loops[i].getInductionVar(), repl);
  }
  spliceBody(inner, par.getBody());
  loops[0]->erase();
  return par;
}

mlir::Value Rewriter::alloc_buffer(mlir::Operation* father, MemorySpace ms, const std::vector<int64_t>& shape,
                                   mlir::Type dtype) {
  assert(father && father->body);
  mlir::OpBuilder b(father->getContext());
  b.setInsertionPointToStart(father->body);
  return b.createAlloc(mlir::Type::memRef(shape, dtype.elem, static_cast<int>(ms)));
}

mlir::Value Rewriter::alloc_buffer(mlir::Operation* contextOp, Position pos, MemorySpace ms,
                                   const std::vector<int64_t>& shape, mlir::Type dtype) {
  mlir::OpBuilder b(contextOp->getContext());
  if (pos == Position::before) b.setInsertionPoint(contextOp);
  else if (pos == Position::after) b.setInsertionPointAfter(contextOp);
  else assert(false && "alloc_buffer: before/after only");
  return b.createAlloc(mlir::Type::memRef(shape, dtype.elem, static_cast<int>(ms)));
}

mlir::gpu::BarrierOp Rewriter::barrier(mlir::AffineForOp compute_at, Position pos) {
  mlir::OpBuilder b = getBuilder(compute_at, pos);
  return b.createBarrier();
}

static mlir::Operation* annotate(mlir::AffineForOp at, Position pos, const std::string& name,
                                 const std::vector<mlir::Value>& operands) {
  mlir::OpBuilder b = Rewriter::getBuilder(at, pos);
  return b.createAnnotation(name, operands);
}

mlir::Operation* Rewriter::read(mlir::Value src, mlir::Value dst, int64_t width, mlir::AffineForOp compute_at,
                                Position pos) {
  assert(src && dst && src.getType().isMemRef() && dst.getType().isMemRef());
  mlir::Operation* op = annotate(compute_at, pos, "read", {src, dst});
  op->setAttr("width", width);
  return op;
}

mlir::Operation* Rewriter::write(mlir::Value src, mlir::Value dst, int64_t width, mlir::AffineForOp compute_at,
                                 Position pos) {
  assert(src && dst && src.getType().isMemRef() && dst.getType().isMemRef());
  mlir::Operation* op = annotate(compute_at, pos, "write", {src, dst});
  op->setAttr("width", width);
  return op;
}

void Rewriter::cache_read(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached) {
  annotate(scope, Position::begin, "cache_read", {src, cached});
}

void Rewriter::cache_write(mlir::AffineForOp scope, mlir::Value src, mlir::Value cached) {
  annotate(scope, Position::begin, "cache_write", {src, cached});
}

mlir::Operation* Rewriter::pipeline(mlir::Value buffer, mlir::AffineForOp compute_at, int64_t stages) {
  assert(stages >= 2);
  mlir::Operation* op = annotate(compute_at, Position::begin, "pipeline", {buffer});
  op->setAttr("stages", stages);
  return op;
}

void Rewriter::unrollAttribute(mlir::ModuleOp module, const std::function<bool(mlir::AffineForOp)>& unrollCheckFn) {
  module->walk([&](mlir::Operation* op) {
    if (op->kind == OpKind::For && unrollCheckFn(mlir::AffineForOp(op)))
      op->setAttr("affine.loop", std::string("unroll"));
  });
}

std::vector<std::vector<mlir::AffineForOp>> Rewriter::get_write(mlir::AffineParallelOp parallelLevel, mlir::Value dst) {
  std::vector<std::vector<mlir::AffineForOp>> results;
  parallelLevel->walk([&](mlir::Operation* op) {
    if (op->kind != OpKind::Store || op->operands[1] != dst) return;
    std::vector<mlir::AffineForOp> nest;
    for (mlir::Operation* p = op->getParentOp(); p && p != parallelLevel.getOperation(); p = p->getParentOp())
      if (p->kind == OpKind::For) nest.insert(nest.begin(), mlir::AffineForOp(p));
    results.push_back(std::move(nest));
  });
  return results;
}

void Rewriter::set_buffer(mlir::OpBuilder& builder, mlir::Value mem, mlir::Value targetValue) {
  const auto shape = mem.getType().getShape();
  std::vector<int64_t> zeros(shape.size(), 0), ones(shape.size(), 1);
  builder.buildAffineLoopNest(zeros, shape, ones, [&](mlir::OpBuilder& nb, const std::vector<mlir::Value>& ivs) {
    nb.createStore(targetValue, mem, std::vector<IndexExpr>(ivs.begin(), ivs.end()));
  });
}

mlir::AffineForOp Rewriter::create_constant_loop(mlir::OpBuilder& builder, int64_t lowerBound, int64_t upperBound,
                                                 int64_t step) {
  return builder.createFor(lowerBound, upperBound, step);
}

}  // namespace KernelCodeGen
