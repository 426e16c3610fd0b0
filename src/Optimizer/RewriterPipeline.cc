// Double buffering and the loop surgery around it (see include/Optimizer/Rewriter.h and the file
// comment of RewriterSchedule.cc for the reference's counterparts).
#include <algorithm>
#include <cassert>
#include <functional>
#include <iostream>
#include <unordered_map>

#include "Optimizer/Rewriter.h"

namespace KernelCodeGen {

using kcgir::AffineExpr;
using kcgir::IndexExpr;
using kcgir::OpKind;

namespace {

mlir::Value accessedMemref(mlir::Operation* op) {
  switch (op->kind) {
    case OpKind::Load:
    case OpKind::VectorLoad: return op->operands.at(0);
    case OpKind::Store:
    case OpKind::VectorStore: return op->operands.at(1);
    default: return mlir::Value();
  }
}

void toGeneralForm(mlir::Operation* op) {
  if (!op->exprs.empty() || op->indices.empty()) return;
  for (auto& e : op->indices) op->exprs.push_back(AffineExpr::fromLinear(e));
  op->indices.clear();
}

// Deep copy of `op` placed at the builder's position; values defined inside are remapped, values
// from outside are shared.
mlir::Operation* cloneInto(mlir::OpBuilder& b, mlir::Operation* src, std::unordered_map<kcgir::ValueImpl*, kcgir::ValueImpl*>& vmap) {
  kcgir::Context* ctx = b.getContext();
  mlir::Operation* dst = ctx->newOp(src->kind);
  dst->name = src->name;
  dst->attrs = src->attrs;
  dst->lb = src->lb;
  dst->ub = src->ub;
  dst->step = src->step;
  dst->extents = src->extents;
  dst->fvalue = src->fvalue;
  dst->resultTypes = src->resultTypes;
  dst->width = src->width;
  dst->ivalue = src->ivalue;
  auto remap = [&](mlir::Value v) {
    auto it = vmap.find(v.impl());
    return it == vmap.end() ? v : mlir::Value(it->second);
  };
  for (auto v : src->operands) dst->operands.push_back(remap(v));
  for (auto& e : src->indices) {
    IndexExpr ne;
    ne.constant = e.constant;
    for (auto& t : e.terms) ne.terms.emplace_back(remap(t.first), t.second);
    dst->indices.push_back(std::move(ne));
  }
  for (auto& e : src->exprs) dst->exprs.push_back(e.mapValues(remap));
  dst->cond = src->cond.mapValues(remap);
  for (size_t i = 0; i < src->results.size(); ++i) {
    kcgir::ValueImpl* nv = ctx->newValue(src->results[i]->type, dst, nullptr, static_cast<int>(i));
    vmap[src->results[i]] = nv;
    dst->results.push_back(nv);
  }
  b.insert(dst);
  if (src->body) {
    dst->body = ctx->newBlock(dst);
    for (size_t i = 0; i < src->body->args.size(); ++i) {
      kcgir::ValueImpl* na = ctx->newValue(src->body->args[i]->type, nullptr, dst->body, static_cast<int>(i));
      vmap[src->body->args[i]] = na;
      dst->body->args.push_back(na);
    }
    mlir::OpBuilder inner(ctx);
    inner.setInsertionPointToEnd(dst->body);
    for (mlir::Operation* child : src->body->ops) cloneInto(inner, child, vmap);
  }
  return dst;
}

mlir::Operation* cloneInto(mlir::OpBuilder& b, mlir::Operation* src) {
  std::unordered_map<kcgir::ValueImpl*, kcgir::ValueImpl*> vmap;
  return cloneInto(b, src, vmap);
}

// moves the operations of `from` in front of `before` (same order) and leaves `from` empty
void spliceBefore(mlir::Block* from, mlir::Operation* before) {
  std::vector<mlir::Operation*> ops(from->ops.begin(), from->ops.end());
  from->ops.clear();
  for (mlir::Operation* op : ops) {
    op->parent = nullptr;
    mlir::OpBuilder b(before->getContext());
    b.setInsertionPoint(before);
    b.insert(op);
  }
}

// `arith.constant v : index` at the top of the block that holds the outermost loop around
// `anchor` (where the reference hoists the constants it substitutes for induction variables), so
// that later moves and copies of the operations using it stay in its scope.
mlir::Value hoistedIndexConstant(mlir::Operation* anchor, int64_t v) {
  mlir::Operation* root = anchor;
  while (mlir::Operation* p = root->getParentOp()) {
    if (p->kind != OpKind::For && p->kind != OpKind::If) break;
    root = p;
  }
  // reuse a constant of the same value that already stands at the top of that block
  for (mlir::Operation* op : root->parent->ops) {
    if (op->kind != OpKind::IndexConstant) break;
    if (op->ivalue == v) return op->getResult(0);
  }
  mlir::OpBuilder b(anchor->getContext());
  b.setInsertionPointToStart(root->parent);
  return b.createIndexConstant(v);
}

// smallest and largest value an index operand of an affine.if can take (a loop's or a parallel
// level's induction variable, or an index constant)
bool valueRange(mlir::Value v, int64_t* lo, int64_t* hi) {
  if (mlir::Operation* def = v.getDefiningOp()) {
    if (def->kind != OpKind::IndexConstant) return false;
    *lo = *hi = def->ivalue;
    return true;
  }
  mlir::Block* owner = v.getOwnerBlock();
  mlir::Operation* parent = owner ? owner->parentOp : nullptr;
  if (!parent) return false;
  if (parent->kind == OpKind::For && v == mlir::Value(owner->args.at(0))) {
    if (parent->ub <= parent->lb) return false;
    *lo = parent->lb;
    *hi = parent->lb + ((parent->ub - 1 - parent->lb) / parent->step) * parent->step;
    return true;
  }
  if (parent->kind == OpKind::Parallel) {
    for (size_t i = 0; i < owner->args.size(); ++i)
      if (v == mlir::Value(owner->args[i])) {
        *lo = 0;
        *hi = parent->extents.at(i) - 1;
        return true;
      }
  }
  return false;
}

// The condition of an affine.if at the extreme values of its operands.  Conditions here are
// monotone in every operand (a bound on one induction variable), so the two corners decide:
// +1 always true, -1 always false, 0 undecided.
int decideIf(mlir::Operation* ifOp) {
  std::vector<mlir::Value> leaves;
  ifOp->cond.collectValues(leaves);
  std::unordered_map<kcgir::ValueImpl*, std::pair<int64_t, int64_t>> range;
  for (auto v : leaves) {
    int64_t lo = 0, hi = 0;
    if (!valueRange(v, &lo, &hi)) return 0;
    range[v.impl()] = {lo, hi};
  }
  const int64_t atMin = ifOp->cond.evaluate([&](mlir::Value v) { return range[v.impl()].first; });
  const int64_t atMax = ifOp->cond.evaluate([&](mlir::Value v) { return range[v.impl()].second; });
  if (atMin >= 0 && atMax >= 0) return 1;
  if (atMin < 0 && atMax < 0) return -1;
  return 0;
}

}  // namespace

std::vector<std::vector<mlir::AffineForOp>> Rewriter::pipeline(std::vector<mlir::AffineForOp> readBodys,
                                                               mlir::Value& buffer, mlir::AffineForOp compute_at) {
  assert(!readBodys.empty() && buffer && buffer.getType().isMemRef());
  mlir::Operation* oldAlloc = buffer.getDefiningOp();
  assert(oldAlloc && oldAlloc->kind == OpKind::Alloc && "pipeline: the buffer must come from alloc_buffer");
  const int64_t lb = compute_at.getConstantLowerBound(), ub = compute_at.getConstantUpperBound();
  const int64_t step = compute_at.getStep();
  const mlir::Value iv = compute_at.getInductionVar();
  for (auto body : readBodys) {
    bool inside = false;
    for (mlir::Operation* p = body->getParentOp(); p; p = p->getParentOp()) inside = inside || p == compute_at.getOperation();
    assert(inside && "pipeline: the copy loops must sit inside the loop they are pipelined around");
    (void)inside;
  }

  // 1. the buffer doubles: [2, old shape...]
  const mlir::Type oldType = buffer.getType();
  std::vector<int64_t> shape{2};
  shape.insert(shape.end(), oldType.getShape().begin(), oldType.getShape().end());
  mlir::OpBuilder ab(oldAlloc->getContext());
  ab.setInsertionPoint(oldAlloc);
  const mlir::Value doubled = ab.createAlloc(mlir::Type::memRef(shape, oldType.elem, oldType.getMemorySpace()));

  // 2. copies of the read bodies in front of the loop: first iteration, half 0
  std::vector<mlir::AffineForOp> before, within;
  mlir::OpBuilder pb(compute_at->getContext());
  pb.setInsertionPoint(compute_at);
  const mlir::Value first = hoistedIndexConstant(compute_at, lb);
  for (auto body : readBodys) {
    mlir::Operation* copy = cloneInto(pb, body);
    copy->replaceUsesOfWith(iv, first);
    copy->walk([&](mlir::Operation* op) {
      if (accessedMemref(op) != buffer) return;
      toGeneralForm(op);
      op->exprs.insert(op->exprs.begin(), AffineExpr::constant(0));
      op->operands[op->kind == OpKind::Load || op->kind == OpKind::VectorLoad ? 0 : 1] = doubled;
    });
    before.push_back(mlir::AffineForOp(copy));
  }

  // 3. every access inside the loop selects the half of the current iteration ...
  const AffineExpr half = AffineExpr::value(iv).floorDiv(step) % 2;
  compute_at->walk([&](mlir::Operation* op) {
    if (accessedMemref(op) != buffer) return;
    toGeneralForm(op);
    op->exprs.insert(op->exprs.begin(), half);
    op->operands[op->kind == OpKind::Load || op->kind == OpKind::VectorLoad ? 0 : 1] = doubled;
  });

  // 4. ... and the read bodies run one iteration ahead, guarded: iv + 2 * step <= ub
  mlir::OpBuilder ib(compute_at->getContext());
  ib.setInsertionPoint(readBodys.front());
  mlir::Operation* guard = ib.createIf(AffineExpr::value(iv) * -1 + AffineExpr::constant(ub - 2 * step));
  for (auto body : readBodys) {
    body->erase();
    mlir::OpBuilder gb(compute_at->getContext());
    gb.setInsertionPointToEnd(guard->body);
    gb.insert(body);
    body->substituteExpr(iv, AffineExpr::value(iv) + AffineExpr::constant(step));
    within.push_back(body);
  }
  // the guard itself still tests the un-shifted induction variable
  guard->cond = AffineExpr::value(iv) * -1 + AffineExpr::constant(ub - 2 * step);

  // 5. no access to the old buffer may remain
  mlir::Operation* root = oldAlloc->getParentOp();
  bool stale = false;
  root->walk([&](mlir::Operation* op) { stale = stale || accessedMemref(op) == buffer; });
  assert(!stale && "pipeline: the buffer is accessed outside the pipelined loop");
  (void)stale;
  oldAlloc->erase();
  buffer = doubled;
  return {before, within};
}

void Rewriter::change_double_buffer(mlir::AffineForOp scope, mlir::Value buffer) {
  scope->walk([&](mlir::Operation* op) {
    if (op->kind != OpKind::VectorLoad || op->operands[0] != buffer || op->exprs.empty()) return;
    // first index x mod 2 -> (x + 1) mod 2
    const AffineExpr e = op->exprs[0];
    assert(e.kind() == AffineExpr::Kind::Mod && e.rhs().constantValue() == 2 &&
           "change_double_buffer: the first index selects a half");
    op->exprs[0] = (e.lhs() + 1) % 2;
  });
}

void Rewriter::detach_last_loop(mlir::AffineForOp forOp) {
  assert(forOp.getNumIterOperands() == 0);
  const int64_t step = forOp.getStep(), ub = forOp.getConstantUpperBound();
  assert(ub - step >= forOp.getConstantLowerBound());
  mlir::OpBuilder b = getBuilder(forOp, Position::after);
  const mlir::Value last = hoistedIndexConstant(forOp, ub - step);
  mlir::Operation* copy = cloneInto(b, forOp);
  copy->replaceUsesOfWith(mlir::Value(copy->body->args.at(0)), last);
  spliceBefore(copy->body, copy);
  copy->erase();
  forOp->ub = ub - step;
}

void Rewriter::schedule(mlir::Operation* srcOp, mlir::Operation* dstOp, Position pos) {
  assert(srcOp && dstOp && srcOp != dstOp);
  switch (pos) {
    case Position::after: srcOp->moveAfter(dstOp); break;
    case Position::before: srcOp->moveBefore(dstOp); break;
    case Position::end: {
      assert(dstOp->kind == OpKind::For && "schedule(end): the destination must be a loop");
      srcOp->erase();
      mlir::OpBuilder b(dstOp->getContext());
      b.setInsertionPointToEnd(dstOp->body);
      b.insert(srcOp);
      break;
    }
    default: assert(false && "schedule: before, after or end");
  }
}

void Rewriter::extract_loop(mlir::Operation* srcOp, mlir::AffineForOp forOp, int64_t iteration) {
  mlir::OpBuilder b(forOp->getContext());
  b.setInsertionPoint(forOp);
  const mlir::Value at = hoistedIndexConstant(forOp, forOp.getConstantLowerBound() + iteration * forOp.getStep());
  mlir::Operation* copy = cloneInto(b, srcOp);
  copy->replaceUsesOfWith(forOp.getInductionVar(), at);
}

void Rewriter::take_off_true_if(mlir::ModuleOp module) {
  std::vector<mlir::Operation*> ifs;
  module->walk([&](mlir::Operation* op) {
    if (op->kind == OpKind::If) ifs.push_back(op);
  });
  for (mlir::Operation* op : ifs) {
    if (decideIf(op) != 1) continue;
    spliceBefore(op->body, op);
    op->erase();
  }
}

void Rewriter::delete_false_if(mlir::ModuleOp module) {
  std::vector<mlir::Operation*> ifs;
  module->walk([&](mlir::Operation* op) {
    if (op->kind == OpKind::If) ifs.push_back(op);
  });
  for (mlir::Operation* op : ifs)
    if (decideIf(op) == -1) op->erase();
}

void Rewriter::unroll(mlir::ModuleOp module, mlir::function_ref<bool(mlir::AffineForOp)> unrollCheckFn) {
  // innermost first, so that an unrolled outer loop copies already unrolled bodies
  std::vector<mlir::Operation*> loops;
  std::function<void(mlir::Operation*)> post = [&](mlir::Operation* op) {
    if (op->body) {
      std::vector<mlir::Operation*> kids(op->body->ops.begin(), op->body->ops.end());
      for (mlir::Operation* k : kids) post(k);
    }
    if (op->kind == OpKind::For) loops.push_back(op);
  };
  post(module.getOperation());
  for (mlir::Operation* loop : loops) {
    mlir::AffineForOp forOp(loop);
    if (forOp.getNumIterOperands() != 0 || !unrollCheckFn(forOp)) continue;
    mlir::OpBuilder b(loop->getContext());
    b.setInsertionPoint(loop);
    for (int64_t i = loop->lb; i < loop->ub; i += loop->step) {
      const mlir::Value at = hoistedIndexConstant(loop, i);
      mlir::Operation* copy = cloneInto(b, loop);
      copy->replaceUsesOfWith(mlir::Value(copy->body->args.at(0)), at);
      spliceBefore(copy->body, copy);
      copy->erase();
    }
    loop->erase();
  }
}

void Rewriter::loweringAffineDialect(mlir::ModuleOp module) {
  std::string why;
  if (!kcgir::verify(module, &why)) std::cerr << "loweringAffineDialect: the module does not verify: " << why << "\n";
}

mlir::AffineForOp Rewriter::outer_product(mlir::OpBuilder& builder, mlir::Value tileC, mlir::Value fragA, mlir::Value fragB,
                                          int64_t m, int64_t n) {
  mlir::AffineForOp outer = builder.createFor(0, m, 1);
  mlir::OpBuilder ob(builder.getContext());
  ob.setInsertionPointToEnd(outer.getBody());
  mlir::AffineForOp inner = ob.createFor(0, n, 1);
  mlir::OpBuilder ib(builder.getContext());
  ib.setInsertionPointToEnd(inner.getBody());
  const IndexExpr i(outer.getInductionVar()), j(inner.getInductionVar());
  mlir::Value a = ib.createLoad(fragA, {i});
  mlir::Value b = ib.createLoad(fragB, {j});
  mlir::Value c = ib.createLoad(tileC, {i, j});
  mlir::Value mul = ib.createBinary(OpKind::MulF, a, b);
  mlir::Value add = ib.createBinary(OpKind::AddF, mul, c);
  ib.createStore(add, tileC, {i, j});
  return outer;
}

}  // namespace KernelCodeGen
