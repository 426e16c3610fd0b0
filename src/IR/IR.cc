// Implementation of the mini affine IR declared in include/IR/IR.h: arena, builder, textual
// printer (MLIR-flavoured, so the schedule stages can be compared by eye with the snapshots in
// the reference's README.md:7-190), deep clone and a structural verifier.
#include "IR/IR.h"

#include <algorithm>
#include <iomanip>
#include <iostream>
#include <sstream>
#include <unordered_map>

namespace kcgir {

const char* scalarName(ScalarKind k) {
  switch (k) {
    case ScalarKind::F16: return "f16";
    case ScalarKind::BF16: return "bf16";
    case ScalarKind::F32: return "f32";
    case ScalarKind::F64: return "f64";
    case ScalarKind::Index: return "index";
    default: return "none";
  }
}

int scalarBytes(ScalarKind k) {
  switch (k) {
    case ScalarKind::F16:
    case ScalarKind::BF16: return 2;
    case ScalarKind::F32: return 4;
    case ScalarKind::F64:
    case ScalarKind::Index: return 8;
    default: return 0;
  }
}

std::string Type::str() const {
  if (!memref) return scalarName(elem);
  std::ostringstream os;
  os << "memref<";
  for (int64_t d : shape) os << d << "x";
  os << scalarName(elem);
  if (memorySpace != 0) os << ", " << memorySpace;
  os << ">";
  return os.str();
}

Type Value::getType() const { return impl_ ? impl_->type : Type(); }
Operation* Value::getDefiningOp() const { return impl_ ? impl_->def : nullptr; }
Block* Value::getOwnerBlock() const { return impl_ ? impl_->owner : nullptr; }

// ---- IndexExpr ----------------------------------------------------------------------------------
void IndexExpr::simplify() {
  std::vector<std::pair<Value, int64_t>> out;
  for (auto& t : terms) {
    bool merged = false;
    for (auto& o : out)
      if (o.first == t.first) { o.second += t.second; merged = true; break; }
    if (!merged) out.push_back(t);
  }
  out.erase(std::remove_if(out.begin(), out.end(), [](auto& t) { return t.second == 0; }), out.end());
  terms = std::move(out);
}

IndexExpr IndexExpr::operator+(const IndexExpr& o) const {
  IndexExpr r = *this;
  r.terms.insert(r.terms.end(), o.terms.begin(), o.terms.end());
  r.constant += o.constant;
  r.simplify();
  return r;
}

IndexExpr IndexExpr::operator*(int64_t f) const {
  IndexExpr r = *this;
  for (auto& t : r.terms) t.second *= f;
  r.constant *= f;
  r.simplify();
  return r;
}

bool IndexExpr::uses(Value v) const {
  for (auto& t : terms) if (t.first == v) return true;
  return false;
}

int64_t IndexExpr::coefficientOf(Value v) const {
  for (auto& t : terms) if (t.first == v) return t.second;
  return 0;
}

void IndexExpr::substitute(Value from, const IndexExpr& to) {
  const int64_t c = coefficientOf(from);
  if (c == 0) return;
  // keep the position of the replaced term so that printed sums stay in loop order
  std::vector<std::pair<Value, int64_t>> out;
  for (auto& t : terms) {
    if (t.first == from) {
      for (auto& n : to.terms) out.emplace_back(n.first, n.second * c);
    } else {
      out.push_back(t);
    }
  }
  terms = std::move(out);
  constant += to.constant * c;
  simplify();
}

// ---- Operation ----------------------------------------------------------------------------------
const char* opKindName(OpKind k) {
  switch (k) {
    case OpKind::Module: return "module";
    case OpKind::Func: return "func.func";
    case OpKind::Return: return "return";
    case OpKind::Call: return "func.call";
    case OpKind::Alloc: return "memref.alloc";
    case OpKind::For: return "affine.for";
    case OpKind::Parallel: return "affine.parallel";
    case OpKind::Yield: return "affine.yield";
    case OpKind::Apply: return "affine.apply";
    case OpKind::Load: return "affine.load";
    case OpKind::Store: return "affine.store";
    case OpKind::Constant: return "arith.constant";
    case OpKind::MulF: return "arith.mulf";
    case OpKind::AddF: return "arith.addf";
    case OpKind::MaxF: return "arith.maxf";
    case OpKind::DivF: return "arith.divf";
    case OpKind::Exp: return "math.exp";
    case OpKind::Barrier: return "gpu.barrier";
    case OpKind::Annotation: return "kcg.annotation";
    case OpKind::VectorLoad: return "affine.vector_load";
    case OpKind::VectorStore: return "affine.vector_store";
    case OpKind::If: return "affine.if";
    case OpKind::IndexConstant: return "arith.constant";
  }
  return "?";
}

int64_t Operation::getIntAttr(const std::string& key, int64_t dflt) const {
  auto it = attrs.find(key);
  if (it == attrs.end()) return dflt;
  if (auto p = std::get_if<int64_t>(&it->second)) return *p;
  return dflt;
}

std::string Operation::getStringAttr(const std::string& key, const std::string& dflt) const {
  auto it = attrs.find(key);
  if (it == attrs.end()) return dflt;
  if (auto p = std::get_if<std::string>(&it->second)) return *p;
  return dflt;
}

void Operation::erase() {
  if (!parent) return;
  parent->ops.remove(this);
  parent = nullptr;
}

void Operation::moveBefore(Operation* other) {
  erase();
  auto& ops = other->parent->ops;
  ops.insert(std::find(ops.begin(), ops.end(), other), this);
  parent = other->parent;
}

void Operation::moveAfter(Operation* other) {
  erase();
  auto& ops = other->parent->ops;
  auto it = std::find(ops.begin(), ops.end(), other);
  ops.insert(std::next(it), this);
  parent = other->parent;
}

void Operation::walk(const std::function<void(Operation*)>& fn) {
  fn(this);
  if (body) {
    std::vector<Operation*> snapshot(body->ops.begin(), body->ops.end());
    for (Operation* op : snapshot) op->walk(fn);
  }
}

void Operation::replaceUsesOfWith(Value from, Value to) {
  walk([&](Operation* op) {
    for (auto& v : op->operands) if (v == from) v = to;
    for (auto& e : op->indices) {
      for (auto& t : e.terms) if (t.first == from) t.first = to;
      e.simplify();
    }
    for (auto& e : op->exprs) e = e.replaceValue(from, AffineExpr::value(to));
    if (op->kind == OpKind::If) op->cond = op->cond.replaceValue(from, AffineExpr::value(to));
  });
}

void Operation::substituteIndex(Value from, const IndexExpr& to) {
  const AffineExpr general = AffineExpr::fromLinear(to);
  walk([&](Operation* op) {
    for (auto& e : op->indices) e.substitute(from, to);
    for (auto& e : op->exprs) e = e.replaceValue(from, general);
    if (op->kind == OpKind::If) op->cond = op->cond.replaceValue(from, general);
  });
}

void Operation::substituteExpr(Value from, const AffineExpr& to) {
  IndexExpr linear;
  if (to.toLinear(&linear)) {
    substituteIndex(from, linear);
    return;
  }
  walk([&](Operation* op) {
    bool used = false;
    for (auto& e : op->indices) used = used || e.uses(from);
    if (used && op->kind != OpKind::Apply) {
      // the access leaves the linear form
      for (auto& e : op->indices) op->exprs.push_back(AffineExpr::fromLinear(e));
      op->indices.clear();
    }
    for (auto& e : op->exprs) e = e.replaceValue(from, to);
    if (op->kind == OpKind::If) op->cond = op->cond.replaceValue(from, to);
  });
}

AffineExpr Operation::indexExpr(size_t d) const {
  return exprs.empty() ? AffineExpr::fromLinear(indices.at(d)) : exprs.at(d);
}

// ---- Context ------------------------------------------------------------------------------------
Operation* Context::newOp(OpKind k) {
  ops_.push_back(std::make_unique<Operation>());
  Operation* op = ops_.back().get();
  op->kind = k;
  op->ctx = this;
  return op;
}

Block* Context::newBlock(Operation* parent) {
  blocks_.push_back(std::make_unique<Block>());
  Block* b = blocks_.back().get();
  b->parentOp = parent;
  return b;
}

ValueImpl* Context::newValue(Type t, Operation* def, Block* owner, int index) {
  values_.push_back(std::make_unique<ValueImpl>());
  ValueImpl* v = values_.back().get();
  v->type = std::move(t);
  v->def = def;
  v->owner = owner;
  v->index = index;
  return v;
}

// ---- handles ------------------------------------------------------------------------------------
ModuleOp ModuleOp::create(Context* ctx, const std::string& name) {
  Operation* op = ctx->newOp(OpKind::Module);
  op->name = name;
  op->body = ctx->newBlock(op);
  return ModuleOp(op);
}

std::vector<Value> AffineParallelOp::getIVs() const {
  std::vector<Value> ivs;
  for (auto* a : op_->body->args) ivs.emplace_back(a);
  return ivs;
}

namespace {

Operation* cloneOp(Operation* src, Context* ctx, std::unordered_map<ValueImpl*, ValueImpl*>& vmap) {
  Operation* dst = ctx->newOp(src->kind);
  dst->name = src->name;
  dst->attrs = src->attrs;
  dst->lb = src->lb;
  dst->ub = src->ub;
  dst->step = src->step;
  dst->extents = src->extents;
  dst->fvalue = src->fvalue;
  dst->resultTypes = src->resultTypes;
  auto remap = [&](Value v) {
    auto it = vmap.find(v.impl());
    return it == vmap.end() ? v : Value(it->second);
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
  dst->width = src->width;
  dst->ivalue = src->ivalue;
  for (size_t i = 0; i < src->results.size(); ++i) {
    ValueImpl* nv = ctx->newValue(src->results[i]->type, dst, nullptr, static_cast<int>(i));
    vmap[src->results[i]] = nv;
    dst->results.push_back(nv);
  }
  if (src->body) {
    dst->body = ctx->newBlock(dst);
    for (size_t i = 0; i < src->body->args.size(); ++i) {
      ValueImpl* na = ctx->newValue(src->body->args[i]->type, nullptr, dst->body, static_cast<int>(i));
      vmap[src->body->args[i]] = na;
      dst->body->args.push_back(na);
    }
    for (Operation* child : src->body->ops) {
      Operation* c = cloneOp(child, ctx, vmap);
      c->parent = dst->body;
      dst->body->ops.push_back(c);
    }
  }
  return dst;
}

}  // namespace

Operation* ModuleOp::clone() const {
  std::unordered_map<ValueImpl*, ValueImpl*> vmap;
  return cloneOp(op_, op_->ctx, vmap);
}

// ---- OpBuilder ----------------------------------------------------------------------------------
void OpBuilder::setInsertionPointAfter(Operation* op) {
  ip_.block = op->parent;
  auto& ops = op->parent->ops;
  auto it = std::find(ops.begin(), ops.end(), op);
  ++it;
  ip_.before = (it == ops.end()) ? nullptr : *it;
}

Operation* OpBuilder::insert(Operation* op) {
  assert(ip_.block && "builder has no insertion point");
  auto& ops = ip_.block->ops;
  if (ip_.before) ops.insert(std::find(ops.begin(), ops.end(), ip_.before), op);
  else ops.push_back(op);
  op->parent = ip_.block;
  return op;
}

static Value addResult(Context* ctx, Operation* op, const Type& t) {
  ValueImpl* v = ctx->newValue(t, op, nullptr, static_cast<int>(op->results.size()));
  op->results.push_back(v);
  return Value(v);
}

Value OpBuilder::createAlloc(const Type& t) {
  Operation* op = ctx_->newOp(OpKind::Alloc);
  Value r = addResult(ctx_, op, t);
  insert(op);
  return r;
}

FuncOp OpBuilder::createFunc(const std::string& name, const std::vector<Type>& inputs,
                             const std::vector<Type>& results) {
  Operation* op = ctx_->newOp(OpKind::Func);
  op->name = name;
  op->resultTypes = results;
  op->body = ctx_->newBlock(op);
  for (size_t i = 0; i < inputs.size(); ++i)
    op->body->args.push_back(ctx_->newValue(inputs[i], nullptr, op->body, static_cast<int>(i)));
  insert(op);
  return FuncOp(op);
}

Operation* OpBuilder::createReturn(const std::vector<Value>& values) {
  Operation* op = ctx_->newOp(OpKind::Return);
  op->operands = values;
  return insert(op);
}

CallOp OpBuilder::createCall(FuncOp callee, const std::vector<Value>& operands) {
  Operation* op = ctx_->newOp(OpKind::Call);
  op->name = callee.getName();
  op->operands = operands;
  for (auto& t : callee->resultTypes) addResult(ctx_, op, t);
  insert(op);
  return CallOp(op);
}

AffineForOp OpBuilder::createFor(int64_t lb, int64_t ub, int64_t step, const std::vector<Value>& iterInits,
                                 const std::function<void(OpBuilder&, Value, const std::vector<Value>&)>& body) {
  Operation* op = ctx_->newOp(OpKind::For);
  op->lb = lb;
  op->ub = ub;
  op->step = step;
  op->operands = iterInits;
  op->body = ctx_->newBlock(op);
  op->body->args.push_back(ctx_->newValue(Type::index(), nullptr, op->body, 0));
  std::vector<Value> iterArgs;
  for (size_t i = 0; i < iterInits.size(); ++i) {
    ValueImpl* a = ctx_->newValue(iterInits[i].getType(), nullptr, op->body, static_cast<int>(i + 1));
    op->body->args.push_back(a);
    iterArgs.emplace_back(a);
    addResult(ctx_, op, iterInits[i].getType());
  }
  insert(op);
  if (body) {
    InsertPoint saved = ip_;
    setInsertionPointToEnd(op->body);
    body(*this, Value(op->body->args[0]), iterArgs);
    ip_ = saved;
  }
  return AffineForOp(op);
}

AffineParallelOp OpBuilder::createParallel(const std::vector<int64_t>& extents, const std::string& level) {
  Operation* op = ctx_->newOp(OpKind::Parallel);
  op->extents = extents;
  op->body = ctx_->newBlock(op);
  for (size_t i = 0; i < extents.size(); ++i)
    op->body->args.push_back(ctx_->newValue(Type::index(), nullptr, op->body, static_cast<int>(i)));
  if (!level.empty()) op->setAttr("gpu.level", level);
  insert(op);
  return AffineParallelOp(op);
}

Operation* OpBuilder::createYield(const std::vector<Value>& values) {
  Operation* op = ctx_->newOp(OpKind::Yield);
  op->operands = values;
  return insert(op);
}

Value OpBuilder::createApply(const IndexExpr& e) {
  Operation* op = ctx_->newOp(OpKind::Apply);
  op->indices.push_back(e);
  Value r = addResult(ctx_, op, Type::index());
  insert(op);
  return r;
}

Value OpBuilder::createLoad(Value memref, const std::vector<IndexExpr>& idx) {
  Operation* op = ctx_->newOp(OpKind::Load);
  op->operands = {memref};
  op->indices = idx;
  Value r = addResult(ctx_, op, memref.getType().elementType());
  insert(op);
  return r;
}

Operation* OpBuilder::createStore(Value v, Value memref, const std::vector<IndexExpr>& idx) {
  Operation* op = ctx_->newOp(OpKind::Store);
  op->operands = {v, memref};
  op->indices = idx;
  return insert(op);
}

Value OpBuilder::createVectorLoad(Value memref, const std::vector<AffineExpr>& idx, int64_t width) {
  Operation* op = ctx_->newOp(OpKind::VectorLoad);
  op->operands = {memref};
  op->exprs = idx;
  op->width = width;
  Value r = addResult(ctx_, op, memref.getType().elementType());
  insert(op);
  return r;
}

Operation* OpBuilder::createVectorStore(Value v, Value memref, const std::vector<AffineExpr>& idx, int64_t width) {
  Operation* op = ctx_->newOp(OpKind::VectorStore);
  op->operands = {v, memref};
  op->exprs = idx;
  op->width = width;
  return insert(op);
}

Operation* OpBuilder::createIf(const AffineExpr& cond) {
  Operation* op = ctx_->newOp(OpKind::If);
  op->cond = cond;
  op->body = ctx_->newBlock(op);
  return insert(op);
}

Value OpBuilder::createIndexConstant(int64_t v) {
  Operation* op = ctx_->newOp(OpKind::IndexConstant);
  op->ivalue = v;
  Value r = addResult(ctx_, op, Type::index());
  insert(op);
  return r;
}

Value OpBuilder::createConstant(double v, ScalarKind k) {
  Operation* op = ctx_->newOp(OpKind::Constant);
  op->fvalue = v;
  Value r = addResult(ctx_, op, Type::scalar(k));
  insert(op);
  return r;
}

Value OpBuilder::createBinary(OpKind k, Value a, Value b) {
  Operation* op = ctx_->newOp(k);
  op->operands = {a, b};
  Value r = addResult(ctx_, op, a.getType());
  insert(op);
  return r;
}

Value OpBuilder::createExp(Value a) {
  Operation* op = ctx_->newOp(OpKind::Exp);
  op->operands = {a};
  Value r = addResult(ctx_, op, a.getType());
  insert(op);
  return r;
}

BarrierOp OpBuilder::createBarrier() {
  Operation* op = ctx_->newOp(OpKind::Barrier);
  insert(op);
  return BarrierOp(op);
}

Operation* OpBuilder::createAnnotation(const std::string& name, const std::vector<Value>& operands) {
  Operation* op = ctx_->newOp(OpKind::Annotation);
  op->name = name;
  op->operands = operands;
  return insert(op);
}

void OpBuilder::buildAffineLoopNest(const std::vector<int64_t>& lbs, const std::vector<int64_t>& ubs,
                                    const std::vector<int64_t>& steps,
                                    const std::function<void(OpBuilder&, const std::vector<Value>&)>& body) {
  InsertPoint saved = ip_;
  std::vector<Value> ivs;
  for (size_t i = 0; i < ubs.size(); ++i) {
    AffineForOp loop = createFor(lbs[i], ubs[i], steps[i]);
    ivs.push_back(loop.getInductionVar());
    setInsertionPointToEnd(loop.getBody());
  }
  if (body) body(*this, ivs);
  ip_ = saved;
}

// ---- printer ------------------------------------------------------------------------------------
namespace {

struct Printer {
  std::ostream& os;
  std::unordered_map<ValueImpl*, std::string> names;
  int nextResult = 0, nextArg = 0, nextCst = 0;

  explicit Printer(std::ostream& o) : os(o) {}

  std::string name(Value v) {
    auto it = names.find(v.impl());
    if (it != names.end()) return it->second;
    return "<<unknown>>";
  }
  void nameArg(ValueImpl* a) { names[a] = "%arg" + std::to_string(nextArg++); }
  void nameResult(ValueImpl* r, bool cst) {
    if (cst) {
      names[r] = nextCst == 0 ? "%cst" : "%cst_" + std::to_string(nextCst - 1);
      ++nextCst;
    } else {
      names[r] = "%" + std::to_string(nextResult++);
    }
  }
  std::string expr(const IndexExpr& e) {
    std::ostringstream s;
    bool first = true;
    for (auto& t : e.terms) {
      if (!first) s << " + ";
      first = false;
      s << name(t.first);
      if (t.second != 1) s << " * " << t.second;
    }
    if (e.constant != 0 || first) {
      if (!first) s << " + ";
      s << e.constant;
    }
    return s.str();
  }
  std::string indexList(const std::vector<IndexExpr>& idx) {
    std::string s = "[";
    for (size_t i = 0; i < idx.size(); ++i) s += (i ? ", " : "") + expr(idx[i]);
    return s + "]";
  }
  // index list of an access in either form
  std::string accessList(const Operation* op) {
    if (op->exprs.empty()) return indexList(op->indices);
    std::string s = "[";
    for (size_t i = 0; i < op->exprs.size(); ++i)
      s += (i ? ", " : "") + op->exprs[i].str([&](Value v) { return name(v); });
    return s + "]";
  }
  int nextIdxCst = 0;
  static std::string fp(double v) {
    std::ostringstream s;
    s << std::scientific << std::setprecision(6) << v;
    return s.str();
  }
  void attrs(const Operation* op) {
    if (op->attrs.empty()) return;
    os << " attributes {";
    bool first = true;
    for (auto& kv : op->attrs) {
      if (!first) os << ", ";
      first = false;
      os << kv.first << " = ";
      if (auto p = std::get_if<int64_t>(&kv.second)) os << *p;
      else if (auto d = std::get_if<double>(&kv.second)) os << fp(*d);
      else if (auto s = std::get_if<std::string>(&kv.second)) os << '"' << *s << '"';
      else if (auto v = std::get_if<std::vector<int64_t>>(&kv.second)) {
        os << "[";
        for (size_t i = 0; i < v->size(); ++i) os << (i ? ", " : "") << (*v)[i];
        os << "]";
      }
    }
    os << "}";
  }
  void block(Block* b, int indent) {
    for (Operation* op : b->ops) print(op, indent);
  }
  void print(Operation* op, int indent) {
    const std::string pad(indent, ' ');
    switch (op->kind) {
      case OpKind::Module:
        os << pad << "module @" << op->name << " {\n";
        block(op->body, indent + 2);
        os << pad << "}\n";
        break;
      case OpKind::Func: {
        // functions are isolated: restart numbering inside
        Printer inner(os);
        for (auto* a : op->body->args) inner.nameArg(a);
        os << pad << "func.func @" << op->name << "(";
        for (size_t i = 0; i < op->body->args.size(); ++i)
          os << (i ? ", " : "") << inner.name(Value(op->body->args[i])) << ": " << op->body->args[i]->type.str();
        os << ")";
        if (!op->resultTypes.empty()) {
          os << " -> ";
          for (size_t i = 0; i < op->resultTypes.size(); ++i) os << (i ? ", " : "") << op->resultTypes[i].str();
        }
        inner.attrs(op);
        os << " {\n";
        inner.block(op->body, indent + 2);
        os << pad << "}\n";
        break;
      }
      case OpKind::Return:
        os << pad << "return";
        for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : " ") << name(op->operands[i]);
        if (!op->operands.empty()) {
          os << " : ";
          for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : "") << op->operands[i].getType().str();
        }
        os << "\n";
        break;
      case OpKind::Call: {
        for (auto* r : op->results) nameResult(r, false);
        os << pad;
        for (size_t i = 0; i < op->results.size(); ++i) os << (i ? ", " : "") << names[op->results[i]];
        if (!op->results.empty()) os << " = ";
        os << "func.call @" << op->name << "(";
        for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : "") << name(op->operands[i]);
        os << ") : (";
        for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : "") << op->operands[i].getType().str();
        os << ") -> ";
        for (size_t i = 0; i < op->results.size(); ++i) os << (i ? ", " : "") << op->results[i]->type.str();
        os << "\n";
        break;
      }
      case OpKind::Alloc:
        nameResult(op->results[0], false);
        os << pad << names[op->results[0]] << " = memref.alloc() : " << op->results[0]->type.str() << "\n";
        break;
      case OpKind::For: {
        for (auto* r : op->results) nameResult(r, false);
        for (auto* a : op->body->args) nameArg(a);
        os << pad;
        for (size_t i = 0; i < op->results.size(); ++i) os << (i ? ", " : "") << names[op->results[i]];
        if (!op->results.empty()) os << " = ";
        os << "affine.for " << name(Value(op->body->args[0])) << " = " << op->lb << " to " << op->ub;
        if (op->step != 1) os << " step " << op->step;
        if (!op->operands.empty()) {
          os << " iter_args(";
          for (size_t i = 0; i < op->operands.size(); ++i)
            os << (i ? ", " : "") << name(Value(op->body->args[i + 1])) << " = " << name(op->operands[i]);
          os << ") -> (";
          for (size_t i = 0; i < op->results.size(); ++i) os << (i ? ", " : "") << op->results[i]->type.str();
          os << ")";
        }
        os << " {\n";
        block(op->body, indent + 2);
        os << pad << "}";
        attrs(op);
        os << "\n";
        break;
      }
      case OpKind::Parallel: {
        for (auto* a : op->body->args) nameArg(a);
        os << pad << "affine.parallel (";
        for (size_t i = 0; i < op->body->args.size(); ++i) os << (i ? ", " : "") << name(Value(op->body->args[i]));
        os << ") = (";
        for (size_t i = 0; i < op->extents.size(); ++i) os << (i ? ", " : "") << 0;
        os << ") to (";
        for (size_t i = 0; i < op->extents.size(); ++i) os << (i ? ", " : "") << op->extents[i];
        os << ") {\n";
        block(op->body, indent + 2);
        os << pad << "}";
        attrs(op);
        os << "\n";
        break;
      }
      case OpKind::Yield:
        os << pad << "affine.yield";
        for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : " ") << name(op->operands[i]);
        if (!op->operands.empty()) os << " : " << op->operands[0].getType().str();
        os << "\n";
        break;
      case OpKind::Apply: {
        nameResult(op->results[0], false);
        const IndexExpr& e = op->indices[0];
        os << pad << names[op->results[0]] << " = affine.apply affine_map<(";
        for (size_t i = 0; i < e.terms.size(); ++i) os << (i ? ", " : "") << "d" << i;
        os << ") -> (";
        for (size_t i = 0; i < e.terms.size(); ++i) {
          os << (i ? " + " : "") << "d" << i;
          if (e.terms[i].second != 1) os << " * " << e.terms[i].second;
        }
        if (e.constant != 0 || e.terms.empty()) os << (e.terms.empty() ? "" : " + ") << e.constant;
        os << ")>(";
        for (size_t i = 0; i < e.terms.size(); ++i) os << (i ? ", " : "") << name(e.terms[i].first);
        os << ")\n";
        break;
      }
      case OpKind::Load:
        nameResult(op->results[0], false);
        os << pad << names[op->results[0]] << " = affine.load " << name(op->operands[0]) << accessList(op)
           << " : " << op->operands[0].getType().str() << "\n";
        break;
      case OpKind::Store:
        os << pad << "affine.store " << name(op->operands[0]) << ", " << name(op->operands[1])
           << accessList(op) << " : " << op->operands[1].getType().str() << "\n";
        break;
      case OpKind::VectorLoad:
        nameResult(op->results[0], false);
        os << pad << names[op->results[0]] << " = affine.vector_load " << name(op->operands[0]) << accessList(op) << " : "
           << op->operands[0].getType().str() << ", vector<" << op->width << "x"
           << scalarName(op->operands[0].getType().elem) << ">\n";
        break;
      case OpKind::VectorStore:
        os << pad << "affine.vector_store " << name(op->operands[0]) << ", " << name(op->operands[1]) << accessList(op)
           << " : " << op->operands[1].getType().str() << ", vector<" << op->width << "x"
           << scalarName(op->operands[1].getType().elem) << ">\n";
        break;
      case OpKind::If: {
        // affine.if affine_set<(d0, ...) : (expr >= 0)>(operands)
        std::vector<Value> leaves;
        op->cond.collectValues(leaves);
        std::vector<Value> uniq;
        for (auto v : leaves)
          if (std::find(uniq.begin(), uniq.end(), v) == uniq.end()) uniq.push_back(v);
        os << pad << "affine.if affine_set<(";
        for (size_t i = 0; i < uniq.size(); ++i) os << (i ? ", " : "") << "d" << i;
        os << ") : (" << op->cond.str([&](Value v) {
          return "d" + std::to_string(std::find(uniq.begin(), uniq.end(), v) - uniq.begin());
        }) << " >= 0)>(";
        for (size_t i = 0; i < uniq.size(); ++i) os << (i ? ", " : "") << name(uniq[i]);
        os << ") {\n";
        block(op->body, indent + 2);
        os << pad << "}\n";
        break;
      }
      case OpKind::IndexConstant:
        names[op->results[0]] = nextIdxCst == 0 ? "%c" + std::to_string(op->ivalue)
                                                : "%c" + std::to_string(op->ivalue) + "_" + std::to_string(nextIdxCst - 1);
        ++nextIdxCst;
        os << pad << names[op->results[0]] << " = arith.constant " << op->ivalue << " : index\n";
        break;
      case OpKind::Constant:
        nameResult(op->results[0], true);
        os << pad << names[op->results[0]] << " = arith.constant " << fp(op->fvalue) << " : "
           << op->results[0]->type.str() << "\n";
        break;
      case OpKind::MulF:
      case OpKind::AddF:
      case OpKind::MaxF:
      case OpKind::DivF:
        nameResult(op->results[0], false);
        os << pad << names[op->results[0]] << " = " << opKindName(op->kind) << " " << name(op->operands[0]) << ", "
           << name(op->operands[1]) << " : " << op->results[0]->type.str() << "\n";
        break;
      case OpKind::Exp:
        nameResult(op->results[0], false);
        os << pad << names[op->results[0]] << " = math.exp " << name(op->operands[0]) << " : "
           << op->results[0]->type.str() << "\n";
        break;
      case OpKind::Barrier:
        os << pad << "gpu.barrier\n";
        break;
      case OpKind::Annotation:
        os << pad << "kcg." << op->name << "(";
        for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : "") << name(op->operands[i]);
        os << ")";
        attrs(op);
        os << "\n";
        break;
    }
  }
};

}  // namespace

void Operation::print(std::ostream& os) const {
  Printer p(os);
  p.print(const_cast<Operation*>(this), 0);
}

void Operation::dump() const { print(std::cerr); }

std::string ModuleOp::str() const {
  std::ostringstream os;
  op_->print(os);
  return os.str();
}

// ---- verifier -----------------------------------------------------------------------------------
namespace {

struct Verifier {
  std::string msg;
  std::vector<std::vector<ValueImpl*>> scopes;
  std::map<std::string, Operation*> funcs;

  bool visible(Value v) const {
    for (auto& s : scopes)
      if (std::find(s.begin(), s.end(), v.impl()) != s.end()) return true;
    return false;
  }
  bool fail(Operation* op, const std::string& m) {
    msg = std::string(opKindName(op->kind)) + (op->name.empty() ? "" : " @" + op->name) + ": " + m;
    return false;
  }
  bool checkBlock(Block* b, bool isolated) {
    std::vector<std::vector<ValueImpl*>> saved;
    if (isolated) saved.swap(scopes);
    scopes.emplace_back(b->args.begin(), b->args.end());
    bool ok = true;
    for (Operation* op : b->ops) {
      if (!check(op)) { ok = false; break; }
      for (auto* r : op->results) scopes.back().push_back(r);
    }
    scopes.pop_back();
    if (isolated) saved.swap(scopes);
    return ok;
  }
  bool check(Operation* op) {
    for (auto v : op->operands) {
      if (!v) return fail(op, "null operand");
      if (!visible(v)) return fail(op, "operand is not defined in an enclosing scope before its use");
    }
    for (auto& e : op->indices)
      for (auto& t : e.terms) {
        if (!visible(t.first)) return fail(op, "index operand is not visible");
        if (t.first.getType() != Type::index()) return fail(op, "index operand is not of index type");
      }
    {
      std::vector<Value> leaves;
      for (auto& e : op->exprs) e.collectValues(leaves);
      if (op->kind == OpKind::If) op->cond.collectValues(leaves);
      for (auto v : leaves) {
        if (!visible(v)) return fail(op, "index operand is not visible");
        if (v.getType() != Type::index()) return fail(op, "index operand is not of index type");
      }
    }
    switch (op->kind) {
      case OpKind::If:
        return checkBlock(op->body, false);
      case OpKind::VectorLoad:
      case OpKind::VectorStore: {
        const Value mem = op->operands[op->kind == OpKind::VectorLoad ? 0 : 1];
        if (!mem.getType().isMemRef()) return fail(op, "vector access to a non-memref");
        if (op->exprs.size() != mem.getType().shape.size()) return fail(op, "rank mismatch");
        if (op->width < 1) return fail(op, "vector width");
        return true;
      }
      case OpKind::For:
        if (op->step <= 0) return fail(op, "non-positive step");
        if (op->operands.size() != op->results.size()) return fail(op, "iter_args / results mismatch");
        if (!op->operands.empty()) {
          if (op->body->ops.empty() || op->body->ops.back()->kind != OpKind::Yield)
            return fail(op, "loop with iter_args must end in affine.yield");
          if (op->body->ops.back()->operands.size() != op->operands.size()) return fail(op, "yield arity");
        }
        return checkBlock(op->body, false);
      case OpKind::Parallel:
        if (op->extents.empty() || op->extents.size() > 3) return fail(op, "1 to 3 parallel dimensions");
        return checkBlock(op->body, false);
      case OpKind::Func:
        funcs[op->name] = op;
        return checkBlock(op->body, true);
      case OpKind::Module:
        return checkBlock(op->body, true);
      case OpKind::Load:
        if (!op->operands[0].getType().isMemRef()) return fail(op, "load from a non-memref");
        if (op->indexRank() != op->operands[0].getType().shape.size()) return fail(op, "rank mismatch");
        return true;
      case OpKind::Store:
        if (!op->operands[1].getType().isMemRef()) return fail(op, "store to a non-memref");
        if (op->indexRank() != op->operands[1].getType().shape.size()) return fail(op, "rank mismatch");
        if (op->operands[0].getType() != op->operands[1].getType().elementType()) return fail(op, "element type");
        return true;
      case OpKind::Call: {
        auto it = funcs.find(op->name);
        if (it == funcs.end()) return fail(op, "callee not defined before the call");
        Operation* f = it->second;
        if (f->body->args.size() != op->operands.size()) return fail(op, "argument count");
        for (size_t i = 0; i < op->operands.size(); ++i)
          if (f->body->args[i]->type != op->operands[i].getType()) return fail(op, "argument type");
        return true;
      }
      default:
        return true;
    }
  }
};

}  // namespace

bool verify(ModuleOp module, std::string* message) {
  Verifier v;
  bool ok = v.check(module.getOperation());
  if (!ok && message) *message = v.msg;
  return ok;
}

std::vector<Operation*> usersOf(Operation* root, Value v) {
  std::vector<Operation*> users;
  root->walk([&](Operation* op) {
    bool used = std::find(op->operands.begin(), op->operands.end(), v) != op->operands.end();
    for (auto& e : op->indices) used = used || e.uses(v);
    if (used) users.push_back(op);
  });
  return users;
}

}  // namespace kcgir
