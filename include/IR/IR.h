// A small affine loop-nest IR that hosts the operator API (Frontend graph builder, Optimizer
// schedule primitives, Backend dispatch) without depending on MLIR.
//
// The reference keeps this slot for its MLIR include hub (include/IR/IR.h:1-6 pulls in
// include/IR/MLIR.h:1-167, i.e. upstream LLVM/MLIR 15).  Only the handful of concepts the two
// operators need are modelled here: memrefs with a memory space, functions and calls,
// affine.for (with one loop-carried value), affine.parallel, loads/stores with linear index
// expressions, a few arith/math ops, and free-form "kcg.*" annotation ops that record
// schedule steps which have no structural effect on this backend.
//
// Handles (Value, ModuleOp, AffineForOp, ...) are cheap pointer wrappers, as in MLIR; the
// objects live in a Context-owned arena.  The spelling `mlir::...` is provided as aliases so
// that code written against the reference's signatures keeps compiling.
#pragma once

#include <cassert>
#include <cstdint>
#include <functional>
#include <iosfwd>
#include <list>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <variant>
#include <vector>

namespace kcgir {

struct Operation;
struct Block;
struct ValueImpl;
class Context;

enum class ScalarKind { None, F16, BF16, F32, F64, Index };

const char* scalarName(ScalarKind k);
int scalarBytes(ScalarKind k);

struct Type {
  ScalarKind elem = ScalarKind::None;
  bool memref = false;
  std::vector<int64_t> shape;
  int memorySpace = 0;

  static Type scalar(ScalarKind k) { Type t; t.elem = k; return t; }
  static Type index() { return scalar(ScalarKind::Index); }
  static Type memRef(std::vector<int64_t> shape, ScalarKind k, int space) {
    Type t; t.elem = k; t.memref = true; t.shape = std::move(shape); t.memorySpace = space; return t;
  }
  bool isMemRef() const { return memref; }
  bool isNone() const { return elem == ScalarKind::None; }
  Type elementType() const { return scalar(elem); }
  Type getElementType() const { return scalar(elem); }
  template <class T> T dyn_cast() const { return *this; }   // `type.dyn_cast<mlir::MemRefType>()` keeps compiling
  const std::vector<int64_t>& getShape() const { return shape; }
  int getMemorySpace() const { return memorySpace; }
  std::string str() const;
  bool operator==(const Type& o) const {
    return elem == o.elem && memref == o.memref && shape == o.shape && memorySpace == o.memorySpace;
  }
  bool operator!=(const Type& o) const { return !(*this == o); }
};

// SSA value: a result of an operation or an argument of a block.
class Value {
 public:
  Value() = default;
  Value(std::nullptr_t) {}
  explicit Value(ValueImpl* i) : impl_(i) {}
  explicit operator bool() const { return impl_ != nullptr; }
  bool operator==(const Value& o) const { return impl_ == o.impl_; }
  bool operator!=(const Value& o) const { return impl_ != o.impl_; }
  bool operator<(const Value& o) const { return impl_ < o.impl_; }
  Type getType() const;
  Operation* getDefiningOp() const;   // nullptr for block arguments
  Block* getOwnerBlock() const;       // non-null for block arguments
  bool isBlockArgument() const { return getDefiningOp() == nullptr; }
  ValueImpl* impl() const { return impl_; }
 private:
  ValueImpl* impl_ = nullptr;
};

struct ValueImpl {
  Type type;
  Operation* def = nullptr;
  Block* owner = nullptr;
  int index = 0;
};

// Linear index expression: sum_i coeff_i * value_i + constant.
struct IndexExpr {
  std::vector<std::pair<Value, int64_t>> terms;
  int64_t constant = 0;
  IndexExpr() = default;
  IndexExpr(Value v) { terms.emplace_back(v, 1); }  // NOLINT: implicit on purpose
  static IndexExpr cst(int64_t c) { IndexExpr e; e.constant = c; return e; }
  IndexExpr operator+(const IndexExpr& o) const;
  IndexExpr operator*(int64_t f) const;
  void substitute(Value from, const IndexExpr& to);
  bool uses(Value v) const;
  int64_t coefficientOf(Value v) const;
  void simplify();
};

// Quasi-affine expression: sums, products with constants, floordiv and mod by constants over
// leaves that are either map dimensions (d0, d1, ...; the form user code builds, as with MLIR's
// AffineExpr) or SSA values (the form stored on operations, after a map has been applied to its
// operands).  Cheap to copy (shared immutable nodes); constants are folded on construction.
class AffineExpr {
 public:
  enum class Kind { Cst, Dim, Val, Add, Mul, FloorDiv, Mod };
  AffineExpr();                                   // the constant 0
  static AffineExpr constant(int64_t c);
  static AffineExpr dim(unsigned position);
  static AffineExpr value(Value v);
  static AffineExpr fromLinear(const IndexExpr& e);

  AffineExpr operator+(const AffineExpr& o) const;
  AffineExpr operator+(int64_t c) const { return *this + constant(c); }
  AffineExpr operator-(int64_t c) const { return *this + constant(-c); }
  AffineExpr operator*(const AffineExpr& o) const;   // one side must be a constant
  AffineExpr operator*(int64_t c) const;
  AffineExpr floorDiv(int64_t c) const;
  AffineExpr floorDiv(uint64_t c) const { return floorDiv(static_cast<int64_t>(c)); }
  AffineExpr floorDiv(int c) const { return floorDiv(static_cast<int64_t>(c)); }
  AffineExpr operator%(int64_t c) const;
  AffineExpr operator%(uint64_t c) const { return *this % static_cast<int64_t>(c); }
  AffineExpr operator%(int c) const { return *this % static_cast<int64_t>(c); }

  Kind kind() const;
  int64_t constantValue() const;                  // Cst
  unsigned dimPosition() const;                   // Dim
  Value leafValue() const;                        // Val
  bool isConstant() const { return kind() == Kind::Cst; }
  AffineExpr lhs() const;                         // Add / Mul / FloorDiv / Mod: the (left) operand
  AffineExpr rhs() const;                         // Add: the right operand; Mul / FloorDiv / Mod: the constant

  // dims -> the given expressions (application of a map to operands, composition of maps)
  AffineExpr replaceDims(const std::vector<AffineExpr>& by) const;
  // every leaf equal to `from` -> `to`
  AffineExpr replaceValue(Value from, const AffineExpr& to) const;
  // leaves remapped through `fn` (cloning)
  AffineExpr mapValues(const std::function<Value(Value)>& fn) const;
  bool uses(Value v) const;
  void collectValues(std::vector<Value>& out) const;
  // numeric value for given leaf values; dims are not allowed here
  int64_t evaluate(const std::function<int64_t(Value)>& valueOf) const;
  // true (and the linear form) when no floordiv / mod occurs
  bool toLinear(IndexExpr* out) const;
  // text in MLIR's infix spelling, leaves named by `nameOf` (dims print as d<i>)
  std::string str(const std::function<std::string(Value)>& nameOf) const;

  struct Node;
 private:
  explicit AffineExpr(std::shared_ptr<const Node> n) : node_(std::move(n)) {}
  static AffineExpr make(Kind k, int64_t c, const AffineExpr* a, const AffineExpr* b);
  std::shared_ptr<const Node> node_;
};
inline AffineExpr operator*(int64_t c, const AffineExpr& e) { return e * c; }
inline AffineExpr operator+(int64_t c, const AffineExpr& e) { return e + c; }

// (d0, ..., d{n-1}) -> (results...)
class AffineMap {
 public:
  AffineMap() = default;
  static AffineMap get(unsigned dimCount, unsigned symbolCount, const std::vector<AffineExpr>& results, Context* ctx = nullptr) {
    (void)symbolCount;
    (void)ctx;
    AffineMap m;
    m.numDims_ = dimCount;
    m.results_ = results;
    return m;
  }
  unsigned getNumDims() const { return numDims_; }
  unsigned getNumResults() const { return static_cast<unsigned>(results_.size()); }
  const std::vector<AffineExpr>& getResults() const { return results_; }
  AffineExpr getResult(unsigned i) const { return results_.at(i); }
  // the results with dim i replaced by operands[i]
  std::vector<AffineExpr> apply(const std::vector<AffineExpr>& operands) const;
 private:
  unsigned numDims_ = 0;
  std::vector<AffineExpr> results_;
};

using Attribute = std::variant<int64_t, double, std::string, std::vector<int64_t>>;

enum class OpKind {
  Module, Func, Return, Call, Alloc,
  For, Parallel, Yield, Apply,
  Load, Store, Constant, MulF, AddF, MaxF, DivF, Exp,
  Barrier, Annotation,
  VectorLoad, VectorStore,   // affine.vector_load / affine.vector_store: `width` contiguous elements
  If,                        // affine.if with one condition `cond >= 0`, no else branch
  IndexConstant              // arith.constant <n> : index
};

const char* opKindName(OpKind k);

struct Block {
  std::vector<ValueImpl*> args;
  std::list<Operation*> ops;
  Operation* parentOp = nullptr;
  Value getArgument(size_t i) const { return Value(args.at(i)); }
  size_t getNumArguments() const { return args.size(); }
  std::list<Operation*>& getOperations() { return ops; }
};

struct Operation {
  OpKind kind;
  std::string name;                       // func symbol / callee / annotation name
  std::vector<Value> operands;
  std::vector<ValueImpl*> results;
  std::map<std::string, Attribute> attrs;
  Block* body = nullptr;                  // Module, Func, For, Parallel
  Block* parent = nullptr;
  Context* ctx = nullptr;
  // For
  int64_t lb = 0, ub = 0, step = 1;
  // Parallel: extent per dimension (lower bound 0, step 1)
  std::vector<int64_t> extents;
  // Load / Store / Apply
  std::vector<IndexExpr> indices;
  // Load / Store / VectorLoad / VectorStore in general form: one quasi-affine expression per
  // memref dimension over SSA values (floordiv / mod allowed).  Used instead of `indices` when
  // not empty.
  std::vector<AffineExpr> exprs;
  int64_t width = 1;                      // VectorLoad / VectorStore
  AffineExpr cond;                        // If: the body runs when cond >= 0
  int64_t ivalue = 0;                     // IndexConstant
  // Constant
  double fvalue = 0.0;
  // Func
  std::vector<Type> resultTypes;

  Value getResult(size_t i = 0) const { return Value(results.at(i)); }
  size_t getNumResults() const { return results.size(); }
  Operation* getParentOp() const { return parent ? parent->parentOp : nullptr; }
  Context* getContext() const { return ctx; }
  void setAttr(const std::string& key, Attribute a) { attrs[key] = std::move(a); }
  bool hasAttr(const std::string& key) const { return attrs.count(key) != 0; }
  int64_t getIntAttr(const std::string& key, int64_t dflt = 0) const;
  std::string getStringAttr(const std::string& key, const std::string& dflt = "") const;
  void erase();                           // unlink from the parent block
  void moveBefore(Operation* other);
  void moveAfter(Operation* other);
  void walk(const std::function<void(Operation*)>& fn);  // pre-order, includes this
  void replaceUsesOfWith(Value from, Value to);          // inside this op (recursively)
  void substituteIndex(Value from, const IndexExpr& to); // inside this op (recursively)
  void substituteExpr(Value from, const AffineExpr& to); // same with a general expression: ops that use
                                                         // `from` in a linear index switch to the general form
  // index expression of memref dimension d, whichever form the op is in
  AffineExpr indexExpr(size_t d) const;
  size_t indexRank() const { return exprs.empty() ? indices.size() : exprs.size(); }
  void dump() const;
  void print(std::ostream& os) const;
};

// Owns every Operation / Block / ValueImpl ever created through it.
class Context {
 public:
  Context() = default;
  Context(const Context&) = delete;
  Context& operator=(const Context&) = delete;
  Operation* newOp(OpKind k);
  Block* newBlock(Operation* parent);
  ValueImpl* newValue(Type t, Operation* def, Block* owner, int index);
  template <class Dialect> void getOrLoadDialect() {}  // source compatibility only
 private:
  std::vector<std::unique_ptr<Operation>> ops_;
  std::vector<std::unique_ptr<Block>> blocks_;
  std::vector<std::unique_ptr<ValueImpl>> values_;
};

// ---- typed handles ------------------------------------------------------------------------------
class OpHandle {
 public:
  OpHandle() = default;
  OpHandle(Operation* op) : op_(op) {}  // NOLINT: implicit on purpose
  explicit operator bool() const { return op_ != nullptr; }
  operator Operation*() const { return op_; }  // NOLINT
  Operation* operator->() const { return op_; }
  Operation* getOperation() const { return op_; }
  bool operator==(const OpHandle& o) const { return op_ == o.op_; }
  bool operator!=(const OpHandle& o) const { return op_ != o.op_; }
 protected:
  Operation* op_ = nullptr;
};

class ModuleOp : public OpHandle {
 public:
  using OpHandle::OpHandle;
  static ModuleOp create(Context* ctx, const std::string& name);
  Block* getBody() const { return op_->body; }
  std::string getName() const { return op_->name; }
  Operation* clone() const;               // deep copy, values remapped
  void dump() const { op_->dump(); }
  std::string str() const;
};

class FuncOp : public OpHandle {
 public:
  using OpHandle::OpHandle;
  Block& front() const { return *op_->body; }
  Block* getBody() const { return op_->body; }
  std::string getName() const { return op_->name; }
  std::string getSymName() const { return op_->name; }
  Value getArgument(size_t i) const { return op_->body->getArgument(i); }
  size_t getNumArguments() const { return op_->body->getNumArguments(); }
};

class CallOp : public OpHandle {
 public:
  using OpHandle::OpHandle;
  std::string getCallee() const { return op_->name; }
  std::vector<Value> getOperands() const { return op_->operands; }
  Value getResult(size_t i = 0) const { return op_->getResult(i); }
};

class AllocOp : public OpHandle {
 public:
  using OpHandle::OpHandle;
  Value getResult() const { return op_->getResult(0); }
};

class AffineForOp : public OpHandle {
 public:
  using OpHandle::OpHandle;
  Block* getBody() const { return op_->body; }
  Value getInductionVar() const { return op_->body->getArgument(0); }
  int64_t getConstantLowerBound() const { return op_->lb; }
  int64_t getConstantUpperBound() const { return op_->ub; }
  int64_t getStep() const { return op_->step; }
  int64_t tripCount() const { return (op_->ub - op_->lb + op_->step - 1) / op_->step; }
  bool hasConstantBounds() const { return true; }
  size_t getNumIterOperands() const { return op_->operands.size(); }
  Value getRegionIterArg(size_t i) const { return op_->body->getArgument(1 + i); }
  Value getResult(size_t i = 0) const { return op_->getResult(i); }
};

class AffineParallelOp : public OpHandle {
 public:
  using OpHandle::OpHandle;
  Block* getBody() const { return op_->body; }
  size_t getNumDims() const { return op_->extents.size(); }
  std::vector<Value> getIVs() const;
  int64_t getExtent(size_t i) const { return op_->extents.at(i); }
  std::string getLevel() const { return op_->getStringAttr("gpu.level"); }  // "grid" / "block"
};

class BarrierOp : public OpHandle {
 public:
  using OpHandle::OpHandle;
};

template <class H> H dyn_cast_kind(Operation* op, OpKind k) { return (op && op->kind == k) ? H(op) : H(); }

// Insertion-point based construction.
class OpBuilder {
 public:
  struct InsertPoint { Block* block = nullptr; Operation* before = nullptr; };  // before == nullptr: at end

  OpBuilder() = default;
  explicit OpBuilder(Context* ctx) : ctx_(ctx) {}
  Context* getContext() const { return ctx_; }

  void setInsertionPointToStart(Block* b) { ip_.block = b; ip_.before = b->ops.empty() ? nullptr : b->ops.front(); }
  void setInsertionPointToEnd(Block* b) { ip_.block = b; ip_.before = nullptr; }
  void setInsertionPoint(Operation* op) { ip_.block = op->parent; ip_.before = op; }
  void setInsertionPointAfter(Operation* op);
  InsertPoint saveInsertionPoint() const { return ip_; }
  void restoreInsertionPoint(InsertPoint ip) { ip_ = ip; }
  Block* getInsertionBlock() const { return ip_.block; }

  Operation* insert(Operation* op);       // place an unlinked op at the insertion point

  // memref.alloc
  Value createAlloc(const Type& memrefType);
  // func.func @name(args...) -> results ; the body block gets one argument per input type
  FuncOp createFunc(const std::string& name, const std::vector<Type>& inputs, const std::vector<Type>& results);
  Operation* createReturn(const std::vector<Value>& values);
  CallOp createCall(FuncOp callee, const std::vector<Value>& operands);
  // affine.for %iv = lb to ub step s [iter_args(%x = init)]; body receives (builder, iv, iterArgs)
  AffineForOp createFor(int64_t lb, int64_t ub, int64_t step, const std::vector<Value>& iterInits = {},
                        const std::function<void(OpBuilder&, Value, const std::vector<Value>&)>& body = nullptr);
  AffineParallelOp createParallel(const std::vector<int64_t>& extents, const std::string& level);
  Operation* createYield(const std::vector<Value>& values);
  Value createApply(const IndexExpr& e);
  Value createLoad(Value memref, const std::vector<IndexExpr>& idx);
  Operation* createStore(Value v, Value memref, const std::vector<IndexExpr>& idx);
  // general-form accesses (see Operation::exprs); width 1 = affine.load / affine.store spelling
  Value createVectorLoad(Value memref, const std::vector<AffineExpr>& idx, int64_t width);
  Operation* createVectorStore(Value v, Value memref, const std::vector<AffineExpr>& idx, int64_t width);
  // affine.if (cond >= 0) { body }
  Operation* createIf(const AffineExpr& cond);
  Value createIndexConstant(int64_t v);
  // user-facing expression builders, spelled as on MLIR's OpBuilder
  AffineExpr getAffineDimExpr(unsigned position) const { return AffineExpr::dim(position); }
  AffineExpr getAffineConstantExpr(int64_t c) const { return AffineExpr::constant(c); }
  std::string getStringAttr(const std::string& s) const { return s; }
  Value createConstant(double v, ScalarKind k);
  Value createBinary(OpKind k, Value a, Value b);
  Value createExp(Value a);
  BarrierOp createBarrier();
  Operation* createAnnotation(const std::string& name, const std::vector<Value>& operands = {});

  // nest of affine.for loops with unit step; body gets the induction variables
  void buildAffineLoopNest(const std::vector<int64_t>& lbs, const std::vector<int64_t>& ubs,
                           const std::vector<int64_t>& steps,
                           const std::function<void(OpBuilder&, const std::vector<Value>&)>& body);

 private:
  Context* ctx_ = nullptr;
  InsertPoint ip_;
};

// module verification: every operand is defined before use in an enclosing scope, loops have
// positive steps, loads/stores index memrefs with the right rank, calls match their callee.
bool verify(ModuleOp module, std::string* message = nullptr);

std::vector<Operation*> usersOf(Operation* root, Value v);

}  // namespace kcgir

// Spellings used by the reference's signatures.
namespace mlir {
using Value = kcgir::Value;
using Type = kcgir::Type;
using Operation = kcgir::Operation;
using Block = kcgir::Block;
using MLIRContext = kcgir::Context;
using OpBuilder = kcgir::OpBuilder;
using ModuleOp = kcgir::ModuleOp;
using AffineForOp = kcgir::AffineForOp;
using AffineParallelOp = kcgir::AffineParallelOp;
using IndexExpr = kcgir::IndexExpr;
using AffineExpr = kcgir::AffineExpr;
using AffineMap = kcgir::AffineMap;
using MemRefType = kcgir::Type;
template <class Sig> using function_ref = std::function<Sig>;
namespace func {
using FuncOp = kcgir::FuncOp;
using CallOp = kcgir::CallOp;
}  // namespace func
namespace memref {
using AllocOp = kcgir::AllocOp;
}
namespace gpu {
using BarrierOp = kcgir::BarrierOp;
}
inline bool failed(bool ok) { return !ok; }
}  // namespace mlir

// Container spellings used by schedules written against the reference's signatures.
namespace llvm {
template <class T, unsigned N = 4> using SmallVector = std::vector<T>;
template <class T> using ArrayRef = std::vector<T>;
}  // namespace llvm
