// Quasi-affine index expressions of the mini IR (include/IR/IR.h): what MLIR's AffineExpr /
// AffineMap provide to the reference's schedule code (src/Optimizer/Optimizer.cc:272-381 builds
// its tile maps from dims with +, *, floorDiv and %), reduced to what those maps need.
#include <cassert>
#include <sstream>

#include "IR/IR.h"

namespace kcgir {

struct AffineExpr::Node {
  Kind kind = Kind::Cst;
  int64_t c = 0;          // Cst: the value; Dim: the position; Mul / FloorDiv / Mod: the constant operand
  Value v;                // Val
  AffineExpr a, b;        // Add: both; Mul / FloorDiv / Mod: a
};

static int64_t floordiv(int64_t x, int64_t d) {
  int64_t q = x / d;
  if ((x % d != 0) && ((x < 0) != (d < 0))) --q;
  return q;
}

AffineExpr::AffineExpr() : node_(nullptr) {}

AffineExpr AffineExpr::make(Kind k, int64_t c, const AffineExpr* a, const AffineExpr* b) {
  auto n = std::make_shared<Node>();
  n->kind = k;
  n->c = c;
  if (a) n->a = *a;
  if (b) n->b = *b;
  return AffineExpr(std::shared_ptr<const Node>(std::move(n)));
}

AffineExpr AffineExpr::constant(int64_t c) { return make(Kind::Cst, c, nullptr, nullptr); }
AffineExpr AffineExpr::dim(unsigned position) { return make(Kind::Dim, position, nullptr, nullptr); }
AffineExpr AffineExpr::value(Value v) {
  auto n = std::make_shared<Node>();
  n->kind = Kind::Val;
  n->v = v;
  return AffineExpr(std::shared_ptr<const Node>(std::move(n)));
}

AffineExpr AffineExpr::fromLinear(const IndexExpr& e) {
  AffineExpr r = constant(0);
  for (const auto& t : e.terms)
    if (t.second != 0) r = r + value(t.first) * t.second;
  return r + constant(e.constant);
}

AffineExpr::Kind AffineExpr::kind() const { return node_ ? node_->kind : Kind::Cst; }
int64_t AffineExpr::constantValue() const { return node_ ? node_->c : 0; }
unsigned AffineExpr::dimPosition() const { return static_cast<unsigned>(node_->c); }
Value AffineExpr::leafValue() const { return node_ ? node_->v : Value(); }

AffineExpr AffineExpr::lhs() const { return node_ ? node_->a : AffineExpr(); }
AffineExpr AffineExpr::rhs() const {
  if (!node_) return AffineExpr();
  return node_->kind == Kind::Add ? node_->b : constant(node_->c);
}

AffineExpr AffineExpr::operator+(const AffineExpr& o) const {
  if (isConstant() && o.isConstant()) return constant(constantValue() + o.constantValue());
  if (isConstant() && constantValue() == 0) return o;
  if (o.isConstant() && o.constantValue() == 0) return *this;
  // keep a single trailing constant: (x + c1) + c2 -> x + (c1 + c2)
  if (o.isConstant() && kind() == Kind::Add && node_->b.isConstant())
    return node_->a + constant(node_->b.constantValue() + o.constantValue());
  if (isConstant()) return o + *this;           // constants go last, as MLIR prints them
  return make(Kind::Add, 0, this, &o);
}

AffineExpr AffineExpr::operator*(int64_t c) const {
  if (isConstant()) return constant(constantValue() * c);
  if (c == 1) return *this;
  if (c == 0) return constant(0);
  if (kind() == Kind::Mul) return node_->a * (node_->c * c);
  return make(Kind::Mul, c, this, nullptr);
}

AffineExpr AffineExpr::operator*(const AffineExpr& o) const {
  if (o.isConstant()) return *this * o.constantValue();
  assert(isConstant() && "affine expressions multiply by constants only");
  return o * constantValue();
}

AffineExpr AffineExpr::floorDiv(int64_t c) const {
  assert(c > 0 && "floordiv by a positive constant");
  if (isConstant()) return constant(floordiv(constantValue(), c));
  if (c == 1) return *this;
  if (kind() == Kind::Mul && node_->c % c == 0) return node_->a * (node_->c / c);
  // (x + k * c) floordiv c = x floordiv c + k
  if (kind() == Kind::Add && node_->b.isConstant() && node_->b.constantValue() % c == 0)
    return node_->a.floorDiv(c) + constant(node_->b.constantValue() / c);
  return make(Kind::FloorDiv, c, this, nullptr);
}

AffineExpr AffineExpr::operator%(int64_t c) const {
  assert(c > 0 && "mod by a positive constant");
  if (isConstant()) return constant(constantValue() - floordiv(constantValue(), c) * c);
  if (c == 1) return constant(0);
  if (kind() == Kind::Mul && node_->c % c == 0) return constant(0);
  return make(Kind::Mod, c, this, nullptr);
}

AffineExpr AffineExpr::replaceDims(const std::vector<AffineExpr>& by) const {
  switch (kind()) {
    case Kind::Cst:
    case Kind::Val: return *this;
    case Kind::Dim: assert(dimPosition() < by.size() && "map applied to too few operands"); return by[dimPosition()];
    case Kind::Add: return node_->a.replaceDims(by) + node_->b.replaceDims(by);
    case Kind::Mul: return node_->a.replaceDims(by) * node_->c;
    case Kind::FloorDiv: return node_->a.replaceDims(by).floorDiv(node_->c);
    case Kind::Mod: return node_->a.replaceDims(by) % node_->c;
  }
  return *this;
}

AffineExpr AffineExpr::replaceValue(Value from, const AffineExpr& to) const {
  switch (kind()) {
    case Kind::Cst:
    case Kind::Dim: return *this;
    case Kind::Val: return node_->v == from ? to : *this;
    case Kind::Add: return node_->a.replaceValue(from, to) + node_->b.replaceValue(from, to);
    case Kind::Mul: return node_->a.replaceValue(from, to) * node_->c;
    case Kind::FloorDiv: return node_->a.replaceValue(from, to).floorDiv(node_->c);
    case Kind::Mod: return node_->a.replaceValue(from, to) % node_->c;
  }
  return *this;
}

AffineExpr AffineExpr::mapValues(const std::function<Value(Value)>& fn) const {
  switch (kind()) {
    case Kind::Cst:
    case Kind::Dim: return *this;
    case Kind::Val: return value(fn(node_->v));
    case Kind::Add: return node_->a.mapValues(fn) + node_->b.mapValues(fn);
    case Kind::Mul: return node_->a.mapValues(fn) * node_->c;
    case Kind::FloorDiv: return node_->a.mapValues(fn).floorDiv(node_->c);
    case Kind::Mod: return node_->a.mapValues(fn) % node_->c;
  }
  return *this;
}

bool AffineExpr::uses(Value v) const {
  switch (kind()) {
    case Kind::Cst:
    case Kind::Dim: return false;
    case Kind::Val: return node_->v == v;
    case Kind::Add: return node_->a.uses(v) || node_->b.uses(v);
    default: return node_->a.uses(v);
  }
}

void AffineExpr::collectValues(std::vector<Value>& out) const {
  switch (kind()) {
    case Kind::Cst:
    case Kind::Dim: return;
    case Kind::Val: out.push_back(node_->v); return;
    case Kind::Add: node_->a.collectValues(out); node_->b.collectValues(out); return;
    default: node_->a.collectValues(out); return;
  }
}

int64_t AffineExpr::evaluate(const std::function<int64_t(Value)>& valueOf) const {
  switch (kind()) {
    case Kind::Cst: return constantValue();
    case Kind::Dim: assert(false && "evaluate: apply the map to operands first"); return 0;
    case Kind::Val: return valueOf(node_->v);
    case Kind::Add: return node_->a.evaluate(valueOf) + node_->b.evaluate(valueOf);
    case Kind::Mul: return node_->a.evaluate(valueOf) * node_->c;
    case Kind::FloorDiv: return floordiv(node_->a.evaluate(valueOf), node_->c);
    case Kind::Mod: {
      const int64_t x = node_->a.evaluate(valueOf);
      return x - floordiv(x, node_->c) * node_->c;
    }
  }
  return 0;
}

bool AffineExpr::toLinear(IndexExpr* out) const {
  switch (kind()) {
    case Kind::Cst: *out = IndexExpr::cst(constantValue()); return true;
    case Kind::Dim: return false;
    case Kind::Val: *out = IndexExpr(node_->v); return true;
    case Kind::Add: {
      IndexExpr a, b;
      if (!node_->a.toLinear(&a) || !node_->b.toLinear(&b)) return false;
      *out = a + b;
      out->simplify();
      return true;
    }
    case Kind::Mul: {
      IndexExpr a;
      if (!node_->a.toLinear(&a)) return false;
      *out = a * node_->c;
      return true;
    }
    default: return false;
  }
}

std::string AffineExpr::str(const std::function<std::string(Value)>& nameOf) const {
  // precedence: add (1) < mul / floordiv / mod (2) < leaf (3); operands of the tighter operators
  // are parenthesised when they are sums or themselves compound, as MLIR prints them
  std::function<std::string(const AffineExpr&, int)> go = [&](const AffineExpr& e, int parent) -> std::string {
    std::ostringstream os;
    switch (e.kind()) {
      case Kind::Cst: os << e.constantValue(); return os.str();
      case Kind::Dim: os << "d" << e.dimPosition(); return os.str();
      case Kind::Val: return nameOf(e.leafValue());
      case Kind::Add: {
        const AffineExpr& b = e.node_->b;
        std::string s = go(e.node_->a, 1);
        if (b.isConstant() && b.constantValue() < 0) s += " - " + std::to_string(-b.constantValue());
        else s += " + " + go(b, 1);
        return parent > 1 ? "(" + s + ")" : s;
      }
      case Kind::Mul: {
        std::string s = go(e.node_->a, 3) + " * " + std::to_string(e.node_->c);
        return parent > 2 ? "(" + s + ")" : s;
      }
      case Kind::FloorDiv: {
        std::string s = go(e.node_->a, 3) + " floordiv " + std::to_string(e.node_->c);
        return parent > 2 ? "(" + s + ")" : s;
      }
      case Kind::Mod: {
        std::string s = go(e.node_->a, 3) + " mod " + std::to_string(e.node_->c);
        return parent > 2 ? "(" + s + ")" : s;
      }
    }
    return "?";
  };
  return go(*this, 0);
}

std::vector<AffineExpr> AffineMap::apply(const std::vector<AffineExpr>& operands) const {
  assert(operands.size() >= numDims_ && "map applied to too few operands");
  std::vector<AffineExpr> out;
  for (const auto& r : results_) out.push_back(r.replaceDims(operands));
  return out;
}

}  // namespace kcgir
