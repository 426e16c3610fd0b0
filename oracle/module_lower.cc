// TEST INFRASTRUCTURE ONLY (like the rest of oracle/): lowers the loop nests that the product's
// own Frontend builds to scalar LLVM IR, so that the very module `Matmul::build`,
// `Relu::build`, `BatchedMatmul::build`, `Softmax::build` and `Transpose::build` produce can be
// executed on the host CPU (JIT-compiled by oracle/module_jit.py).
//
// This stands in for the step the reference declares and never wrote: lowering its affine
// module to a CPU target (`Rewriter::loweringAffineDialect`, include/Optimizer/Rewriter.h:221;
// its body is commented out, src/Optimizer/Rewriter.cc:1605-1612).  An MLIR
// affine -> scf -> cf -> LLVM lowering of these nests yields exactly this shape of code: one
// basic-block loop per `affine.for` with the induction variable and the loop-carried value as
// phi nodes, a linearised row-major address per load/store, and one separately rounded
// `fmul` / `fadd` per `arith.mulf` / `arith.addf` (no fast-math flags, so nothing is contracted
// or re-associated).  It is a second, independently derived execution of the same operator
// definitions as oracle.c: the two are compared bit for bit in tests/test_oracle_module.py.
//
// Only the un-scheduled nests are handled (for, load, store, constant, mulf, addf, maxf, divf,
// exp, alloc, return); a scheduled module (affine.parallel, kcg.* annotations) is refused.
//
// Output of oracle_module_lower(): a text with one line per module-level operation
//     alloc <value id> <dtype> <rank> <dims...>
//     call <callee> <n args> <arg value ids...> -> <result value id>
// then the line ";;;IR" and the LLVM IR of every function.  Each function `@F(ptr...)` returns
// the pointer of its result memref; `@F.rows(ptr..., i64 lo, i64 hi)` runs only iterations
// [lo, hi) of the outermost loop (rows of the result are independent in every nest, so a host
// can spread them over threads and get the same bits).
#include <cstdint>
#include <cstring>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "KernelCodeGen.h"

using namespace KernelCodeGen;
using kcgir::Block;
using kcgir::IndexExpr;
using kcgir::OpKind;
using kcgir::Operation;
using kcgir::ScalarKind;
using kcgir::ValueImpl;

namespace {

// Errors are recorded, not thrown: the library is loaded into a Python process whose C++
// runtime may differ from the one this file was built with.
thread_local std::string g_error;
void fail(const std::string& what) {
  if (g_error.empty()) g_error = what;
}

const char* llvmType(ScalarKind k) {
  switch (k) {
    case ScalarKind::F32: return "float";
    case ScalarKind::F64: return "double";
    default: fail("only float32 / float64 nests run on the CPU"); return "float";
  }
}
const char* suffix(ScalarKind k) { return k == ScalarKind::F64 ? "f64" : "f32"; }

class FuncLowering {
 public:
  FuncLowering(Operation* func, bool rows_variant) : func_(func), rows_(rows_variant) {}

  std::string run() {
    std::ostringstream head;
    head << "define ptr @\"" << func_->name << (rows_ ? ".rows" : "") << "\"(";
    Block* body = func_->body;
    for (size_t i = 0; i < body->args.size(); ++i) {
      if (i) head << ", ";
      head << "ptr %arg" << i;
      names_[body->args[i]] = "%arg" + std::to_string(i);
    }
    if (rows_) head << (body->args.empty() ? "" : ", ") << "i64 %rows.lo, i64 %rows.hi";
    head << ") {\nentry:\n";
    cur_ = "entry";
    std::ostringstream text;
    outermost_pending_ = rows_;
    emitOps(body, text);
    return head.str() + text.str() + "}\n\n";
  }

 private:
  std::string fresh(const char* p) { return std::string("%") + p + std::to_string(tmp_++); }

  std::string nameOf(kcgir::Value v) {
    auto it = names_.find(v.impl());
    if (it == names_.end()) {
      fail("use of a value the lowering has not seen");
      return "undef";
    }
    return it->second;
  }

  // i64 value of a linear index expression
  std::string index(const IndexExpr& e, std::ostringstream& os) {
    std::string acc;
    for (const auto& term : e.terms) {
      if (term.second == 0) continue;
      std::string v = nameOf(term.first);
      if (term.second != 1) {
        const std::string m = fresh("m");
        os << "  " << m << " = mul i64 " << v << ", " << term.second << "\n";
        v = m;
      }
      if (acc.empty()) acc = v;
      else {
        const std::string a = fresh("a");
        os << "  " << a << " = add i64 " << acc << ", " << v << "\n";
        acc = a;
      }
    }
    if (acc.empty()) return std::to_string(e.constant);
    if (e.constant != 0) {
      const std::string a = fresh("a");
      os << "  " << a << " = add i64 " << acc << ", " << e.constant << "\n";
      acc = a;
    }
    return acc;
  }

  // address of memref[idx...] (row-major, static shape)
  std::string address(kcgir::Value memref, const std::vector<IndexExpr>& idx, std::ostringstream& os) {
    const auto type = memref.getType();
    if (!type.isMemRef() || type.shape.size() != idx.size()) {
      fail("index rank does not match the memref");
      return "null";
    }
    IndexExpr lin = IndexExpr::cst(0);
    int64_t stride = 1;
    for (int d = static_cast<int>(idx.size()) - 1; d >= 0; --d) {
      lin = lin + idx[d] * stride;
      stride *= type.shape[d];
    }
    lin.simplify();
    const std::string off = index(lin, os);
    const std::string p = fresh("p");
    os << "  " << p << " = getelementptr " << llvmType(type.elem) << ", ptr " << nameOf(memref) << ", i64 " << off << "\n";
    return p;
  }

  void emitOps(Block* block, std::ostringstream& os) {
    for (Operation* op : block->ops) emitOp(op, os);
  }

  void emitOp(Operation* op, std::ostringstream& os) {
    switch (op->kind) {
      case OpKind::For: emitFor(op, os); break;
      case OpKind::Constant: {
        std::ostringstream lit;
        lit.precision(17);
        lit << std::scientific << op->fvalue;
        names_[op->results.at(0)] = lit.str();
        break;
      }
      case OpKind::Load: {
        const std::string p = address(op->operands.at(0), op->indices, os);
        const std::string v = fresh("v");
        os << "  " << v << " = load " << llvmType(op->getResult().getType().elem) << ", ptr " << p << "\n";
        names_[op->results.at(0)] = v;
        break;
      }
      case OpKind::Store: {
        const std::string p = address(op->operands.at(1), op->indices, os);
        os << "  store " << llvmType(op->operands.at(0).getType().elem) << " " << nameOf(op->operands.at(0)) << ", ptr " << p
           << "\n";
        break;
      }
      case OpKind::MulF:
      case OpKind::AddF:
      case OpKind::DivF: {
        const char* ins = op->kind == OpKind::MulF ? "fmul" : op->kind == OpKind::AddF ? "fadd" : "fdiv";
        const std::string v = fresh("f");
        os << "  " << v << " = " << ins << " " << llvmType(op->getResult().getType().elem) << " " << nameOf(op->operands.at(0))
           << ", " << nameOf(op->operands.at(1)) << "\n";
        names_[op->results.at(0)] = v;
        break;
      }
      case OpKind::MaxF: {   // arith.maxf: the larger operand, NaN if either is NaN
        const ScalarKind k = op->getResult().getType().elem;
        const std::string v = fresh("f");
        os << "  " << v << " = call " << llvmType(k) << " @llvm.maximum." << suffix(k) << "(" << llvmType(k) << " "
           << nameOf(op->operands.at(0)) << ", " << llvmType(k) << " " << nameOf(op->operands.at(1)) << ")\n";
        names_[op->results.at(0)] = v;
        break;
      }
      case OpKind::Exp: {    // math.exp -> the C library's exp / expf
        const ScalarKind k = op->getResult().getType().elem;
        const std::string v = fresh("f");
        os << "  " << v << " = call " << llvmType(k) << " @" << (k == ScalarKind::F64 ? "exp" : "expf") << "(" << llvmType(k)
           << " " << nameOf(op->operands.at(0)) << ")\n";
        names_[op->results.at(0)] = v;
        break;
      }
      case OpKind::Apply: {
        names_[op->results.at(0)] = index(op->indices.at(0), os);
        break;
      }
      case OpKind::Alloc: {
        const auto type = op->getResult().getType();
        int64_t bytes = kcgir::scalarBytes(type.elem);
        for (int64_t d : type.shape) bytes *= d;
        const std::string p = fresh("buf");
        os << "  " << p << " = call ptr @malloc(i64 " << bytes << ")\n";
        names_[op->results.at(0)] = p;
        break;
      }
      case OpKind::Yield:   // read by emitFor once the body has been emitted
        break;
      case OpKind::Return:
        os << "  ret ptr " << (op->operands.empty() ? std::string("null") : nameOf(op->operands.at(0))) << "\n";
        break;
      default:
        fail(std::string("operation not handled by the CPU lowering: ") + kcgir::opKindName(op->kind));
    }
  }

  void emitFor(Operation* op, std::ostringstream& os) {
    const int id = loops_++;
    const std::string L = "for" + std::to_string(id);
    const std::string pred = cur_;
    const std::string iv = "%iv" + std::to_string(id);
    const bool outer = outermost_pending_;
    outermost_pending_ = false;
    Block* body = op->body;
    names_[body->args.at(0)] = iv;
    std::vector<std::string> carried;
    for (size_t i = 0; i < op->operands.size(); ++i) {
      const std::string c = "%acc" + std::to_string(id) + "_" + std::to_string(i);
      carried.push_back(c);
      names_[body->args.at(1 + i)] = c;
    }
    std::vector<std::string> inits;
    for (auto v : op->operands) inits.push_back(nameOf(v));
    // body first (its last block and yielded values feed the phi nodes of the head)
    std::ostringstream btext;
    cur_ = L + ".body";
    emitOps(body, btext);
    std::vector<std::string> yields;
    for (Operation* child : body->ops)
      if (child->kind == OpKind::Yield)
        for (auto v : child->operands) yields.push_back(nameOf(v));
    const std::string latch = cur_;
    if (yields.size() != carried.size()) {
      fail("affine.for yields a different number of values than it carries");
      yields.resize(carried.size(), "undef");
    }
    const std::string lb = outer ? std::string("%rows.lo") : std::to_string(op->lb);
    const std::string ub = outer ? std::string("%rows.hi") : std::to_string(op->ub);
    os << "  br label %" << L << ".head\n" << L << ".head:\n";
    os << "  " << iv << " = phi i64 [ " << lb << ", %" << pred << " ], [ " << iv << ".next, %" << latch << " ]\n";
    for (size_t i = 0; i < carried.size(); ++i)
      os << "  " << carried[i] << " = phi " << llvmType(op->operands[i].getType().elem) << " [ " << inits[i] << ", %" << pred
         << " ], [ " << yields[i] << ", %" << latch << " ]\n";
    const std::string c = fresh("c");
    os << "  " << c << " = icmp slt i64 " << iv << ", " << ub << "\n";
    os << "  br i1 " << c << ", label %" << L << ".body, label %" << L << ".exit\n";
    os << L << ".body:\n" << btext.str();
    os << "  " << iv << ".next = add i64 " << iv << ", " << op->step << "\n";
    os << "  br label %" << L << ".head\n" << L << ".exit:\n";
    cur_ = L + ".exit";
    for (size_t i = 0; i < carried.size(); ++i) names_[op->results.at(i)] = carried[i];
  }

  Operation* func_;
  bool rows_;
  bool outermost_pending_ = false;
  int tmp_ = 0, loops_ = 0;
  std::string cur_;
  std::map<ValueImpl*, std::string> names_;
};

std::string dtypeName(ScalarKind k) { return k == ScalarKind::F64 ? "float64" : "float32"; }

std::string lowerModule(mlir::ModuleOp module) {
  std::ostringstream prog, ir;
  std::map<ValueImpl*, int> ids;
  int next = 0;
  ir << "declare ptr @malloc(i64)\ndeclare float @expf(float)\ndeclare double @exp(double)\n"
     << "declare float @llvm.maximum.f32(float, float)\ndeclare double @llvm.maximum.f64(double, double)\n\n";
  for (Operation* op : module.getBody()->getOperations()) {
    if (op->kind == OpKind::Func) {
      ir << FuncLowering(op, false).run() << FuncLowering(op, true).run();
    } else if (op->kind == OpKind::Alloc) {
      const auto type = op->getResult().getType();
      ids[op->results.at(0)] = next;
      prog << "alloc " << next++ << " " << dtypeName(type.elem) << " " << type.shape.size();
      for (int64_t d : type.shape) prog << " " << d;
      prog << "\n";
    } else if (op->kind == OpKind::Call) {
      prog << "call " << op->name << " " << op->operands.size();
      for (auto v : op->operands) {
        auto it = ids.find(v.impl());
        if (it == ids.end()) {
          fail("call operand is not a module-level value");
          continue;
        }
        prog << " " << it->second;
      }
      ids[op->results.at(0)] = next;
      prog << " -> " << next++ << "\n";
    } else {
      fail(std::string("module-level operation not handled: ") + kcgir::opKindName(op->kind));
    }
  }
  return prog.str() + ";;;IR\n" + ir.str();
}

// Builds one of the graphs the tests and the CPU baseline use through the Frontend.
mlir::ModuleOp buildGraph(KernelCodeGenerator& gen, const std::string& graph, const std::vector<int64_t>& d,
                          const std::string& dtype) {
  auto& g = gen.createGraph("oracle_" + graph);
  auto ph = [&](std::vector<int64_t> shape) { return g.create<PlaceHolder>(shape, dtype); };
  auto lead = [&](size_t tail) { return std::vector<int64_t>(d.begin(), d.end() - tail); };
  auto with = [](std::vector<int64_t> v, std::initializer_list<int64_t> t) {
    v.insert(v.end(), t);
    return v;
  };
  if (graph == "matmul" || graph == "matmul_relu") {           // dims: m n k
    if (d.size() != 3) { fail("matmul takes m n k"); return g.module; }
    auto A = ph({d[0], d[2]}), B = ph({d[2], d[1]});
    auto C = g.create<Matmul>(A, B, MemorySpace::global);
    if (graph == "matmul_relu") g.create<Relu>(C, MemorySpace::inplace);
  } else if (graph == "relu") {                                  // dims: shape...
    g.create<Relu>(ph(d), MemorySpace::inplace);
  } else if (graph == "batched_matmul_nn" || graph == "batched_matmul_nt") {   // dims: batch... m n k
    if (d.size() < 3) { fail("batched matmul takes batch... m n k"); return g.module; }
    const int64_t m = d[d.size() - 3], n = d[d.size() - 2], k = d[d.size() - 1];
    const bool nt = graph == "batched_matmul_nt";
    auto A = ph(with(lead(3), {m, k}));
    auto B = nt ? ph(with(lead(3), {n, k})) : ph(with(lead(3), {k, n}));
    g.create<BatchedMatmul>(A, Layout::rowMajor, B, nt ? Layout::colMajor : Layout::rowMajor);
  } else if (graph == "softmax") {                               // dims: shape...
    g.create<Softmax>(ph(d), -1, MemorySpace::inplace);
  } else if (graph == "transpose") {
    g.create<Transpose>(ph(d));
  } else if (graph == "attention") {                             // dims: batch... sq skv hd (test/test.cc:80-90)
    if (d.size() < 3) { fail("attention takes batch... sq skv hd"); return g.module; }
    const int64_t sq = d[d.size() - 3], skv = d[d.size() - 2], hd = d[d.size() - 1];
    auto Q = ph(with(lead(3), {sq, hd})), K = ph(with(lead(3), {skv, hd})), V = ph(with(lead(3), {skv, hd}));
    auto S = g.create<BatchedMatmul>(Q, Layout::rowMajor, K, Layout::colMajor);
    auto P = g.create<Softmax>(S, -1, MemorySpace::inplace);
    g.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor);
  } else {
    fail("unknown graph \"" + graph + "\"");
  }
  return g.module;
}

}  // namespace

extern "C" {

// Returns the number of bytes of the text (excluding the terminating 0) and copies at most
// cap - 1 of them to `out`; a negative value reports an error, whose message is copied instead.
long oracle_module_lower(const char* graph, const char* dtype, const int64_t* dims, int ndims, char* out, size_t cap) {
  std::string text;
  long rc = 0;
  g_error.clear();
  {
    KernelCodeGenerator gen("CUDA");
    gen.setLogMode(Log::Release);
    mlir::ModuleOp module = buildGraph(gen, graph ? graph : "", std::vector<int64_t>(dims, dims + ndims), dtype ? dtype : "float32");
    std::string why;
    if (g_error.empty() && !kcgir::verify(module, &why)) fail("the Frontend's module does not verify: " + why);
    if (g_error.empty()) text = lowerModule(module);
  }
  if (g_error.empty()) {
    rc = static_cast<long>(text.size());
  } else {
    text = g_error;
    rc = -1;
  }
  if (out && cap) {
    const size_t n = text.size() < cap - 1 ? text.size() : cap - 1;
    std::memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return rc;
}

}  // extern "C"
