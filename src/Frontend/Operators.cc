// Frontend operators: each emits `func.func @<Name>` with the naive affine nest and a call to
// it at the builder's position.  Semantics follow the reference line by line (citations at each
// operator); construction goes through the IR of include/IR/IR.h.
#include "Frontend/Operators.h"

namespace KernelCodeGen {

using kcgir::IndexExpr;
using kcgir::OpKind;
using kcgir::ScalarKind;

mlir::Type getDType(mlir::OpBuilder&, const std::string& dtype) {
  if (dtype == "float32") return mlir::Type::scalar(ScalarKind::F32);
  if (dtype == "float64") return mlir::Type::scalar(ScalarKind::F64);
  if (dtype == "float16") return mlir::Type::scalar(ScalarKind::F16);
  if (dtype == "bfloat16") return mlir::Type::scalar(ScalarKind::BF16);  // not in the reference
  return mlir::Type();
}

std::string toStr(const mlir::Type& type) {
  switch (type.elem) {
    case ScalarKind::F16: return "float16";
    case ScalarKind::BF16: return "bfloat16";
    case ScalarKind::F32: return "float32";
    case ScalarKind::F64: return "float64";
    default: return "";
  }
}

mlir::func::FuncOp buildFuction(mlir::ModuleOp module, mlir::OpBuilder& builder, const std::string& funcName,
                                const std::vector<mlir::Type>& inputsTypes,
                                const std::vector<mlir::Type>& outputsTypes) {
  // An operator used twice with the same shapes shares one function (reference :26-36).
  for (mlir::Operation* op : module.getBody()->getOperations())
    if (op->kind == OpKind::Func && op->name == funcName) return mlir::func::FuncOp(op);
  builder.setInsertionPointToStart(module.getBody());
  return builder.createFunc(funcName, inputsTypes, outputsTypes);
}

static bool hasBody(mlir::func::FuncOp f) { return !f.getBody()->getOperations().empty(); }

// reference: src/Frontend/Operators.cc:64-75
mlir::Value PlaceHolder::build(ComputeDAG* graph, const std::vector<int64_t>& shapes, const std::string& dtype) {
  auto& builder = graph->builder;
  mlir::Type elem = getDType(builder, dtype);
  if (elem.isNone()) {
    std::cerr << "PlaceHolder: unknown dtype \"" << dtype << "\".\n";
    return nullptr;
  }
  return builder.createAlloc(mlir::Type::memRef(shapes, elem.elem, static_cast<int>(MemorySpace::global)));
}

// reference: src/Frontend/Operators.cc:77-179
//   for i < m, j < n { acc = 0; for k < K: acc = A[i,k]*B[k,j] + acc; C[i,j] = acc }
mlir::Value Matmul::build(ComputeDAG* graph, mlir::Value A, mlir::Value B, MemorySpace ms,
                          const std::string& dtype_) {
  auto& builder = graph->builder;
  if (!A || !A.getType().isMemRef()) {
    std::cerr << "Type of left operand of Matmul is not Memref.\n";
    return nullptr;
  }
  if (!B || !B.getType().isMemRef()) {
    std::cerr << "Type of right operand of Matmul is not Memref.\n";
    return nullptr;
  }
  const auto typeA = A.getType(), typeB = B.getType();
  if (typeA.shape.size() != 2 || typeB.shape.size() != 2) {
    std::cerr << "Matmul takes rank-2 operands.\n";
    return nullptr;
  }
  const int64_t m = typeA.shape[0], k1 = typeA.shape[1], k2 = typeB.shape[0], n = typeB.shape[1];
  if (k1 != k2) {
    std::cerr << "Can't apply Matmul Operation due to imcompatible K-dim.\n";
    return nullptr;
  }
  const std::string dtype = dtype_ != "" ? dtype_ : toStr(typeA);
  const mlir::Type em = getDType(builder, dtype);
  const auto funcName = "Matmul_m" + std::to_string(m) + "n" + std::to_string(n) + "k" + std::to_string(k1);
  const auto typeC = mlir::Type::memRef({m, n}, em.elem, static_cast<int>(ms));
  mlir::Value C = builder.createAlloc(typeC);

  auto ip = builder.saveInsertionPoint();
  auto funcOp = buildFuction(graph->module, builder, funcName, {typeA, typeB, typeC}, {typeC});
  if (!hasBody(funcOp)) {
    builder.setInsertionPointToStart(funcOp.getBody());
    const mlir::Value a = funcOp.getArgument(0), b = funcOp.getArgument(1), c = funcOp.getArgument(2);
    builder.buildAffineLoopNest({0, 0}, {m, n}, {1, 1}, [&](mlir::OpBuilder& nb, const std::vector<mlir::Value>& ivs) {
      const mlir::Value i = ivs[0], j = ivs[1];
      mlir::Value zero = nb.createConstant(0.0, em.elem);
      auto kLoop = nb.createFor(0, k1, 1, {zero}, [&](mlir::OpBuilder& kb, mlir::Value k, const std::vector<mlir::Value>& it) {
        mlir::Value ld_a = kb.createLoad(a, {IndexExpr(i), IndexExpr(k)});
        mlir::Value ld_b = kb.createLoad(b, {IndexExpr(k), IndexExpr(j)});
        mlir::Value mul = kb.createBinary(OpKind::MulF, ld_a, ld_b);
        mlir::Value add = kb.createBinary(OpKind::AddF, mul, it[0]);
        kb.createYield({add});
      });
      nb.createStore(kLoop.getResult(0), c, {IndexExpr(i), IndexExpr(j)});
    });
    builder.setInsertionPointToEnd(funcOp.getBody());
    builder.createReturn({c});
    funcOp->setAttr("func.state", std::string("cpu"));
  }
  builder.restoreInsertionPoint(ip);
  return builder.createCall(funcOp, {A, B, C}).getResult(0);
}

// reference: src/Frontend/Operators.cc:182-250: out[idx] = arith.maxf(0, in[idx])
mlir::Value Relu::build(ComputeDAG* graph, mlir::Value input, MemorySpace ms, const std::string& dtype_) {
  auto& builder = graph->builder;
  if (!input || !input.getType().isMemRef()) {
    std::cerr << "Type of input of Relu is not Memref.\n";
    return nullptr;
  }
  const auto type = input.getType();
  const std::string dtype = dtype_ != "" ? dtype_ : toStr(type);
  const mlir::Type em = getDType(builder, dtype);
  std::string funcName = "Relu_Elementwise";
  for (auto dim : type.shape) funcName += "_" + std::to_string(dim);

  auto ip = builder.saveInsertionPoint();
  auto funcOp = buildFuction(graph->module, builder, funcName, {type}, {type});
  if (!hasBody(funcOp)) {
    builder.setInsertionPointToStart(funcOp.getBody());
    mlir::Value in = funcOp.getArgument(0);
    mlir::Value out = in;
    if (ms != MemorySpace::inplace) out = builder.createAlloc(mlir::Type::memRef(type.shape, em.elem, static_cast<int>(ms)));
    std::vector<int64_t> zeros(type.shape.size(), 0), ones(type.shape.size(), 1);
    builder.buildAffineLoopNest(zeros, type.shape, ones, [&](mlir::OpBuilder& nb, const std::vector<mlir::Value>& ivs) {
      std::vector<IndexExpr> idx(ivs.begin(), ivs.end());
      mlir::Value zero = nb.createConstant(0.0, em.elem);
      mlir::Value x = nb.createLoad(in, idx);
      mlir::Value mx = nb.createBinary(OpKind::MaxF, zero, x);
      nb.createStore(mx, out, idx);
    });
    builder.setInsertionPointToEnd(funcOp.getBody());
    builder.createReturn({out});
    funcOp->setAttr("func.state", std::string("cpu"));
    funcOp->setAttr("kcg.inplace", static_cast<int64_t>(ms == MemorySpace::inplace));
  }
  builder.restoreInsertionPoint(ip);
  return builder.createCall(funcOp, {input}).getResult(0);
}

// reference: src/Frontend/Operators.cc:253-420
mlir::Value BatchedMatmul::build(ComputeDAG* graph, mlir::Value A, Layout layoutA, mlir::Value B, Layout layoutB,
                                 const std::string& dtype_) {
  auto& builder = graph->builder;
  if (!A || !A.getType().isMemRef()) {
    std::cerr << "Type of left operand of BatchedMatmul is not Memref.\n";
    return nullptr;
  }
  if (!B || !B.getType().isMemRef()) {
    std::cerr << "Type of right operand of BatchedMatmul is not Memref.\n";
    return nullptr;
  }
  const auto typeA = A.getType(), typeB = B.getType();
  const int totalDims = static_cast<int>(typeA.shape.size());
  if (totalDims < 2) {
    std::cerr << "BatchedMatmul needs at least 2 dim but got " << totalDims << "\n";
    return nullptr;
  }
  if (static_cast<int>(typeB.shape.size()) != totalDims) {
    std::cerr << "BatchedMatmul: A, B dim not matched.\n";
    return nullptr;
  }
  std::vector<int64_t> shapeC = typeA.shape;
  int64_t m, n, k1, k2;
  if (layoutA == Layout::rowMajor) { m = typeA.shape[totalDims - 2]; k1 = typeA.shape[totalDims - 1]; }
  else { m = typeA.shape[totalDims - 1]; k1 = typeA.shape[totalDims - 2]; }
  if (layoutB == Layout::colMajor) { k2 = typeB.shape[totalDims - 1]; n = typeB.shape[totalDims - 2]; }
  else { k2 = typeB.shape[totalDims - 2]; n = typeB.shape[totalDims - 1]; }
  shapeC[totalDims - 2] = m;
  shapeC[totalDims - 1] = n;
  if (k1 != k2) {
    std::cerr << "Can't apply BatchedMatmul Operation due to imcompatible K-dim.\n";
    return nullptr;
  }
  const std::string dtype = dtype_ != "" ? dtype_ : toStr(typeA);
  const mlir::Type em = getDType(builder, dtype);
  mlir::Value C = graph->create<PlaceHolder>(shapeC, dtype);
  const auto typeC = C.getType();

  const int batchDims = totalDims - 2;
  std::string funcName = "BatchMatmul";
  for (int i = 0; i < batchDims; ++i) funcName += "_" + std::to_string(shapeC[i]);
  funcName += "_m" + std::to_string(m) + "_n" + std::to_string(n) + "_k" + std::to_string(k1) + "_" +
              (layoutA == Layout::rowMajor ? 'N' : 'T') + (layoutB == Layout::rowMajor ? 'N' : 'T');

  auto ip = builder.saveInsertionPoint();
  auto funcOp = buildFuction(graph->module, builder, funcName, {typeA, typeB, typeC}, {typeC});
  if (!hasBody(funcOp)) {
    builder.setInsertionPointToStart(funcOp.getBody());
    const mlir::Value a = funcOp.getArgument(0), b = funcOp.getArgument(1), c = funcOp.getArgument(2);
    std::vector<int64_t> zeros(totalDims, 0), ones(totalDims, 1);
    builder.buildAffineLoopNest(zeros, shapeC, ones, [&](mlir::OpBuilder& nb, const std::vector<mlir::Value>& ivs) {
      const mlir::Value i = ivs[totalDims - 2], j = ivs[totalDims - 1];
      std::vector<IndexExpr> batch(ivs.begin(), ivs.begin() + batchDims);
      mlir::Value zero = nb.createConstant(0.0, em.elem);
      auto kLoop = nb.createFor(0, k1, 1, {zero}, [&](mlir::OpBuilder& kb, mlir::Value k, const std::vector<mlir::Value>& it) {
        std::vector<IndexExpr> ia = batch, ib = batch;
        // The reference indexes a colMajor A with (k, j) (src/Frontend/Operators.cc:391), which
        // reads the wrong element; the transposed operand is addressed (k, i) here.
        if (layoutA == Layout::rowMajor) { ia.push_back(i); ia.push_back(k); } else { ia.push_back(k); ia.push_back(i); }
        if (layoutB == Layout::rowMajor) { ib.push_back(k); ib.push_back(j); } else { ib.push_back(j); ib.push_back(k); }
        mlir::Value ld_a = kb.createLoad(a, ia);
        mlir::Value ld_b = kb.createLoad(b, ib);
        mlir::Value mul = kb.createBinary(OpKind::MulF, ld_a, ld_b);
        mlir::Value add = kb.createBinary(OpKind::AddF, mul, it[0]);
        kb.createYield({add});
      });
      std::vector<IndexExpr> ic = batch;
      ic.push_back(i);
      ic.push_back(j);
      nb.createStore(kLoop.getResult(0), c, ic);
    });
    builder.setInsertionPointToEnd(funcOp.getBody());
    builder.createReturn({c});
    funcOp->setAttr("func.state", std::string("cpu"));
  }
  builder.restoreInsertionPoint(ip);
  return builder.createCall(funcOp, {A, B, C}).getResult(0);
}

// reference: src/Frontend/Operators.cc:425-542 (last axis only, no max subtraction)
mlir::Value Softmax::build(ComputeDAG* graph, mlir::Value input, int axis, MemorySpace ms, const std::string& dtype_) {
  auto& builder = graph->builder;
  if (!input || !input.getType().isMemRef()) {
    std::cerr << "Type of input of Softmax is not Memref.\n";
    return nullptr;
  }
  const auto type = input.getType();
  const int totalDims = static_cast<int>(type.shape.size());
  const int reduceAxis = axis == -1 ? totalDims - 1 : axis;
  if (reduceAxis != totalDims - 1) {
    std::cerr << "At present, only support reduction on the last dim.\n";
    return nullptr;
  }
  const std::string dtype = dtype_ != "" ? dtype_ : toStr(type);
  const mlir::Type em = getDType(builder, dtype);
  std::string funcName = "Softmax";
  for (auto dim : type.shape) funcName += "_" + std::to_string(dim);
  funcName += "_axis" + std::to_string(reduceAxis);

  auto ip = builder.saveInsertionPoint();
  auto funcOp = buildFuction(graph->module, builder, funcName, {type}, {type});
  if (!hasBody(funcOp)) {
    builder.setInsertionPointToStart(funcOp.getBody());
    mlir::Value x = funcOp.getArgument(0);
    mlir::Value out = x;
    if (ms != MemorySpace::inplace && ms != MemorySpace::global)
      out = builder.createAlloc(mlir::Type::memRef(type.shape, em.elem, static_cast<int>(ms)));
    std::vector<int64_t> ubs(type.shape.begin(), type.shape.begin() + reduceAxis);
    std::vector<int64_t> zeros(ubs.size(), 0), ones(ubs.size(), 1);
    const int64_t cols = type.shape.back();
    builder.buildAffineLoopNest(zeros, ubs, ones, [&](mlir::OpBuilder& nb, const std::vector<mlir::Value>& ivs) {
      std::vector<IndexExpr> lead(ivs.begin(), ivs.end());
      mlir::Value zero = nb.createConstant(0.0, em.elem);
      auto sum = nb.createFor(0, cols, 1, {zero}, [&](mlir::OpBuilder& kb, mlir::Value k, const std::vector<mlir::Value>& it) {
        auto idx = lead;
        idx.push_back(k);
        mlir::Value e = kb.createExp(kb.createLoad(x, idx));
        kb.createYield({kb.createBinary(OpKind::AddF, e, it[0])});
      });
      nb.createFor(0, cols, 1, {}, [&](mlir::OpBuilder& eb, mlir::Value k, const std::vector<mlir::Value>&) {
        auto idx = lead;
        idx.push_back(k);
        mlir::Value e = eb.createExp(eb.createLoad(x, idx));
        eb.createStore(eb.createBinary(OpKind::DivF, e, sum.getResult(0)), out, idx);
      });
    });
    builder.setInsertionPointToEnd(funcOp.getBody());
    builder.createReturn({out});
    funcOp->setAttr("func.state", std::string("cpu"));
  }
  builder.restoreInsertionPoint(ip);
  return builder.createCall(funcOp, {input}).getResult(0);
}

mlir::Value Transpose::build(ComputeDAG* graph, mlir::Value input) {
  auto& builder = graph->builder;
  if (!input || !input.getType().isMemRef()) {
    std::cerr << "Type of input of Transpose is not Memref.\n";
    return nullptr;
  }
  const auto type = input.getType();
  const int totalDims = static_cast<int>(type.shape.size());
  if (totalDims < 2) {
    std::cerr << "Transpose needs at least 2 dim but got " << totalDims << "\n";
    return nullptr;
  }
  std::vector<int64_t> shapeOut = type.shape;
  std::swap(shapeOut[totalDims - 2], shapeOut[totalDims - 1]);
  const std::string dtype = toStr(type);
  mlir::Value out = graph->create<PlaceHolder>(shapeOut, dtype);
  const auto typeOut = out.getType();
  std::string funcName = "Transpose";
  for (auto dim : type.shape) funcName += "_" + std::to_string(dim);

  auto ip = builder.saveInsertionPoint();
  auto funcOp = buildFuction(graph->module, builder, funcName, {type, typeOut}, {typeOut});
  if (!hasBody(funcOp)) {
    builder.setInsertionPointToStart(funcOp.getBody());
    const mlir::Value x = funcOp.getArgument(0), y = funcOp.getArgument(1);
    std::vector<int64_t> zeros(totalDims, 0), ones(totalDims, 1);
    builder.buildAffineLoopNest(zeros, type.shape, ones, [&](mlir::OpBuilder& nb, const std::vector<mlir::Value>& ivs) {
      std::vector<IndexExpr> src(ivs.begin(), ivs.end()), dst(ivs.begin(), ivs.end());
      std::swap(dst[totalDims - 2], dst[totalDims - 1]);
      nb.createStore(nb.createLoad(x, src), y, dst);
    });
    builder.setInsertionPointToEnd(funcOp.getBody());
    builder.createReturn({y});
    funcOp->setAttr("func.state", std::string("cpu"));
  }
  builder.restoreInsertionPoint(ip);
  return builder.createCall(funcOp, {input, out}).getResult(0);
}

}  // namespace KernelCodeGen
