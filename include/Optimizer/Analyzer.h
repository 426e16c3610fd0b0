// Queries over the IR used by the optimizers (reference: include/Optimizer/Analyzer.h:9-82,
// src/Optimizer/Analyzer.cc:42-107).
#pragma once

#include <string>
#include <vector>

#include "IR/IR.h"

namespace KernelCodeGen {

// Strict-weak orderings by handle identity, for std::set / std::map keys.
struct CompareLoop {
  bool operator()(const mlir::AffineForOp& x, const mlir::AffineForOp& y) const {
    return x.getOperation() < y.getOperation();
  }
};
struct CompareFunc {
  bool operator()(const mlir::func::FuncOp& x, const mlir::func::FuncOp& y) const {
    return x.getOperation() < y.getOperation();
  }
};
struct CompareFuncCall {
  bool operator()(const mlir::func::CallOp& x, const mlir::func::CallOp& y) const {
    return x.getOperation() < y.getOperation();
  }
};

struct Analyzer {
  Analyzer() = default;

  // Outermost affine.for of every function and of the module body.
  static std::vector<mlir::AffineForOp> collectOutermostLoop(mlir::ModuleOp& module);

  // Extent of each dimension of a parallel level; totalNumber = their product.
  static std::vector<int64_t> getParallelNumber(mlir::AffineParallelOp parallelLevel, int64_t& totalNumber);

  // Functions whose name contains `targetFuncName` (all functions when empty).
  static std::vector<mlir::func::FuncOp> collectFunctions(mlir::ModuleOp& module,
                                                          const std::string& targetFuncName = {""});
  // All affine.for ops of a function in pre-order (for the matmul nest: [M, N, K]).
  static std::vector<mlir::AffineForOp> collectFuncLoops(mlir::func::FuncOp funcOp);
  // func.call ops of the module body, in program order.
  static std::vector<mlir::func::CallOp> collectFuncCalls(mlir::ModuleOp& module);
  static mlir::func::FuncOp getTargetFunction(mlir::ModuleOp& module, const std::string& targetFuncName);
  // Number of operations that use `value` anywhere below `module`.
  static int getUsersNumber(mlir::ModuleOp& module, mlir::Value value);

  // Last direct child of `father` that is of kind `kind`.
  static mlir::Operation* getLastOp(mlir::Block* body, kcgir::OpKind kind);
};

}  // namespace KernelCodeGen
