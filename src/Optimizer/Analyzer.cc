#include "Optimizer/Analyzer.h"

namespace KernelCodeGen {

using kcgir::OpKind;

std::vector<mlir::AffineForOp> Analyzer::collectOutermostLoop(mlir::ModuleOp& module) {
  std::vector<mlir::AffineForOp> res;
  std::function<void(mlir::Block*)> scan = [&](mlir::Block* b) {
    for (mlir::Operation* op : b->getOperations()) {
      if (op->kind == OpKind::For) res.emplace_back(op);
      else if (op->kind == OpKind::Func || op->kind == OpKind::Parallel) scan(op->body);
    }
  };
  scan(module.getBody());
  return res;
}

std::vector<int64_t> Analyzer::getParallelNumber(mlir::AffineParallelOp parallelLevel, int64_t& totalNumber) {
  totalNumber = 1;
  std::vector<int64_t> result;
  for (size_t i = 0; i < parallelLevel.getNumDims(); ++i) {
    totalNumber *= parallelLevel.getExtent(i);
    result.push_back(parallelLevel.getExtent(i));
  }
  return result;
}

std::vector<mlir::func::FuncOp> Analyzer::collectFunctions(mlir::ModuleOp& module, const std::string& targetFuncName) {
  std::vector<mlir::func::FuncOp> res;
  for (mlir::Operation* op : module.getBody()->getOperations()) {
    if (op->kind != OpKind::Func) continue;
    if (targetFuncName.empty() || op->name.find(targetFuncName) != std::string::npos) res.emplace_back(op);
  }
  return res;
}

std::vector<mlir::AffineForOp> Analyzer::collectFuncLoops(mlir::func::FuncOp funcOp) {
  std::vector<mlir::AffineForOp> res;
  funcOp->walk([&](mlir::Operation* op) {
    if (op->kind == OpKind::For) res.emplace_back(op);
  });
  return res;
}

std::vector<mlir::func::CallOp> Analyzer::collectFuncCalls(mlir::ModuleOp& module) {
  std::vector<mlir::func::CallOp> res;
  for (mlir::Operation* op : module.getBody()->getOperations())
    if (op->kind == OpKind::Call) res.emplace_back(op);
  return res;
}

mlir::func::FuncOp Analyzer::getTargetFunction(mlir::ModuleOp& module, const std::string& targetFuncName) {
  for (mlir::Operation* op : module.getBody()->getOperations())
    if (op->kind == OpKind::Func && op->name == targetFuncName) return mlir::func::FuncOp(op);
  return mlir::func::FuncOp();
}

int Analyzer::getUsersNumber(mlir::ModuleOp& module, mlir::Value value) {
  return static_cast<int>(kcgir::usersOf(module.getOperation(), value).size());
}

mlir::Operation* Analyzer::getLastOp(mlir::Block* body, kcgir::OpKind kind) {
  mlir::Operation* res = nullptr;
  for (mlir::Operation* op : body->getOperations())
    if (op->kind == kind) res = op;
  return res;
}

}  // namespace KernelCodeGen
