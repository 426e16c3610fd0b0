#include "KernelCodeGen.h"

namespace KernelCodeGen {

Log KCGLog::level = Log::Debug;

// Configuration search as in the reference (src/KernelCodeGen.cc:8-53): every optimizer is tried
// with each of its knob maps on a fresh copy of the module; the copy with the lowest evaluate()
// is kept.  Optimizers compose: the next one starts from the best module so far.
mlir::ModuleOp& KernelCodeGenerator::optimize(ComputeDAG& graph_) {
  graph = graph_;
  mlir::ModuleOp module(graph.module.clone());
  saveBestModule(module);
  for (auto& opt : opts) {
    module = mlir::ModuleOp(bestModule.clone());
    backupModule(module);
    minLatency = FLT_MAX;
    std::vector<std::map<std::string, int>> one{{}};
    const bool isFmha = *opt == FMHAOptimizer();
    const bool isMatmul = *opt == MatmulOptimizer();
    auto& configs = isFmha ? fmhaConfigs : (isMatmul ? matmulConfigs : one);
    for (auto& config : configs) {
      if (isFmha) FMHAOptimizer::fmhaConfig = config;
      if (isMatmul) MatmulOptimizer::matmulConfig = config;
      resetModule(module);
      if (!opt->applicable(module)) continue;
      opt->applyOptimzer(module, builder);
      const float latency = evaluate(module);
      if (latency < minLatency) {
        minLatency = latency;
        saveBestModule(module);
      }
    }
  }
  return bestModule;
}

}  // namespace KernelCodeGen
