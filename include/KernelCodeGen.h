// Entry point of the operator API: build a graph, optimize it, generate (and here also launch)
// code.  Same public members as the reference's KernelCodeGenerator
// (include/KernelCodeGen.h:25-144), hosted on the IR of include/IR/IR.h; `launch` and
// `workspaceBytes` are additions (the reference leaves launching to an external harness).
#pragma once

#include <cfloat>
#include <climits>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "Backend/CUDA.h"
#include "Frontend/Operators.h"
#include "Optimizer/Optimizer.h"
#include "log.h"

namespace KernelCodeGen {

class KernelCodeGenerator {
 public:
  explicit KernelCodeGenerator(const std::string& platform_ = {"CUDA"})
      : context(std::make_shared<mlir::MLIRContext>()), builder(context.get()), graph(builder), platform(platform_) {
    // Both optimizers are registered (the reference's HEAD registers only FMHA,
    // include/KernelCodeGen.h:32-33, leaving the matmul path dormant).
    opts.push_back(std::make_unique<MatmulOptimizer>());
    opts.push_back(std::make_unique<FMHAOptimizer>());
    matmulConfigs = {
        {{"BLOCK_SIZE_M", 128}, {"BLOCK_SIZE_N", 128}, {"BLOCK_SIZE_K", 8}, {"GROUP_SIZE_M", 8},
         {"THREAD_SIZE_M", 8}, {"THREAD_SIZE_N", 8}, {"VECTORIZE_WIDTH", 4}, {"WARP_SIZE", 32},
         {"STAGES", 0}, {"PRECISION", 0}}};
    fmhaConfigs = {
        {{"BLOCK_SIZE", 128}, {"HdxBr", 128 * 64}, {"BrxBc", 128 * 64}, {"WarpX_O", 2}, {"Slice", 8},
         {"BrTileS", 8}, {"BcTileS", 8}, {"BrTileO", 8}, {"HdTileO", 8}, {"Width", 4}, {"WARP_SIZE", 32},
         {"CAUSAL", 0}, {"SCALE_RSQRT_D", 0}}};
  }
  KernelCodeGenerator() = delete;

  // Starts a new module named after the graph (the name becomes the namespace of emitted code).
  ComputeDAG& createGraph(const std::string& graphName) {
    minLatency = FLT_MAX;
    graph.module = mlir::ModuleOp::create(context.get(), graphName);
    graph.builder.setInsertionPointToEnd(graph.module.getBody());
    return graph;
  }

  ComputeDAG& getGraph() { return graph; }

  // Prints and verifies a module (Log::Debug only).
  void dump(mlir::ModuleOp& module, const std::string& info = "") {
    if (KCGLog::level == Log::Release) return;
    std::cerr << "----------------------------------------------------------\n";
    std::cerr << "           " << info << "\n";
    std::cerr << "----------------------------------------------------------\n";
    module.dump();
    std::string why;
    if (!kcgir::verify(module, &why)) {
      std::cerr << "module verification error: " << why << "\n";
      assert(false);
    }
  }

  // Writes `str` to `file`; the file name "terminal" means stdout.
  void save(const std::string& str, const std::string& file) {
    if (file == "terminal") {
      std::cout << str;
      return;
    }
    std::ofstream fileWriter(file.c_str());
    if (!fileWriter.is_open()) {
      std::cerr << "Can't open file \"" << file << "\"\n";
      return;
    }
    fileWriter << str;
  }

  void resetModule(mlir::ModuleOp& module) { module = mlir::ModuleOp(backupModule_.clone()); }
  void backupModule(mlir::ModuleOp& module) { backupModule_ = mlir::ModuleOp(module.clone()); }
  void saveBestModule(mlir::ModuleOp& module) { bestModule = mlir::ModuleOp(module.clone()); }

  // Runs every registered optimizer over every configuration of its knob list on a clone of the
  // graph's module and returns the best scheduled module.
  mlir::ModuleOp& optimize(ComputeDAG& graph_);

  // Cost of a scheduled module; lower is better.  A stub returning 0 in the reference
  // (include/KernelCodeGen.h:119-121).  Here: the measured device time (ms) of the module's
  // launches when a GPU is present, so that several knob configurations really compete; 0 when
  // nothing can be measured (no device), in which case the first applicable configuration wins
  // as in the reference.
  float evaluate(mlir::ModuleOp& module) {
    if (platform != "CUDA") return 0.0f;
    const float ms = timeModule(module);
    return ms > 0.f ? ms : 0.0f;
  }

  // Launcher source for the module (see include/Backend/CUDA.h).
  std::string codegen(mlir::ModuleOp module) {
    if (platform == "CUDA") return CUDAGen(module);
    std::cerr << "KernelCodeGenerator: platform \"" << platform << "\" has no backend (CUDA / sm_100a only)\n";
    return std::string();
  }

  // Bytes of device scratch `launch` needs for this module.
  size_t workspaceBytes(mlir::ModuleOp module) { return KernelCodeGen::workspaceBytes(module); }

  // Runs the module's kernels.  `buffers[i]` = device pointer of the i-th tensor of the graph in
  // creation order (PlaceHolders and operator results alike).
  kcg_status_t launch(mlir::ModuleOp module, const std::vector<void*>& buffers, void* workspace = nullptr,
                      size_t workspaceBytes_ = 0, void* stream = nullptr) {
    if (platform != "CUDA") return KCG_UNSUPPORTED;
    return launchModule(module, buffers, workspace, workspaceBytes_, stream);
  }

  void setLogMode(Log level) { KCGLog::level = level; }

  // Knob lists the optimizers are tried with (one configuration each by default).
  std::vector<std::map<std::string, int>>& matmulConfigList() { return matmulConfigs; }
  std::vector<std::map<std::string, int>>& fmhaConfigList() { return fmhaConfigs; }

 private:
  std::shared_ptr<mlir::MLIRContext> context;
  mlir::OpBuilder builder;
  mlir::ModuleOp backupModule_;
  mlir::ModuleOp bestModule;
  ComputeDAG graph;
  std::string platform;
  float minLatency = FLT_MAX;
  std::vector<std::unique_ptr<Optimizer>> opts;
  std::vector<std::map<std::string, int>> matmulConfigs;
  std::vector<std::map<std::string, int>> fmhaConfigs;
};

}  // namespace KernelCodeGen
