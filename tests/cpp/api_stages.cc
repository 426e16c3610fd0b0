// Drives the operator API stage by stage and prints the IR after every schedule primitive, for
// tests/test_cpp_api.py to compare with the loop structures documented in the reference's
// README.md:7-190 (problem 4096 x 2048 x 1024, tiles 128 / 8, k-slab 8).
#include <cassert>
#include <iostream>
#include <string>
#include <vector>

#include "KernelCodeGen.h"
using namespace KernelCodeGen;

static void stage(const char* name, mlir::ModuleOp m) {
  std::string why;
  if (!kcgir::verify(m, &why)) {
    std::cout << "VERIFY-FAILED " << name << ": " << why << "\n";
    std::exit(2);
  }
  std::cout << "=== " << name << "\n" << m.str();
}

int main() {
  KernelCodeGenerator generator("CUDA");
  generator.setLogMode(Log::Release);

  // ---- manual schedule of the matmul nest ------------------------------------------------------
  {
    auto graph = generator.createGraph("fuse_matmul_relu");
    int64_t m = 4096, n = 2048, k = 1024;
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"float32"});
    auto C = graph.create<Matmul>(A, B, MemorySpace::global);
    (void)C;
    stage("naive", graph.module);
    auto func = Analyzer::getTargetFunction(graph.module, "Matmul_m4096n2048k1024");
    assert(func);
    auto loops = Analyzer::collectFuncLoops(func);
    assert(loops.size() == 3);
    auto m_axes = Rewriter::split(loops[0], 3, {8, 128});
    auto n_axes = Rewriter::split(loops[1], 3, {8, 128});
    stage("split", graph.module);
    Rewriter::reorder({m_axes[0], n_axes[0], m_axes[1], n_axes[1], m_axes[2], n_axes[2]});
    stage("reorder", graph.module);
    auto grid = Rewriter::parallel({m_axes[0], n_axes[0]});
    auto block = Rewriter::parallel({m_axes[1], n_axes[1]});
    stage("parallel", graph.module);
    int64_t total = 0;
    auto gd = Analyzer::getParallelNumber(grid, total);
    std::cout << "grid " << gd[0] << " " << gd[1] << " total " << total << "\n";
    auto bd = Analyzer::getParallelNumber(block, total);
    std::cout << "block " << bd[0] << " " << bd[1] << " total " << total << "\n";
    std::vector<mlir::AffineForOp> kmn{loops[2], m_axes[2], n_axes[2]};
    auto tileC = Rewriter::bufferizeLoopCarryVar(kmn);
    std::cout << "tileC " << tileC.getType().str() << "\n";
    stage("bufferize", graph.module);
    Rewriter::reorder({loops[2], m_axes[2], n_axes[2]});
    stage("reorder_k", graph.module);
    auto k_axes = Rewriter::split(loops[2], 2, {8});
    assert(k_axes.size() == 2);
    stage("split_k", graph.module);
  }

  // ---- the same through optimize(): schedule + ReLU fusion + dispatch text -----------------------
  {
    auto graph = generator.createGraph("matmul_demo");
    int m = 4096, n = 2048, k = 1024;
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"float32"});
    auto C = graph.create<Matmul>(A, B, MemorySpace::global);
    auto D = graph.create<Relu>(C, MemorySpace::inplace);
    (void)D;
    stage("graph_matmul_relu", graph.module);
    auto module = generator.optimize(graph);
    stage("optimized_matmul_relu", module);
    std::cout << "=== codegen_matmul_relu\n" << generator.codegen(module);
    auto plans = planLaunches(module);
    std::cout << "plans " << plans.size() << " status " << plans[0].status << " epilogue " << plans[0].gemm.epilogue
              << " buffers " << plans[0].buffers[0] << plans[0].buffers[1] << plans[0].buffers[2] << " ws "
              << generator.workspaceBytes(module) << "\n";
  }

  // ---- attention chain -> fused function -------------------------------------------------------
  {
    auto graph = generator.createGraph("flash_attn_demo");
    std::vector<int64_t> shape{8, 32, 2048, 64};
    auto Q = graph.create<PlaceHolder>(shape, std::string{"float32"});
    auto K = graph.create<PlaceHolder>(shape, std::string{"float32"});
    auto V = graph.create<PlaceHolder>(shape, std::string{"float32"});
    auto S = graph.create<BatchedMatmul>(Q, Layout::rowMajor, K, Layout::colMajor);
    auto P = graph.create<Softmax>(S, -1, MemorySpace::inplace);
    auto O = graph.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor);
    (void)O;
    stage("graph_fmha", graph.module);
    auto module = generator.optimize(graph);
    stage("optimized_fmha", module);
    std::cout << "=== codegen_fmha\n" << generator.codegen(module);
    auto plans = planLaunches(module);
    std::cout << "plans " << plans.size() << " status " << plans[0].status << " B " << plans[0].fmha.B << " H "
              << plans[0].fmha.H << " S " << plans[0].fmha.Sq << " D " << plans[0].fmha.D << " buffers "
              << plans[0].buffers[0] << plans[0].buffers[1] << plans[0].buffers[2] << plans[0].buffers[3] << "\n";
  }

  // ---- BatchedMatmul / Softmax outside an attention chain: dispatched as library operators ------
  {
    auto graph = generator.createGraph("standalone_ops");
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{3, 256, 64}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{3, 64, 128}, std::string{"float32"});
    auto C = graph.create<BatchedMatmul>(A, Layout::rowMajor, B, Layout::rowMajor);
    auto X = graph.create<PlaceHolder>(std::vector<int64_t>{5, 7, 300}, std::string{"float32"});
    auto Y = graph.create<Softmax>(X, -1, MemorySpace::inplace);
    (void)C;
    (void)Y;
    auto module = generator.optimize(graph);
    stage("standalone_ops", module);
    auto plans = planLaunches(module);
    std::cout << "plans " << plans.size();
    for (auto& p : plans) std::cout << " kind " << static_cast<int>(p.kind) << " status " << p.status;
    std::cout << " batch " << plans[0].batch << " M " << plans[0].gemm.M << " N " << plans[0].gemm.N << " K "
              << plans[0].gemm.K << " rows " << plans[1].rows << " cols " << plans[1].cols << "\n";
    std::cout << "=== codegen_standalone\n" << generator.codegen(module);
  }

  // ---- Transpose: a copy nest, dispatched to the tiled transpose kernel ---------------------------
  {
    auto graph = generator.createGraph("transpose_demo");
    auto X = graph.create<PlaceHolder>(std::vector<int64_t>{6, 300, 520}, std::string{"float32"});
    auto Y = graph.create<Transpose>(X);
    (void)Y;
    auto module = generator.optimize(graph);
    stage("transpose", module);
    auto plans = planLaunches(module);
    std::cout << "plans " << plans.size() << " kind " << static_cast<int>(plans[0].kind) << " status " << plans[0].status
              << " batch " << plans[0].batch << " rows " << plans[0].rows << " cols " << plans[0].cols << " buffers "
              << plans[0].buffers[0] << plans[0].buffers[1] << "\n";
    std::cout << "=== codegen_transpose\n" << generator.codegen(module);
  }

  // ---- error behaviour -------------------------------------------------------------------------
  {
    auto graph = generator.createGraph("errors");
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{64, 32}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{48, 16}, std::string{"float32"});
    auto C = graph.create<Matmul>(A, B, MemorySpace::global);  // K mismatch: message + null value
    std::cout << "=== errors\nmismatch_is_null " << (C ? 0 : 1) << "\n";
    auto X = graph.create<PlaceHolder>(std::vector<int64_t>{64, 32}, std::string{"int8"});
    std::cout << "bad_dtype_is_null " << (X ? 0 : 1) << "\n";
    // an operator nobody schedules is reported, not silently run on some fallback
    auto R = graph.create<Relu>(A, MemorySpace::inplace);
    (void)R;
    auto module = generator.optimize(graph);
    auto plans = planLaunches(module);
    std::cout << "unscheduled_status " << plans[0].status << "\n";
    std::vector<void*> bufs{nullptr};
    std::cout << "launch_status " << generator.launch(module, bufs) << "\n";
  }
  return 0;
}
