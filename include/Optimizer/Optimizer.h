// Optimizers: recognise an operator (or a chain of operators) in the module and schedule it.
// Same class names, members and knob maps as the reference (include/Optimizer/Optimizer.h:29-123);
// the schedules target the tcgen05 kernels instead of an FFMA register-tiling recipe:
//
//   knob (reference key)            meaning on B200
//   BLOCK_SIZE_M / BLOCK_SIZE_N     CTA output tile = UMMA M x N (M fixed at 128; N 128 or 256)
//   THREAD_SIZE_M / THREAD_SIZE_N   sub-tile a thread drains from TMEM in the epilogue
//   BLOCK_SIZE_K                    k-slab of the loop nest; the kernel's slab is one 128-byte
//                                   swizzle row (32 fp32 / 64 bf16), recorded as TILE_K
//   GROUP_SIZE_M                    row blocks walked before the next column block (L2 reuse)
//   VECTORIZE_WIDTH                 16-byte TMA / epilogue accesses
//   STAGES (new)                    depth of the TMA->UMMA shared-memory ring (0 = as deep as fits)
//   PRECISION (new)                 0 = by dtype (f32 -> 3xTF32, bf16 -> bf16), 1 = single TF32
#pragma once

#include <map>
#include <set>
#include <string>
#include <vector>

#include "Frontend/Operators.h"
#include "IR/IR.h"
#include "Optimizer/Analyzer.h"
#include "Optimizer/Rewriter.h"

// Shape of one batched matmul of the attention chain.
struct BatchMatmulDescriptor {
  int m = 0;
  int n = 0;
  int k = 0;
  bool transA = false;
  bool transB = false;
  std::vector<int> batch;
  void log() const;
};

namespace KernelCodeGen {

struct Optimizer {
  virtual ~Optimizer() = default;
  virtual bool applicable(mlir::ModuleOp& module) = 0;
  // (Spelling kept from the reference.)
  virtual void applyOptimzer(mlir::ModuleOp& module, mlir::OpBuilder& builder) = 0;
  bool operator==(const Optimizer& other) const { return name == other.name; }
  std::string name;
};

struct MatmulOptimizer : Optimizer {
  MatmulOptimizer() { this->name = "Matmul"; }

  bool applicable(mlir::ModuleOp& module) override;
  void applyOptimzer(mlir::ModuleOp& module, mlir::OpBuilder& builder) override;

  void clear() {
    matmuls.clear();
    matmulLoops.clear();
    matmulBuffers.clear();
  }

  std::set<mlir::func::FuncOp, CompareFunc> matmuls;
  // function -> [loopM, loopN, loopK]
  std::map<mlir::func::FuncOp, std::vector<mlir::AffineForOp>, CompareFunc> matmulLoops;
  struct MemoryBuffer {
    mlir::Value A;
    mlir::Value B;
    mlir::Value C;
  };
  std::map<mlir::func::FuncOp, MemoryBuffer, CompareFunc> matmulBuffers;

  static std::map<std::string, int> matmulConfig;
};

struct FMHAOptimizer : Optimizer {
  FMHAOptimizer() { this->name = "FMHA"; }

  bool applicable(mlir::ModuleOp& module) override;
  void applyOptimzer(mlir::ModuleOp& module, mlir::OpBuilder& builder) override;

  void clear() {
    uniqueFuncCalls.clear();
    call2callsMap.clear();
    call2bufferMap.clear();
  }

  std::set<mlir::func::CallOp, CompareFuncCall> uniqueFuncCalls;
  // first batched matmul call -> {softmax call, second batched matmul call}
  std::map<mlir::func::CallOp, std::vector<mlir::func::CallOp>, CompareFuncCall> call2callsMap;
  struct MemoryBuffer {
    mlir::Value Q;
    mlir::Value K;
    mlir::Value S;
    mlir::Value V;
    mlir::Value O;
    BatchMatmulDescriptor matmul1;
    BatchMatmulDescriptor matmul2;
  };
  std::map<mlir::func::CallOp, MemoryBuffer, CompareFuncCall> call2bufferMap;

  // Reference keys (BLOCK_SIZE, HdxBr, BrxBc, ...) plus CAUSAL (0/1) and SCALE_RSQRT_D (0/1:
  // multiply the logits by 1/sqrt(head_dim); 0 = the reference's unscaled graph).
  static std::map<std::string, int> fmhaConfig;
};

}  // namespace KernelCodeGen
