// Frontend graph builder: every operator becomes a `func.func` holding a naive affine loop
// nest plus a `func.call` in the module body, exactly the structure the reference emits
// (include/Frontend/Operators.h:9-102, src/Frontend/Operators.cc) -- re-hosted on the IR of
// include/IR/IR.h.  The nests are what the CPU oracle executes and what the Optimizer
// schedules; the B200 backend recognises the scheduled functions and dispatches them to
// hand-written kernels.
#pragma once

#include <iostream>
#include <string>
#include <utility>
#include <vector>

#include "IR/IR.h"
#include "enum.h"
#include "log.h"

namespace KernelCodeGen {

// Creates (or returns the already existing) function `funcName` at the top of the module.
// (Spelling "Fuction" kept from the reference, src/Frontend/Operators.cc:19-62.)
mlir::func::FuncOp buildFuction(mlir::ModuleOp module, mlir::OpBuilder& builder, const std::string& funcName,
                                const std::vector<mlir::Type>& inputsTypes,
                                const std::vector<mlir::Type>& outputsTypes);

// "float32" | "float64" | "float16" | "bfloat16" -> scalar type ("" / unknown -> none).
mlir::Type getDType(mlir::OpBuilder& builder, const std::string& dtype);
std::string toStr(const mlir::Type& type);

// Holds the module under construction.  Copies share the module (handles).
struct ComputeDAG {
  explicit ComputeDAG(mlir::OpBuilder& builder_) : builder(builder_) {}
  ComputeDAG() = default;

  template <typename OperatorType, typename... Args>
  mlir::Value create(Args&&... args) {
    return OperatorType::build(this, std::forward<Args>(args)...);
  }

  // Prints and verifies the module (Log::Debug only).
  void dump(const std::string& info = "") {
    if (KCGLog::level == Log::Release) return;
    std::cerr << "-----------------------------------------------------------\n";
    std::cerr << "           " << info << "\n";
    std::cerr << "-----------------------------------------------------------\n";
    module.dump();
    std::string why;
    if (!kcgir::verify(module, &why)) {
      std::cerr << "graph verification error: " << why << "\n";
      assert(false);
    }
  }

  mlir::OpBuilder builder;
  mlir::ModuleOp module;
};

template <typename T>
struct Operator {
  template <typename... Args>
  static mlir::Value build(ComputeDAG* graph, Args&&... args) {
    return T::build(graph, std::forward<Args>(args)...);
  }
};

// A tensor handle: memref.alloc of a static shape in global memory.
struct PlaceHolder : Operator<PlaceHolder> {
  static mlir::Value build(ComputeDAG* graph, const std::vector<int64_t>& shapes, const std::string& dtype);
};

// C[m,n] = sum_k A[m,k] * B[k,n]; C is allocated in memory space `ms`.
struct Matmul : Operator<Matmul> {
  static mlir::Value build(ComputeDAG* graph, mlir::Value A, mlir::Value B, MemorySpace ms,
                           const std::string& dtype = {""});
};

// out = max(0, in), elementwise; MemorySpace::inplace writes the input buffer.
struct Relu : Operator<Relu> {
  static mlir::Value build(ComputeDAG* graph, mlir::Value input, MemorySpace ms, const std::string& dtype = {""});
};

// Matmul over the two innermost dimensions, all leading dimensions are batch dimensions.
// Layout::colMajor on B means B is stored [..., n, k] (Q.K^T without a transpose).
struct BatchedMatmul : Operator<BatchedMatmul> {
  static mlir::Value build(ComputeDAG* graph, mlir::Value A, Layout layoutA, mlir::Value B, Layout layoutB,
                           const std::string& dtype = {""});
};

// exp(x) / sum(exp(x)) over the last axis (axis = -1), in place when ms == inplace.
struct Softmax : Operator<Softmax> {
  static mlir::Value build(ComputeDAG* graph, mlir::Value input, int axis = -1,
                           MemorySpace ms = MemorySpace::global, const std::string& dtype = {""});
};

// out[..., j, i] = in[..., i, j] into a new global PlaceHolder.  The reference declares this
// operator (include/Frontend/Operators.h:100-102) with an empty body
// (src/Frontend/Operators.cc:422-423); here it builds the copy nest, and the Backend dispatches
// it to the tiled transpose kernel.
struct Transpose : Operator<Transpose> {
  static mlir::Value build(ComputeDAG* graph, mlir::Value input);
};

}  // namespace KernelCodeGen
