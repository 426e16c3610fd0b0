// Backend for B200: recognises scheduled operator functions in a module and dispatches them
// to the hand-written sm_100a kernels through the C-ABI of include/kcg_capi.h.
//
// The reference's Backend prints generic CUDA C from the scheduled affine IR
// (`std::string CUDAGen(mlir::ModuleOp&)`, include/Backend/CUDA.h:6, src/Backend/CUDA.cc:878-890)
// and leaves compiling and launching to an external harness.  CUDAGen keeps its signature: it
// returns a small launcher translation unit -- `namespace <graph> { kernel0(...) }` as before,
// but the body fills a descriptor and calls kcg_gemm_launch / kcg_fmha_fwd_launch -- so that
// `save()` still writes something a harness can compile.  `launchModule` does the same calls
// directly.  BatchedMatmul, Softmax and Transpose functions that are not part of an attention chain are
// dispatched as they stand to the batched GEMM and the row-softmax kernel.  There is
// deliberately no generic affine->CUDA emitter: any other unscheduled function yields
// KCG_UNSUPPORTED, never a fallback kernel.
#pragma once

#include <string>
#include <vector>

#include "IR/IR.h"
#include "kcg_capi.h"

namespace KernelCodeGen {

// One kernel launch derived from a `func.call` of a function with func.state = "gpu".
struct LaunchPlan {
  enum class Kind { Gemm, Fmha, BatchedGemm, Softmax, Transpose } kind = Kind::Gemm;
  std::string function;            // callee symbol
  kcg_gemm_desc gemm{};
  kcg_fmha_desc fmha{};
  // BatchedGemm: `gemm` describes one product; batch count and element strides between products.
  int64_t batch = 1, strideA = 0, strideB = 0, strideC = 0;
  // Softmax: [rows, cols] fp32, in place on its single buffer.  Transpose: `batch` matrices of
  // [rows, cols] elements of `elem_dtype`, buffers (X, Y).
  int64_t rows = 0, cols = 0;
  int elem_dtype = KCG_F32;
  // Position (among the module-level memref.alloc ops, in program order) of each pointer
  // argument, in the kernel's argument order: (A, B, C), (Q, K, V, O), (X) for Softmax or (X, Y) for Transpose.
  std::vector<int> buffers;
  kcg_status_t status = KCG_OK;    // KCG_UNSUPPORTED when the schedule has no kernel
  std::string why;
};

// Launches of the module body, in program order.
std::vector<LaunchPlan> planLaunches(mlir::ModuleOp& module);

// Launcher source text for the module (see above).
std::string CUDAGen(mlir::ModuleOp& module);

// Bytes of scratch the module's launches need (maximum over launches).
size_t workspaceBytes(mlir::ModuleOp& module);

// Sum of the measured device times (ms) of the module's launches, on scratch buffers; negative
// when nothing could be measured (no device, or an unsupported launch).
float timeModule(mlir::ModuleOp& module, int iters = 10);

// Runs every launch of the module on `stream`.  `buffers[i]` is the device pointer of the i-th
// module-level memref.alloc (PlaceHolders and operator outputs, in creation order); entries of
// buffers no kernel touches may be null.
kcg_status_t launchModule(mlir::ModuleOp& module, const std::vector<void*>& buffers, void* workspace,
                          size_t workspaceBytes, void* stream);

}  // namespace KernelCodeGen
