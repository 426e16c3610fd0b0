// Enumerations of the operator API.  The numeric values of MemorySpace are part of the
// contract: they are the memory-space integers printed in memref types
// (`memref<4096x1024xf32, 1>` = global, `, 3` = local/registers), as in the reference's
// include/enum.h:5-29 and the IR snapshots of its README.md:10,125,239.
#pragma once

namespace KernelCodeGen {

// Code generation target.  Only CUDA (sm_100a) has a backend here.
enum class Target { CUDA = 0, ROCm = 1 };

// Where a buffer lives.  `inplace` is not a space of its own: an operator given it writes its
// input buffer (Relu uses it, which is what makes the ReLU fusable into the GEMM epilogue).
enum class MemorySpace {
  global = 1,       // HBM
  shared = 2,       // shared memory of a CTA
  local = 3,        // per-thread registers (TMEM accumulators on this backend)
  constant = 4,
  unallocated = 5,
  inplace = 6,
};

// Where to put something relative to a loop.
enum class Position { before = 0, after = 1, begin = 2, end = 3 };

// Storage order of the two innermost dimensions of a batched-matmul operand.
enum class Layout { rowMajor = 0, colMajor = 1 };

}  // namespace KernelCodeGen
