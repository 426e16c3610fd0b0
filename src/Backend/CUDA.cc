// Recogniser + dispatcher (see include/Backend/CUDA.h).
#include "Backend/CUDA.h"

#include <cmath>
#include <iomanip>
#include <sstream>

namespace KernelCodeGen {

using kcgir::OpKind;

namespace {

int allocIndex(mlir::ModuleOp& module, mlir::Value v) {
  int i = 0;
  for (mlir::Operation* op : module.getBody()->getOperations()) {
    if (op->kind != OpKind::Alloc) continue;
    if (op->getResult(0) == v) return i;
    ++i;
  }
  return -1;
}

// A call result aliases the buffer the callee returns; follow calls back to an alloc.
mlir::Value underlyingBuffer(mlir::ModuleOp& module, mlir::Value v) {
  for (int guard = 0; guard < 64 && v; ++guard) {
    mlir::Operation* def = v.getDefiningOp();
    if (!def || def->kind == OpKind::Alloc) return v;
    if (def->kind != OpKind::Call) return v;
    // which argument does the callee return?
    mlir::Operation* callee = nullptr;
    for (mlir::Operation* op : module.getBody()->getOperations())
      if (op->kind == OpKind::Func && op->name == def->name) callee = op;
    if (!callee) return v;
    mlir::Operation* ret = nullptr;
    for (mlir::Operation* op : callee->body->getOperations())
      if (op->kind == OpKind::Return) ret = op;
    if (!ret || ret->operands.empty()) return v;
    int argIdx = -1;
    for (size_t i = 0; i < callee->body->args.size(); ++i)
      if (callee->body->getArgument(i) == ret->operands[0]) argIdx = static_cast<int>(i);
    if (argIdx < 0) return v;
    v = def->operands[argIdx];
  }
  return v;
}

int dtypeCode(const std::string& name) {
  if (name == "f32") return KCG_F32;
  if (name == "bf16") return KCG_BF16;
  return -1;
}

}  // namespace

std::vector<LaunchPlan> planLaunches(mlir::ModuleOp& module) {
  std::vector<LaunchPlan> plans;
  for (mlir::Operation* op : module.getBody()->getOperations()) {
    if (op->kind != OpKind::Call) continue;
    mlir::Operation* callee = nullptr;
    for (mlir::Operation* f : module.getBody()->getOperations())
      if (f->kind == OpKind::Func && f->name == op->name) callee = f;
    if (!callee) continue;
    LaunchPlan p;
    p.function = callee->name;
    const std::string kind = callee->getStringAttr("kcg.op");
    const bool is_bmm = callee->name.rfind("BatchMatmul_", 0) == 0 && op->operands.size() == 3;
    const bool is_softmax = callee->name.rfind("Softmax_", 0) == 0 && op->operands.size() == 1;
    const bool is_transpose = callee->name.rfind("Transpose_", 0) == 0 && op->operands.size() == 2;
    if (kind.empty() && is_transpose) {
      for (auto v : op->operands) p.buffers.push_back(allocIndex(module, underlyingBuffer(module, v)));
      const auto t0 = op->operands[0].getType();
      p.kind = LaunchPlan::Kind::Transpose;
      const size_t r = t0.shape.size();
      p.rows = t0.shape[r - 2];
      p.cols = t0.shape[r - 1];
      p.batch = 1;
      for (size_t i = 0; i + 2 < r; ++i) p.batch *= t0.shape[i];
      p.elem_dtype = dtypeCode(kcgir::scalarName(t0.elem));
      if (p.elem_dtype < 0) {
        p.status = KCG_UNSUPPORTED;
        p.why = "element type has no kernel (float32 and bfloat16 do)";
      }
      plans.push_back(p);
      continue;
    }
    if (kind.empty() && (is_bmm || is_softmax)) {
      // library operators: dispatched from the naive nest as it stands
      for (auto v : op->operands) p.buffers.push_back(allocIndex(module, underlyingBuffer(module, v)));
      const auto t0 = op->operands[0].getType();
      const int dt0 = dtypeCode(kcgir::scalarName(t0.elem));
      if (is_softmax) {
        p.kind = LaunchPlan::Kind::Softmax;
        p.cols = t0.shape.back();
        p.rows = 1;
        for (size_t i = 0; i + 1 < t0.shape.size(); ++i) p.rows *= t0.shape[i];
        if (dt0 != KCG_F32) {
          p.status = KCG_UNSUPPORTED;
          p.why = "standalone Softmax is float32 only";
        }
      } else {
        p.kind = LaunchPlan::Kind::BatchedGemm;
        const auto tA = op->operands[0].getType(), tB = op->operands[1].getType(), tC = op->operands[2].getType();
        const std::string& nm = callee->name;
        const bool transA = nm[nm.size() - 2] == 'T', transB = nm[nm.size() - 1] == 'T';
        const size_t r = tC.shape.size();
        auto& d = p.gemm;
        d.M = tC.shape[r - 2];
        d.N = tC.shape[r - 1];
        d.K = tA.shape[r - 1];
        d.lda = d.K;
        d.ldb = transB ? d.K : d.N;
        d.ldc = d.N;
        d.dtype_in = d.dtype_out = dt0;
        d.precision = dt0 == KCG_BF16 ? KCG_PREC_BF16 : KCG_PREC_3XTF32;
        d.b_layout = transB ? KCG_COL_MAJOR : KCG_ROW_MAJOR;
        p.batch = 1;
        for (size_t i = 0; i + 2 < r; ++i) p.batch *= tC.shape[i];
        p.strideA = d.M * d.K;
        p.strideB = d.K * d.N;
        p.strideC = d.M * d.N;
        (void)tB;
        if (transA) {
          p.status = KCG_UNSUPPORTED;
          p.why = "BatchedMatmul with a colMajor A operand has no kernel";
        } else if (dt0 < 0) {
          p.status = KCG_UNSUPPORTED;
          p.why = "element type has no kernel (float32 and bfloat16 do)";
        }
      }
      plans.push_back(p);
      continue;
    }
    if (callee->getStringAttr("func.state") != "gpu" || kind.empty()) {
      p.status = KCG_UNSUPPORTED;
      p.why = "function @" + callee->name + " has not been scheduled for the GPU (no generic code generator)";
      plans.push_back(p);
      continue;
    }
    for (auto v : op->operands) p.buffers.push_back(allocIndex(module, underlyingBuffer(module, v)));
    const int dt = dtypeCode(callee->getStringAttr("kcg.dtype"));
    if (dt < 0) {
      p.status = KCG_UNSUPPORTED;
      p.why = "element type " + callee->getStringAttr("kcg.dtype") + " has no kernel (float32 and bfloat16 do)";
    }
    if (kind == "matmul") {
      p.kind = LaunchPlan::Kind::Gemm;
      auto& d = p.gemm;
      d.M = callee->getIntAttr("kcg.M");
      d.N = callee->getIntAttr("kcg.N");
      d.K = callee->getIntAttr("kcg.K");
      d.lda = d.K;
      d.ldb = d.N;
      d.ldc = d.N;
      d.dtype_in = d.dtype_out = dt;
      const int64_t prec = callee->getIntAttr("kcg.precision");
      d.precision = dt == KCG_BF16 ? KCG_PREC_BF16 : (prec == 1 ? KCG_PREC_TF32 : KCG_PREC_3XTF32);
      d.epilogue = callee->getStringAttr("kcg.epilogue") == "relu" ? KCG_EPI_RELU : KCG_EPI_NONE;
      d.b_layout = KCG_ROW_MAJOR;
      d.tile_n = static_cast<int32_t>(callee->getIntAttr("kcg.tile_n"));
      d.stages = static_cast<int32_t>(callee->getIntAttr("kcg.stages"));
      d.group_m = static_cast<int32_t>(callee->getIntAttr("kcg.group_m"));
      if (callee->getIntAttr("kcg.tile_m") != 128) {
        p.status = KCG_UNSUPPORTED;
        p.why = "BLOCK_SIZE_M must be 128 (one UMMA M)";
      } else if (d.tile_n != 128 && d.tile_n != 256) {
        p.status = KCG_UNSUPPORTED;
        p.why = "BLOCK_SIZE_N must be 128 or 256";
      }
    } else if (kind == "fmha") {
      p.kind = LaunchPlan::Kind::Fmha;
      auto& d = p.fmha;
      d.B = static_cast<int32_t>(callee->getIntAttr("kcg.batch"));
      d.H = static_cast<int32_t>(callee->getIntAttr("kcg.heads"));
      d.Sq = static_cast<int32_t>(callee->getIntAttr("kcg.seq_q"));
      d.Skv = static_cast<int32_t>(callee->getIntAttr("kcg.seq_kv"));
      d.D = static_cast<int32_t>(callee->getIntAttr("kcg.head_dim"));
      d.dtype_in = d.dtype_out = dt;
      d.causal = static_cast<int32_t>(callee->getIntAttr("kcg.causal"));
      d.scale = callee->getIntAttr("kcg.scale_rsqrt_d") ? 1.0f / std::sqrt(static_cast<float>(d.D)) : 1.0f;
      if (d.D != 64 && d.D != 128) {
        p.status = KCG_UNSUPPORTED;
        p.why = "head dim must be 64 or 128";
      }
    } else {
      p.status = KCG_UNSUPPORTED;
      p.why = "unknown operator kind " + kind;
    }
    plans.push_back(p);
  }
  return plans;
}

size_t workspaceBytes(mlir::ModuleOp& module) {
  size_t need = 0;
  for (auto& p : planLaunches(module)) {
    if (p.status != KCG_OK) continue;
    size_t n = 0;
    if (p.kind == LaunchPlan::Kind::Gemm) n = kcg_gemm_workspace_bytes(&p.gemm);
    else if (p.kind == LaunchPlan::Kind::BatchedGemm) n = kcg_batched_gemm_workspace_bytes(&p.gemm, p.batch, p.strideA, p.strideB);
    else if (p.kind == LaunchPlan::Kind::Fmha) n = kcg_fmha_workspace_bytes(&p.fmha);
    need = n > need ? n : need;
  }
  return need;
}

kcg_status_t launchModule(mlir::ModuleOp& module, const std::vector<void*>& buffers, void* workspace, size_t wsBytes,
                          void* stream) {
  for (auto& p : planLaunches(module)) {
    if (p.status != KCG_OK) return p.status;
    std::vector<void*> ptr;
    for (int idx : p.buffers) {
      if (idx < 0 || idx >= static_cast<int>(buffers.size()) || !buffers[idx]) return KCG_BAD_ARGUMENT;
      ptr.push_back(buffers[idx]);
    }
    kcg_status_t st;
    if (p.kind == LaunchPlan::Kind::Gemm) {
      if (ptr.size() != 3) return KCG_BAD_ARGUMENT;
      st = kcg_gemm_launch(&p.gemm, ptr[0], ptr[1], ptr[2], workspace, wsBytes, stream);
    } else if (p.kind == LaunchPlan::Kind::BatchedGemm) {
      if (ptr.size() != 3) return KCG_BAD_ARGUMENT;
      st = kcg_batched_gemm_launch(&p.gemm, p.batch, p.strideA, p.strideB, p.strideC, ptr[0], ptr[1], ptr[2], workspace,
                                   wsBytes, stream);
    } else if (p.kind == LaunchPlan::Kind::Softmax) {
      if (ptr.size() != 1) return KCG_BAD_ARGUMENT;
      st = kcg_softmax_launch(p.rows, p.cols, ptr[0], ptr[0], stream);
    } else if (p.kind == LaunchPlan::Kind::Transpose) {
      if (ptr.size() != 2) return KCG_BAD_ARGUMENT;
      st = kcg_transpose_launch(p.batch, p.rows, p.cols, p.elem_dtype, ptr[0], ptr[1], stream);
    } else {
      if (ptr.size() != 4) return KCG_BAD_ARGUMENT;
      st = kcg_fmha_fwd_launch(&p.fmha, ptr[0], ptr[1], ptr[2], ptr[3], workspace, wsBytes, stream);
    }
    if (st != KCG_OK) return st;
  }
  return KCG_OK;
}

float timeModule(mlir::ModuleOp& module, int iters) {
  float total = 0.f;
  bool any = false;
  for (auto& p : planLaunches(module)) {
    if (p.status != KCG_OK) return -1.f;
    float ms = 0.f;
    if (p.kind != LaunchPlan::Kind::Gemm && p.kind != LaunchPlan::Kind::Fmha) continue;  // fixed-cost library ops
    const kcg_status_t st = p.kind == LaunchPlan::Kind::Gemm ? kcg_gemm_time(&p.gemm, iters, &ms)
                                                             : kcg_fmha_time(&p.fmha, iters, &ms);
    if (st != KCG_OK) return -1.f;
    total += ms;
    any = true;
  }
  return any ? total : -1.f;
}

std::string CUDAGen(mlir::ModuleOp& module) {
  std::ostringstream os;
  os << "// Launcher for graph @" << module.getName() << ": the kernels are the hand-written sm_100a kernels of\n"
     << "// libkcg_b200 (tcgen05 + TMEM + TMA); this file only fills their descriptors.\n"
     << "#include \"cuda_runtime.h\"\n#include \"kcg_capi.h\"\n"
     << "namespace " << module.getName() << " {\n";
  int kid = 0;
  for (auto& p : planLaunches(module)) {
    os << "\n// func.call @" << p.function << "\n";
    if (p.status != KCG_OK) {
      os << "// not dispatched: " << p.why << "\n";
      continue;
    }
    if (p.kind == LaunchPlan::Kind::Softmax) {
      os << "inline kcg_status_t kernel" << kid << "(float* X, void*, size_t, cudaStream_t stream) {\n"
         << "  return kcg_softmax_launch(" << p.rows << ", " << p.cols << ", X, X, stream);\n}\n";
      ++kid;
      continue;
    }
    if (p.kind == LaunchPlan::Kind::Transpose) {
      const char* ct = p.elem_dtype == KCG_BF16 ? "void" : "float";
      os << "inline kcg_status_t kernel" << kid << "(const " << ct << "* X, " << ct
         << "* Y, void*, size_t, cudaStream_t stream) {\n"
         << "  return kcg_transpose_launch(" << p.batch << ", " << p.rows << ", " << p.cols << ", " << p.elem_dtype
         << ", X, Y, stream);\n}\n";
      ++kid;
      continue;
    }
    if (p.kind == LaunchPlan::Kind::BatchedGemm) {
      const auto& d = p.gemm;
      const char* ct = d.dtype_in == KCG_BF16 ? "void" : "float";
      os << "inline kcg_status_t kernel" << kid << "(const " << ct << "* A, const " << ct << "* B, " << ct
         << "* C, void* workspace, size_t workspace_bytes, cudaStream_t stream) {\n"
         << "  kcg_gemm_desc d = {};\n"
         << "  d.M = " << d.M << "; d.N = " << d.N << "; d.K = " << d.K << ";\n"
         << "  d.lda = " << d.lda << "; d.ldb = " << d.ldb << "; d.ldc = " << d.ldc << ";\n"
         << "  d.dtype_in = " << d.dtype_in << "; d.dtype_out = " << d.dtype_out << "; d.precision = " << d.precision
         << "; d.b_layout = " << d.b_layout << ";\n"
         << "  return kcg_batched_gemm_launch(&d, " << p.batch << ", " << p.strideA << ", " << p.strideB << ", "
         << p.strideC << ", A, B, C, workspace, workspace_bytes, stream);\n}\n";
      ++kid;
      continue;
    }
    if (p.kind == LaunchPlan::Kind::Gemm) {
      const auto& d = p.gemm;
      const char* ct = d.dtype_in == KCG_BF16 ? "void" : "float";
      int32_t geo[6] = {0, 0, 0, 0, 0, 0};
      if (kcg_gemm_launch_geometry(&d, geo) == KCG_OK)
        os << "// grid dims:(" << geo[0] << ", ), block dims:(" << geo[1] << ", )  cluster " << geo[2] << ", tile " << geo[3]
           << "x" << geo[4] << ", " << geo[5] << " tiles, persistent (on 148 SMs)\n";
      os << "inline kcg_status_t kernel" << kid << "(const " << ct << "* A, const " << ct << "* B, " << ct
         << "* C, void* workspace, size_t workspace_bytes, cudaStream_t stream) {\n"
         << "  kcg_gemm_desc d = {};\n"
         << "  d.M = " << d.M << "; d.N = " << d.N << "; d.K = " << d.K << ";\n"
         << "  d.lda = " << d.lda << "; d.ldb = " << d.ldb << "; d.ldc = " << d.ldc << ";\n"
         << "  d.dtype_in = " << d.dtype_in << "; d.dtype_out = " << d.dtype_out << ";\n"
         << "  d.precision = " << d.precision << ";  // 0 = 3xTF32, 1 = TF32, 2 = bf16\n"
         << "  d.epilogue = " << d.epilogue << ";   // 1 = fused ReLU\n"
         << "  d.b_layout = " << d.b_layout << "; d.tile_n = " << d.tile_n << "; d.stages = " << d.stages
         << "; d.group_m = " << d.group_m << ";\n"
         << "  return kcg_gemm_launch(&d, A, B, C, workspace, workspace_bytes, stream);\n}\n";
    } else {
      const auto& d = p.fmha;
      const char* ct = d.dtype_in == KCG_BF16 ? "void" : "float";
      int32_t geo[4] = {0, 0, 0, 0};
      if (kcg_fmha_launch_geometry(&d, geo) == KCG_OK)
        os << "// grid dims:(" << geo[0] << ", ), block dims:(" << geo[1] << ", )  " << geo[2] << " queries per CTA, key blocks of "
           << geo[3] << "\n";
      os << "inline kcg_status_t kernel" << kid << "(const " << ct << "* Q, const " << ct << "* K, const " << ct
         << "* V, " << ct << "* O, void* workspace, size_t workspace_bytes, cudaStream_t stream) {\n"
         << "  kcg_fmha_desc d = {};\n"
         << "  d.B = " << d.B << "; d.H = " << d.H << "; d.Sq = " << d.Sq << "; d.Skv = " << d.Skv << "; d.D = " << d.D
         << ";\n"
         << "  d.dtype_in = " << d.dtype_in << "; d.dtype_out = " << d.dtype_out << ";\n"
         << "  d.causal = " << d.causal << "; d.scale = " << std::fixed << std::setprecision(9) << d.scale << "f;\n"
         << "  return kcg_fmha_fwd_launch(&d, Q, K, V, O, workspace, workspace_bytes, stream);\n}\n";
    }
    ++kid;
  }
  os << "\n}  // namespace " << module.getName() << "\n";
  return os.str();
}

}  // namespace KernelCodeGen
