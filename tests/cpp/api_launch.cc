// End-to-end use of the operator API on a GPU: build graph -> optimize -> launch, with device
// buffers from the CUDA runtime.  Writes the results as raw float32 files for
// tests/test_cpp_api.py to compare with the CPU oracle.
#include <cuda_runtime.h>

#include <cstdio>
#include <fstream>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "KernelCodeGen.h"
using namespace KernelCodeGen;

static void writeFile(const std::string& path, const std::vector<float>& v) {
  std::ofstream f(path, std::ios::binary);
  f.write(reinterpret_cast<const char*>(v.data()), static_cast<std::streamsize>(v.size() * sizeof(float)));
}

static std::vector<float> randomVec(size_t n, unsigned seed, bool normal) {
  std::mt19937 rng(seed);
  std::vector<float> v(n);
  if (normal) {
    std::normal_distribution<float> d(0.f, 1.f);
    for (auto& x : v) x = d(rng);
  } else {
    std::uniform_real_distribution<float> d(-1.f, 1.f);
    for (auto& x : v) x = d(rng);
  }
  return v;
}

#define CHECK_CUDA(x)                                                              \
  do {                                                                             \
    cudaError_t e = (x);                                                           \
    if (e != cudaSuccess) {                                                        \
      std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e));          \
      return 3;                                                                    \
    }                                                                              \
  } while (0)

int main(int argc, char** argv) {
  const std::string out = argc > 1 ? argv[1] : ".";
  KernelCodeGenerator generator("CUDA");
  generator.setLogMode(Log::Release);

  // ---- matmul + relu (fp32 contract) -------------------------------------------------------------
  {
    const int m = 512, n = 384, k = 256;
    auto graph = generator.createGraph("matmul_demo");
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"float32"});
    auto C = graph.create<Matmul>(A, B, MemorySpace::global);
    auto D = graph.create<Relu>(C, MemorySpace::inplace);
    (void)D;
    auto module = generator.optimize(graph);
    auto hA = randomVec(size_t(m) * k, 1, false), hB = randomVec(size_t(k) * n, 2, false);
    std::vector<float> hC(size_t(m) * n);
    float *dA, *dB, *dC;
    void* ws = nullptr;
    const size_t wsBytes = generator.workspaceBytes(module);
    CHECK_CUDA(cudaMalloc(&dA, hA.size() * 4));
    CHECK_CUDA(cudaMalloc(&dB, hB.size() * 4));
    CHECK_CUDA(cudaMalloc(&dC, hC.size() * 4));
    CHECK_CUDA(cudaMalloc(&ws, wsBytes ? wsBytes : 16));
    CHECK_CUDA(cudaMemcpy(dA, hA.data(), hA.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dB, hB.data(), hB.size() * 4, cudaMemcpyHostToDevice));
    kcg_status_t st = generator.launch(module, {dA, dB, dC}, ws, wsBytes, nullptr);
    if (st != KCG_OK) {
      std::fprintf(stderr, "launch: %s\n", kcg_status_str(st));
      return 4;
    }
    CHECK_CUDA(cudaMemcpy(hC.data(), dC, hC.size() * 4, cudaMemcpyDeviceToHost));
    if (kcg_last_device_status() != 0) return 5;
    writeFile(out + "/mm_a.bin", hA);
    writeFile(out + "/mm_b.bin", hB);
    writeFile(out + "/mm_c.bin", hC);
    cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaFree(ws);
  }

  // ---- attention chain ---------------------------------------------------------------------------
  {
    const int b = 2, h = 2, s = 256, d = 64;
    auto graph = generator.createGraph("flash_attn_demo");
    std::vector<int64_t> shape{b, h, s, d};
    auto Q = graph.create<PlaceHolder>(shape, std::string{"float32"});
    auto K = graph.create<PlaceHolder>(shape, std::string{"float32"});
    auto V = graph.create<PlaceHolder>(shape, std::string{"float32"});
    auto S = graph.create<BatchedMatmul>(Q, Layout::rowMajor, K, Layout::colMajor);
    auto P = graph.create<Softmax>(S, -1, MemorySpace::inplace);
    auto O = graph.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor);
    (void)O;
    auto module = generator.optimize(graph);
    const size_t n = size_t(b) * h * s * d;
    auto hQ = randomVec(n, 3, true), hK = randomVec(n, 4, true), hV = randomVec(n, 5, true);
    for (auto& x : hQ) x *= 0.35f;  // keep the unscaled logits of the reference graph moderate
    for (auto& x : hK) x *= 0.35f;
    std::vector<float> hO(n);
    float *dQ, *dK, *dV, *dO;
    void* ws = nullptr;
    const size_t wsBytes = generator.workspaceBytes(module);
    CHECK_CUDA(cudaMalloc(&dQ, n * 4));
    CHECK_CUDA(cudaMalloc(&dK, n * 4));
    CHECK_CUDA(cudaMalloc(&dV, n * 4));
    CHECK_CUDA(cudaMalloc(&dO, n * 4));
    CHECK_CUDA(cudaMalloc(&ws, wsBytes ? wsBytes : 16));
    CHECK_CUDA(cudaMemcpy(dQ, hQ.data(), n * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dK, hK.data(), n * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dV, hV.data(), n * 4, cudaMemcpyHostToDevice));
    // tensors in creation order: Q, K, V, S (never materialised: null), O
    kcg_status_t st = generator.launch(module, {dQ, dK, dV, nullptr, dO}, ws, wsBytes, nullptr);
    if (st != KCG_OK) {
      std::fprintf(stderr, "launch: %s\n", kcg_status_str(st));
      return 6;
    }
    CHECK_CUDA(cudaMemcpy(hO.data(), dO, n * 4, cudaMemcpyDeviceToHost));
    if (kcg_last_device_status() != 0) return 7;
    writeFile(out + "/fa_q.bin", hQ);
    writeFile(out + "/fa_k.bin", hK);
    writeFile(out + "/fa_v.bin", hV);
    writeFile(out + "/fa_o.bin", hO);
    cudaFree(dQ); cudaFree(dK); cudaFree(dV); cudaFree(dO); cudaFree(ws);
  }
  // ---- configuration search with a real cost function ---------------------------------------------
  {
    auto graph = generator.createGraph("matmul_search");
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{2048, 1024}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{1024, 2048}, std::string{"float32"});
    auto C = graph.create<Matmul>(A, B, MemorySpace::global);
    (void)C;
    auto wide = generator.matmulConfigList()[0];
    wide["BLOCK_SIZE_N"] = 256;
    generator.matmulConfigList().push_back(wide);   // two candidates: BLOCK_SIZE_N = 128 and 256
    auto module = generator.optimize(graph);
    const float ms = generator.evaluate(module);
    auto plans = planLaunches(module);
    std::cout << "evaluate_ms " << ms << " chosen_tile_n " << plans[0].gemm.tile_n << "\n";
    generator.matmulConfigList().pop_back();
  }
  std::cout << "ok\n";
  return 0;
}
