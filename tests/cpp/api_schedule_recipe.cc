// A complete user schedule of the matmul nest written against the reference's Rewriter signatures
// (the SGEMM recipe the reference's MatmulOptimizer applies, src/Optimizer/Optimizer.cc:383-548:
// tiles 128 x 128 x 8, 8 x 8 per thread, 256 threads as 8 warps of 8 x 4 lanes in a 2 x 4 grid,
// float4 accesses, double-buffered shared and register tiles).  The IR is printed after every
// primitive for tests/test_cpp_schedule.py to compare with the stages documented in the
// reference's README.md:189-1607 (problem 4096 x 2048 x 1024).
#include <algorithm>
#include <cassert>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "KernelCodeGen.h"
using namespace KernelCodeGen;

static void stage(const char* name, mlir::ModuleOp m) {
  std::string why;
  if (!kcgir::verify(m, &why)) {
    std::cout << "VERIFY-FAILED " << name << ": " << why << "\n" << m.str();
    std::exit(2);
  }
  std::cout << "=== " << name << "\n" << m.str();
}

namespace {

constexpr int64_t BM = 128, BN = 128, BK = 8, TM = 8, TN = 8, VEC = 4, WARP = 32;
constexpr int64_t TX = BN / TN, TY = BM / TM;        // 16 x 16 threads
constexpr int64_t WARPS_N = 4, WARPS_M = 2;           // warp grid
constexpr int64_t LANES_N = 4, LANES_M = 8;           // lanes inside a warp

// Where thread (ty, tx) sits: linear id, warp, lane
struct ThreadExprs {
  mlir::AffineExpr tid, warp, lane;
};
ThreadExprs threadExprs(mlir::OpBuilder& b) {
  ThreadExprs t;
  t.tid = b.getAffineDimExpr(0) * TX + b.getAffineDimExpr(1);
  t.warp = t.tid.floorDiv(WARP);
  t.lane = t.tid % WARP;
  return t;
}

// global -> registers: the 256 threads cover a BM x BK (BK x BN) slab with float4 loads;
// operands (ty, tx, blockIdx, k0, copy index)
mlir::AffineMap slabLoadA(mlir::OpBuilder& b) {
  auto t = threadExprs(b);
  auto v = t.tid + b.getAffineDimExpr(4) * (TX * TY);
  return mlir::AffineMap::get(5, 0, {v.floorDiv(BK / VEC) + b.getAffineDimExpr(2) * BM, (v % (BK / VEC)) * VEC + b.getAffineDimExpr(3)});
}
mlir::AffineMap slabLoadB(mlir::OpBuilder& b) {      // operands (ty, tx, k0, blockIdx, copy index)
  auto t = threadExprs(b);
  auto v = t.tid + b.getAffineDimExpr(4) * (TX * TY);
  return mlir::AffineMap::get(5, 0, {v.floorDiv(BN / VEC) + b.getAffineDimExpr(2), (v % (BN / VEC)) * VEC + b.getAffineDimExpr(3) * BN});
}
// registers -> shared: A is stored transposed ([BK][BM]), element by element; B row by row
mlir::AffineMap slabStoreA(mlir::OpBuilder& b) {     // operands (ty, tx, copy index, element)
  auto t = threadExprs(b);
  auto v = t.tid + b.getAffineDimExpr(2) * (TX * TY);
  return mlir::AffineMap::get(4, 0, {(v % (BK / VEC)) * VEC + b.getAffineDimExpr(3), v.floorDiv(BK / VEC)});
}
mlir::AffineMap slabStoreB(mlir::OpBuilder& b) {     // operands (ty, tx, copy index)
  auto t = threadExprs(b);
  auto v = t.tid + b.getAffineDimExpr(2) * (TX * TY);
  return mlir::AffineMap::get(3, 0, {v.floorDiv(BN / VEC), (v % (BN / VEC)) * VEC});
}
// shared -> fragments: a lane reads float4 groups strided by the warp grid; operands (ty, tx, k, copy index)
mlir::AffineMap fragLoadA(mlir::OpBuilder& b) {
  auto t = threadExprs(b);
  auto m = t.lane.floorDiv(LANES_N) + (t.warp.floorDiv(WARPS_N) + b.getAffineDimExpr(3) * WARPS_M) * LANES_M;
  return mlir::AffineMap::get(4, 0, {b.getAffineDimExpr(2), m * VEC});
}
mlir::AffineMap fragLoadB(mlir::OpBuilder& b) {
  auto t = threadExprs(b);
  auto n = t.lane % LANES_N + (t.warp % WARPS_N + b.getAffineDimExpr(3) * WARPS_N) * LANES_N;
  return mlir::AffineMap::get(4, 0, {b.getAffineDimExpr(2), n * VEC});
}
mlir::AffineMap identity1(mlir::OpBuilder& b) { return mlir::AffineMap::get(1, 0, {b.getAffineDimExpr(0)}); }
// register tile -> C: the four 4 x 4 quadrants of a thread's 8 x 8 tile go where its fragments came from;
// operands (ty, tx, by, bx, i0, j0, i1, j1)
mlir::AffineMap tileStoreC(mlir::OpBuilder& b) {
  auto t = threadExprs(b);
  auto m = t.lane.floorDiv(LANES_N) + (t.warp.floorDiv(WARPS_N) + b.getAffineDimExpr(4).floorDiv(VEC) * WARPS_M) * LANES_M;
  auto n = t.lane % LANES_N + (t.warp % WARPS_N + b.getAffineDimExpr(5).floorDiv(VEC) * WARPS_N) * LANES_N;
  return mlir::AffineMap::get(8, 0, {b.getAffineDimExpr(2) * BM + m * VEC + b.getAffineDimExpr(6),
                                     b.getAffineDimExpr(3) * BN + n * VEC + b.getAffineDimExpr(7)});
}

}  // namespace

int main() {
  KernelCodeGenerator generator("CUDA");
  generator.setLogMode(Log::Release);
  auto graph = generator.createGraph("fuse_matmul_relu");
  const int64_t M = 4096, N = 2048, K = 1024;
  auto pa = graph.create<PlaceHolder>(std::vector<int64_t>{M, K}, std::string{"float32"});
  auto pb = graph.create<PlaceHolder>(std::vector<int64_t>{K, N}, std::string{"float32"});
  graph.create<Matmul>(pa, pb, MemorySpace::global);
  auto module = graph.module;
  auto func = Analyzer::getTargetFunction(module, "Matmul_m4096n2048k1024");
  assert(func);
  auto& builder = graph.builder;
  func->setAttr(std::string("func.state"), builder.getStringAttr("gpu"));
  mlir::Value A = func.getArgument(0), B = func.getArgument(1), C = func.getArgument(2);
  auto loops = Analyzer::collectFuncLoops(func);
  auto loopM = loops[0], loopN = loops[1], loopK = loops[2];

  auto ms = Rewriter::split(loopM, 3, {TM, BM});
  auto ns = Rewriter::split(loopN, 3, {TN, BN});
  Rewriter::reorder({ms[0], ns[0], ms[1], ns[1], ms[2], ns[2]});
  auto grid = Rewriter::parallel({ms[0], ns[0]});
  auto block = Rewriter::parallel({ms[1], ns[1]});
  std::vector<mlir::AffineForOp> kmn{loopK, ms[2], ns[2]};
  auto tileC = Rewriter::bufferizeLoopCarryVar(kmn);
  loopK = kmn[0];
  auto m_in = kmn[1], n_in = kmn[2];
  Rewriter::reorder({loopK, m_in, n_in});
  auto ks = Rewriter::split(loopK, 2, {BK});
  auto k_out = ks[0], k_in = ks[1];
  stage("split_k", module);

  int64_t threads = 0;
  Analyzer::getParallelNumber(block, threads);
  const int64_t ldgA = BK * BM / threads, ldgB = BK * BN / threads;     // floats per thread and slab: 4
  const int64_t fragAsz = TM, fragBsz = TN;
  auto elem = A.getType().dyn_cast<mlir::MemRefType>().getElementType();
  auto fragB = Rewriter::alloc_buffer(block, MemorySpace::local, {fragBsz}, elem);
  auto fragA = Rewriter::alloc_buffer(block, MemorySpace::local, {fragAsz}, elem);
  auto regB = Rewriter::alloc_buffer(block, MemorySpace::local, {ldgB}, elem);
  auto regA = Rewriter::alloc_buffer(block, MemorySpace::local, {ldgA}, elem);
  auto smB = Rewriter::alloc_buffer(grid, MemorySpace::shared, {BK, BN}, elem);
  auto smA = Rewriter::alloc_buffer(grid, MemorySpace::shared, {BK, BM}, elem);
  stage("alloc_buffer", module);

  auto bid = Rewriter::getParallelIdx(grid);
  auto tid = Rewriter::getParallelIdx(block);
  auto ldA = Rewriter::read(A, regA, slabLoadA(builder), {tid[0], tid[1], bid[0], k_out.getInductionVar()}, VEC, k_out,
                            Position::begin);
  auto ldB = Rewriter::read(B, regB, slabLoadB(builder), {tid[0], tid[1], k_out.getInductionVar(), bid[1]}, VEC, ldA,
                            Position::after);
  stage("read", module);

  auto stA = Rewriter::write(regA, smA, slabStoreA(builder), {tid[0], tid[1]}, VEC, ldB, Position::after);
  auto stB = Rewriter::write(regB, smB, slabStoreB(builder), {tid[0], tid[1]}, VEC, stA, Position::after);
  auto barrierBefore = Rewriter::barrier(ldA, Position::before);
  auto barrierAfter = Rewriter::barrier(stB, Position::after);
  stage("write", module);

  auto lfA = Rewriter::read(smA, fragA, fragLoadA(builder), {tid[0], tid[1], k_in.getInductionVar()}, VEC, k_in,
                            Position::begin);
  auto lfB = Rewriter::read(smB, fragB, fragLoadB(builder), {tid[0], tid[1], k_in.getInductionVar()}, VEC, lfA,
                            Position::after);
  stage("read_frag", module);

  Rewriter::cache_read(k_in, A, fragA, identity1(builder), {m_in.getInductionVar()});
  Rewriter::cache_read(k_in, B, fragB, identity1(builder), {n_in.getInductionVar()});
  stage("cache_read", module);

  auto writeC = Rewriter::get_write(block, C);
  assert(writeC.size() == 1 && writeC[0].size() == 2);
  auto mi = Rewriter::split(writeC[0][0], 2, {VEC});
  auto ni = Rewriter::split(writeC[0][1], 2, {VEC});
  Rewriter::reorder({mi[0], ni[0], mi[1], ni[1]});
  stage("split_write", module);
  Rewriter::cache_write(mi[0], C, tileC, tileStoreC(builder),
                        {tid[0], tid[1], bid[0], bid[1], mi[0].getInductionVar(), ni[0].getInductionVar(),
                         mi[1].getInductionVar(), ni[1].getInductionVar()});
  stage("cache_write", module);

  Rewriter::vectorize(ni[1], VEC);
  stage("vectorize", module);

  auto dblB = Rewriter::pipeline({ldB, stB}, smB, k_out);
  auto dblA = Rewriter::pipeline({ldA, stA}, smA, k_out);
  auto dblFB = Rewriter::pipeline({lfB}, fragB, k_in);
  auto dblFA = Rewriter::pipeline({lfA}, fragA, k_in);
  std::cout << "buffers " << smA.getType().str() << " " << smB.getType().str() << " " << fragA.getType().str() << " "
            << fragB.getType().str() << "\n";
  stage("pipeline", module);

  Rewriter::detach_last_loop(k_in);
  stage("detach_last_loop", module);

  Rewriter::schedule(dblA[0][0], dblB[0][0], Position::before);
  Rewriter::schedule(dblA[0][1], dblB[0][1], Position::before);
  Rewriter::schedule(barrierBefore, dblB[0][1], Position::after);
  Rewriter::schedule(dblB[1][0], dblA[1][0], Position::after);
  Rewriter::schedule(dblA[1][1], dblB[1][1], Position::before);
  Rewriter::schedule(barrierAfter, dblB[1][1], Position::after);
  auto ifOp = dblA[1][1]->getParentOp();
  Rewriter::schedule(ifOp, k_in, Position::after);
  Rewriter::extract_loop(dblFA[0][0], k_out, 0);
  Rewriter::extract_loop(dblFB[0][0], k_out, 0);
  Rewriter::schedule(dblFB[0][0], k_out, Position::end);
  Rewriter::schedule(dblFA[0][0], k_out, Position::end);
  stage("schedule", module);

  Rewriter::change_double_buffer(dblFA[0][0], smA);
  Rewriter::change_double_buffer(dblFB[0][0], smB);
  stage("change_double_buffer", module);

  Rewriter::take_off_true_if(module);
  Rewriter::delete_false_if(module);
  stage("fold_if", module);

  const int64_t threshold = std::max(BK, std::max(TM, TN));
  Rewriter::unroll(module, [&](mlir::AffineForOp f) -> bool {
    if (!f.hasConstantBounds()) return false;
    const int64_t times = (f.getConstantUpperBound() - f.getConstantLowerBound()) / f.getStep();
    return times < std::min<int64_t>(threshold, VEC);
  });
  stage("unroll", module);

  Rewriter::unrollAttribute(module, [&](mlir::AffineForOp f) -> bool {
    if (!f.hasConstantBounds()) return false;
    const int64_t times = (f.getConstantUpperBound() - f.getConstantLowerBound()) / f.getStep();
    return times <= threshold;
  });
  stage("unroll_attribute", module);

  // the module is still a dispatchable matmul: the Backend recognises the function it came from
  {
    mlir::OpBuilder ob(func->getContext());
    ob.setInsertionPointToEnd(func.getBody());
    (void)ob;
  }
  std::cout << "=== done\n";
  return 0;
}
