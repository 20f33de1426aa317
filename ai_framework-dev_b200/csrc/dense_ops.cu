// Routing of dense-layer calls to kernels.
//
// Forward  D = act(alpha*A.B + beta*C + bias) [+ Z]   -- one fused GEMM launch.
// Backward follows the steps of the reference's gemm_bias_act_bwd_f32
// (backends/cuda/ops/gemm/kernels/regemm_backward.cu:151-301): obtain the gZ scratch, zero gC / gBias,
// gZ = gY*act'(Z) with the bias-gradient reduction, gA = alpha*gZ.B^T, gB = alpha*A^T.gZ, free the scratch.
// The two GEMMs read the caller's row-major tensors directly (no transposed copies).
#include "dense_ops.hpp"

#include <atomic>
#include <cstdlib>
#include <cstring>

namespace ge2b {
namespace {

thread_local int t_last_route = kRouteNone;
std::atomic<long long> g_launches{0};

int run_gemm(const GemmProblem& g, cudaStream_t s) {
  const char* why = nullptr;
  const bool want_tc = (g.in_dtype != kF32) || g.math == 1;
  cudaError_t e;
  if (want_tc && gemm_tc_supported(g, &why)) {
    e = launch_gemm_tc(g, s);
    t_last_route = kRouteTensor;
  } else {
    e = launch_gemm_simt(g, s);
    t_last_route = kRouteSimt;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return e == cudaSuccess ? kOk : kCudaError;
}

}  // namespace

int run_gemm_problem(const GemmProblem& g, cudaStream_t s) {
  if (g.reduce_batch && g.batch > 1) {
    const bool want_tc = (g.in_dtype != kF32) || g.math == 1;
    if (!want_tc || !gemm_tc_supported(g, nullptr)) return kUnimplemented;
  }
  return run_gemm(g, s);
}

int last_route() { return t_last_route; }
long long launches_total() { return g_launches.load(std::memory_order_relaxed); }

int default_fp32_math() {
  const char* e = std::getenv("GE2B_FP32_MATH");
  return (e && std::strcmp(e, "tf32") == 0) ? 1 : 0;
}

int dense_forward(const DenseForward& f, cudaStream_t s) {
  NvtxRange range("gemm.fwd");
  if (f.M <= 0 || f.N <= 0 || f.K <= 0 || !f.A || !f.B || !f.D) return kBadArgs;
  if (f.dtype != kF32 && f.dtype != kF16 && f.dtype != kBF16) return kBadArgs;
  const int batch = f.batch < 1 ? 1 : f.batch;
  GemmProblem g{};
  g.M = f.M; g.N = f.N; g.K = f.K; g.batch = batch;
  g.in_dtype = f.dtype; g.math = f.math;
  g.a_mn = f.trans_a; g.b_mn = !f.trans_b;
  g.A = f.A; g.lda = f.lda; g.strideA = batch > 1 ? f.strideA : 0;
  g.B = f.B; g.ldb = f.ldb; g.strideB = batch > 1 ? f.strideB : 0;
  if (g.lda < (f.trans_a ? f.M : f.K) || g.ldb < (f.trans_b ? f.K : f.N) || f.ldd < f.N) return kBadArgs;
  EpilogueArgs& e = g.epi;
  e.D = f.D; e.ldd = f.ldd; e.strideD = batch > 1 ? f.strideD : 0;
  e.Z = f.Z; e.ldz = f.Z ? (f.ldz > 0 ? f.ldz : f.ldd) : 0; e.strideZ = batch > 1 ? f.strideZ : 0;
  e.C = (f.C && f.beta != 0.f) ? f.C : nullptr; e.ldc = f.ldc; e.strideC = batch > 1 ? f.strideC : 0;
  if (e.Z && e.ldz < f.N) return kBadArgs;
  if (e.C && e.ldc < f.N) return kBadArgs;
  e.bias = (f.bias && f.bias_kind != kBiasNone) ? f.bias : nullptr;
  e.bias_kind = e.bias ? f.bias_kind : kBiasNone;
  e.act = f.act; e.leaky = f.leaky;
  e.alpha = f.alpha; e.beta = f.beta;
  e.d_dtype = f.dtype; e.z_dtype = f.z_dtype;
  return run_gemm(g, s);
}

int dense_backward(const DenseBackward& b, cudaStream_t s) {
  NvtxRange range("gemm.bwd");
  if (b.M <= 0 || b.N <= 0 || b.K <= 0 || !b.gY || !b.Z) return kBadArgs;
  if ((b.gA && !b.B) || (b.gB && !b.A)) return kBadArgs;
  if (b.ldgY < b.N || b.ldZ < b.N) return kBadArgs;
  const int esz = dtype_bytes(b.dtype);
  const size_t need = static_cast<size_t>(b.M) * static_cast<size_t>(b.N) * esz;

  if (b.reuse_gz && !b.scratch) return kBadArgs;
  void* gZ = b.scratch;
  bool owned = false;
  if (gZ) {
    if (b.scratch_bytes > 0 && b.scratch_bytes < need) return kBadArgs;
  } else {
    keep_async_pool_cached();
    if (cudaMallocAsync(&gZ, need, s) != cudaSuccess) return kCudaError;
    owned = true;
  }
  auto finish = [&](int rc) {
    if (owned) cudaFreeAsync(gZ, s);
    return rc;
  };

  if (!b.reuse_gz) {
  // gC is zero when there is no C or beta == 0 (regemm_backward.cu:184-189); gBias accumulates from zero.
  const bool fuse_gc = b.gC && b.C && b.beta != 0.f;
  if (b.gC && !fuse_gc) {
    if (b.ldgC == b.N) {
      if (cudaMemsetAsync(b.gC, 0, static_cast<size_t>(b.M) * b.N * esz, s) != cudaSuccess) return finish(kCudaError);
    } else if (cudaMemset2DAsync(b.gC, static_cast<size_t>(b.ldgC) * esz, 0, static_cast<size_t>(b.N) * esz, b.M, s) !=
               cudaSuccess) {
      return finish(kCudaError);
    }
  }
  const bool want_bias = b.gBias && b.bias_kind != kBiasNone;
  if (want_bias) {
    const size_t n = b.bias_kind == kBiasScalar ? 1 : (b.bias_kind == kBiasPerM ? b.M : b.N);
    if (cudaMemsetAsync(b.gBias, 0, n * sizeof(float), s) != cudaSuccess) return finish(kCudaError);
  }

  BwdPrologueArgs pa{};
  pa.M = b.M; pa.N = b.N;
  pa.gY = b.gY; pa.ldgY = b.ldgY; pa.gy_dtype = b.dtype;
  pa.Z = b.Z; pa.ldZ = b.ldZ; pa.z_dtype = b.z_dtype;
  pa.gZ = gZ; pa.ldgZ = b.N; pa.gz_dtype = b.dtype;
  pa.gC = fuse_gc ? b.gC : nullptr; pa.ldgC = b.ldgC; pa.gc_dtype = b.dtype; pa.beta = b.beta;
  pa.gBias = want_bias ? b.gBias : nullptr; pa.bias_kind = want_bias ? b.bias_kind : kBiasNone;
  pa.act = b.act; pa.leaky = b.leaky;
  {
    NvtxRange epi_range("bwd.epilogue");
    if (launch_bwd_prologue(pa, s) != cudaSuccess) return finish(kCudaError);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  }

  auto plain_epilogue = [&](void* D, long long ldd) {
    EpilogueArgs e{};
    e.D = D; e.ldd = ldd; e.alpha = b.alpha; e.beta = 0.f;
    e.act = kActNone; e.bias_kind = kBiasNone; e.d_dtype = b.dtype; e.z_dtype = b.dtype;
    return e;
  };

  NvtxRange gemms_range("bwd.gemms");
  GemmProblem ga{}, gb{};
  if (b.gA) {   // gA[M,K] = alpha * gZ[M,N] . B[K,N]^T : reduction over N, contiguous in both operands
    if (b.ldb < b.N || b.ldgA < b.K) return finish(kBadArgs);
    ga.M = b.M; ga.N = b.K; ga.K = b.N; ga.batch = 1;
    ga.in_dtype = b.dtype; ga.math = b.math;
    ga.a_mn = false; ga.A = gZ;  ga.lda = b.N;
    ga.b_mn = false; ga.B = b.B; ga.ldb = b.ldb;
    ga.epi = plain_epilogue(b.gA, b.ldgA);
  }
  if (b.gB) {   // gB[K,N] = alpha * A[M,K]^T . gZ[M,N] : reduction over M, the outer index of both operands
    if (b.lda < b.K || b.ldgB < b.N) return finish(kBadArgs);
    gb.M = b.K; gb.N = b.N; gb.K = b.M; gb.batch = 1;
    gb.in_dtype = b.dtype; gb.math = b.math;
    gb.a_mn = true; gb.A = b.A; gb.lda = b.lda;
    gb.b_mn = true; gb.B = gZ;  gb.ldb = b.N;
    gb.epi = plain_epilogue(b.gB, b.ldgB);
  }
  // Both gradients wanted on the tensor-core path: one launch walks the tiles of both (see launch_gemm_tc_dual).
  if (b.gA && b.gB && ((b.dtype != kF32) || b.math == 1)) {
    const cudaError_t e = launch_gemm_tc_dual(ga, gb, s);
    if (e == cudaSuccess) {
      t_last_route = kRouteTensor;
      g_launches.fetch_add(1, std::memory_order_relaxed);
      return finish(kOk);
    }
    if (e != cudaErrorNotSupported) return finish(kCudaError);
    cudaGetLastError();
  }
  if (b.gA) {
    const int rc = run_gemm(ga, s);
    if (rc != kOk) return finish(rc);
  }
  if (b.gB) {
    const int rc = run_gemm(gb, s);
    if (rc != kOk) return finish(rc);
  }
  return finish(kOk);
}

}  // namespace ge2b
