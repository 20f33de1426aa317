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

// fp32 backward GEMMs (tolerance-checked everywhere; the reference runs them through cuBLAS) default to the
// error-compensated tensor-core mode; GE2B_FP32_BWD=exact keeps them on the CUDA-core kernel.
bool fp32_bwd_compensated() {
  static const bool on = [] { const char* e = std::getenv("GE2B_FP32_BWD"); return !(e && std::strcmp(e, "exact") == 0); }();
  return on;
}

bool stream_is_capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  return cudaStreamIsCapturing(s, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone;
}

// Scratch of the compensated mode (big / small copies of the operands), from the stream-ordered allocator; not
// available while the stream is being captured.
struct AsyncScratch {
  cudaStream_t s; void* p = nullptr;
  AsyncScratch(cudaStream_t st, size_t bytes) : s(st) {
    if (bytes == 0 || scratch_lease().no_alloc || stream_is_capturing(st)) return;   // callers that must not allocate
    keep_async_pool_cached();
    if (cudaMallocAsync(&p, bytes, st) != cudaSuccess) { cudaGetLastError(); p = nullptr; }
  }
  ~AsyncScratch() { if (p) cudaFreeAsync(p, s); }
  AsyncScratch(const AsyncScratch&) = delete;
  AsyncScratch& operator=(const AsyncScratch&) = delete;
};

size_t up256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

bool aligned_for_tc(const void* p, long long ld) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (ld * 4) % 16 == 0; }

int run_gemm(const GemmProblem& g, cudaStream_t s) {
  const char* why = nullptr;
  const bool want_tc = (g.in_dtype != kF32) || g.math == 1 || (g.math == 2 && g.A_small && g.B_small);
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
    const bool want_tc = (g.in_dtype != kF32) || g.math == 1;      // (the compensated mode has no batch-reducing form)
    if (!want_tc || !gemm_tc_supported(g, nullptr)) return kUnimplemented;
  }
  return run_gemm(g, s);
}

int last_route() { return t_last_route; }
void note_tensor_launch(int kernels) {
  t_last_route = kRouteTensor;
  g_launches.fetch_add(kernels, std::memory_order_relaxed);
}
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
  if (f.dtype == kF32 && f.math == 2) {
    // error-compensated fp32 on tensor cores: split both operands (big + small), three TF32 products per k-block
    const size_t a_elems = static_cast<size_t>(f.trans_a ? f.K : f.M) * (f.trans_a ? f.M : f.K);
    const size_t b_elems = static_cast<size_t>(f.trans_b ? f.N : f.K) * (f.trans_b ? f.K : f.N);
    const size_t a_b = up256(a_elems * 4), b_b = up256(b_elems * 4);
    AsyncScratch sc(s, batch == 1 ? 2 * (a_b + b_b) : 0);
    if (batch == 1 && sc.p) {
      unsigned char* base = static_cast<unsigned char*>(sc.p);
      float *Ab = reinterpret_cast<float*>(base), *As = reinterpret_cast<float*>(base + a_b);
      float *Bb = reinterpret_cast<float*>(base + 2 * a_b), *Bs = reinterpret_cast<float*>(base + 2 * a_b + b_b);
      const long long a_rows = f.trans_a ? f.K : f.M, a_cols = f.trans_a ? f.M : f.K;
      const long long b_rows = f.trans_b ? f.N : f.K, b_cols = f.trans_b ? f.K : f.N;
      if (a_cols % 4 == 0 && b_cols % 4 == 0 &&
          launch_split_tf32(static_cast<const float*>(f.A), f.lda, Ab, As, a_rows, a_cols, s) == cudaSuccess &&
          launch_split_tf32(static_cast<const float*>(f.B), f.ldb, Bb, Bs, b_rows, b_cols, s) == cudaSuccess) {
        g_launches.fetch_add(2, std::memory_order_relaxed);
        g.A = Ab; g.lda = a_cols; g.A_small = As;
        g.B = Bb; g.ldb = b_cols; g.B_small = Bs;
        return run_gemm(g, s);
      }
    }
    g.math = 0;          // no scratch (stream capture, batched call, odd pitch): the exact CUDA-core kernel
  }
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
  DbFinish db_pending;          // second half of a deterministic bias gradient, owed after the prologue
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
  const bool want_bias = b.gBias && b.bias_kind != kBiasNone;   // (zeroed by the prologue's launcher where it adds atomically)

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
    if (launch_bwd_prologue(pa, s, &db_pending, true) != cudaSuccess) return finish(kCudaError);
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
  // fp32 without a TF32 opt-in: the two GEMMs run in the error-compensated tensor-core mode when their split operands
  // can be staged (not under stream capture; pitches that TMA can address), else on the exact CUDA-core kernel.
  const bool want_x3 = b.dtype == kF32 && (b.math == 2 || (b.math == 0 && fp32_bwd_compensated())) && b.N % 4 == 0 &&
                       b.K % 4 == 0 && (!b.gA || aligned_for_tc(b.gA, b.ldgA)) && (!b.gB || aligned_for_tc(b.gB, b.ldgB));
  const size_t mn = up256(static_cast<size_t>(b.M) * b.N * 4), kn = up256(static_cast<size_t>(b.K) * b.N * 4),
               mk = up256(static_cast<size_t>(b.M) * b.K * 4);
  AsyncScratch x3(s, want_x3 ? 2 * mn + (b.gA ? 2 * kn : 0) + (b.gB ? 2 * mk : 0) : 0);
  float *gZb = nullptr, *gZs = nullptr, *Wb = nullptr, *Ws = nullptr, *Xb = nullptr, *Xs = nullptr;
  bool use_x3 = false;
  if (want_x3 && x3.p) {
    unsigned char* q = static_cast<unsigned char*>(x3.p);
    SplitItem items[3];
    int n_items = 0;
    gZb = reinterpret_cast<float*>(q); gZs = reinterpret_cast<float*>(q + mn); q += 2 * mn;
    items[n_items++] = SplitItem{static_cast<const float*>(gZ), b.N, gZb, gZs, b.M, b.N};
    if (b.gA) {
      Wb = reinterpret_cast<float*>(q); Ws = reinterpret_cast<float*>(q + kn); q += 2 * kn;
      items[n_items++] = SplitItem{static_cast<const float*>(b.B), b.ldb, Wb, Ws, b.K, b.N};
    }
    if (b.gB) {
      Xb = reinterpret_cast<float*>(q); Xs = reinterpret_cast<float*>(q + mk);
      items[n_items++] = SplitItem{static_cast<const float*>(b.A), b.lda, Xb, Xs, b.M, b.K};
    }
    use_x3 = launch_split_tf32_multi(items, n_items, s) == cudaSuccess;      // one launch for all three
    if (use_x3) g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  const int gemm_math = use_x3 ? 2 : (b.math == 2 ? 0 : b.math);

  GemmProblem ga{}, gb{};
  if (b.gA) {   // gA[M,K] = alpha * gZ[M,N] . B[K,N]^T : reduction over N, contiguous in both operands
    if (b.ldb < b.N || b.ldgA < b.K) return finish(kBadArgs);
    ga.M = b.M; ga.N = b.K; ga.K = b.N; ga.batch = 1;
    ga.in_dtype = b.dtype; ga.math = gemm_math;
    ga.a_mn = false; ga.A = gZ;  ga.lda = b.N;
    ga.b_mn = false; ga.B = b.B; ga.ldb = b.ldb;
    if (use_x3) { ga.A = gZb; ga.A_small = gZs; ga.B = Wb; ga.B_small = Ws; ga.ldb = b.N; }
    ga.epi = plain_epilogue(b.gA, b.ldgA);
  }
  if (b.gB) {   // gB[K,N] = alpha * A[M,K]^T . gZ[M,N] : reduction over M, the outer index of both operands
    if (b.lda < b.K || b.ldgB < b.N) return finish(kBadArgs);
    gb.M = b.K; gb.N = b.N; gb.K = b.M; gb.batch = 1;
    gb.in_dtype = b.dtype; gb.math = gemm_math;
    gb.a_mn = true; gb.A = b.A; gb.lda = b.lda;
    gb.b_mn = true; gb.B = gZ;  gb.ldb = b.N;
    if (use_x3) { gb.A = Xb; gb.A_small = Xs; gb.lda = b.K; gb.B = gZb; gb.B_small = gZs; }
    gb.epi = plain_epilogue(b.gB, b.ldgB);
  }
  // The bias gradient's finish rides with the first GEMM launch that goes to the tensor-core kernel; where none does
  // (exact fp32 kernel, unaligned operands, no GEMM asked for) it runs as its own small kernel.
  if (db_pending.partial != nullptr) {
    auto takes_tc = [](const GemmProblem& g) {
      const bool want = (g.in_dtype != kF32) || g.math == 1 || (g.math == 2 && g.A_small && g.B_small);
      return want && gemm_tc_supported(g, nullptr);
    };
    if (b.gA && takes_tc(ga)) ga.db = db_pending;
    else if (b.gB && takes_tc(gb)) gb.db = db_pending;
    else {
      if (launch_db_finish(db_pending, s) != cudaSuccess) return finish(kCudaError);
      g_launches.fetch_add(1, std::memory_order_relaxed);
    }
  }
  // Both gradients wanted on the tensor-core path: one launch walks the tiles of both (see launch_gemm_tc_dual).
  if (b.gA && b.gB && ((b.dtype != kF32) || gemm_math == 1)) {
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
