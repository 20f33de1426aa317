// Exact-fp32 GEMM with the fused dense-layer epilogue, on the CUDA cores.
//
// Every output element is one chain  acc = fmaf(a[m,k], b[k,n], acc)  over k = 0..K-1 in ascending
// order, which is the summation order of the reference's forward kernels
// (backends/cuda/ops/gemm/kernels/regemm_gemm_bias_act.cu:226-252 and :319-355), so for fp32 operands the
// pre-activation Z is bit-identical to the reference's.  The epilogue follows
// backends/cuda/ops/_common/shim/traits.hpp:30-73 (alpha, + beta*C, + bias, stash Z, activation).
//
// It is the parity path for fp32 tensors and the fall-back for operands the TMA path cannot take
// (unaligned base or pitch).  Any operand dtype, either storage order, any pitch, optional batch.
#include <cuda_runtime.h>

#include "epilogue_math.cuh"
#include "ge2_internal.hpp"

namespace ge2b {
namespace {

constexpr int kTM = 128, kTN = 128, kTK = 16;
constexpr int kPad = 4;                 // keeps float4 alignment, spreads banks on transposing stores
constexpr int kThreads = 256;

struct SimtParams {
  int M, N, K;
  const void* A; long long lda, strideA; int a_mn;
  const void* B; long long ldb, strideB; int b_mn;
  int in_dtype;
  EpilogueArgs epi;
};

__device__ __forceinline__ void simt_epilogue(const SimtParams& p, int b, int m, int n, float acc) {
  const EpilogueArgs& e = p.epi;
  float pre = (e.alpha == 1.f) ? acc : e.alpha * acc;
  if (e.C != nullptr && e.beta != 0.f)
    pre = fmaf(e.beta, load_as_f32(e.C, b * e.strideC + static_cast<long long>(m) * e.ldc + n, e.d_dtype), pre);
  if (e.bias != nullptr) {
    if (e.bias_kind == kBiasPerN)        pre += __ldg(e.bias + n);
    else if (e.bias_kind == kBiasPerM)   pre += __ldg(e.bias + m);
    else if (e.bias_kind == kBiasScalar) pre += __ldg(e.bias);
  }
  if (e.Z != nullptr) store_from_f32(e.Z, b * e.strideZ + static_cast<long long>(m) * e.ldz + n, e.z_dtype, pre);
  store_from_f32(e.D, b * e.strideD + static_cast<long long>(m) * e.ldd + n, e.d_dtype, act_fwd_rt(pre, e.act, e.leaky));
}

// One thread per output; used for tiny problems exactly where the reference switches to its
// one-thread-per-output kernel (M*N < 4096 or K < 8, backends/cuda/ops/gemm/launcher.cu:232-239).
__global__ void gemm_simt_small_kernel(const SimtParams p) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int m = blockIdx.y * blockDim.y + threadIdx.y;
  const int b = blockIdx.z;
  if (m >= p.M || n >= p.N) return;
  const long long a0 = static_cast<long long>(b) * p.strideA, b0 = static_cast<long long>(b) * p.strideB;
  float acc = 0.f;
  for (int k = 0; k < p.K; ++k) {
    const float a = load_as_f32(p.A, a0 + (p.a_mn ? static_cast<long long>(k) * p.lda + m
                                                  : static_cast<long long>(m) * p.lda + k), p.in_dtype);
    const float w = load_as_f32(p.B, b0 + (p.b_mn ? static_cast<long long>(k) * p.ldb + n
                                                  : static_cast<long long>(n) * p.ldb + k), p.in_dtype);
    acc = fmaf(a, w, acc);
  }
  simt_epilogue(p, b, m, n, acc);
}

// 128x128 output tile, 16-deep k tiles, 8x8 outputs per thread (two 4-wide strips in each direction).
// kVec: fp32 operands whose base, pitch and extent along the contiguous index are multiples of 4 elements are
// fetched as float4 (a float4 is then entirely inside or outside the matrix); everything else goes element-wise.
// The arithmetic, and so every result bit, is the same in both forms.
template <bool kVec>
__global__ void __launch_bounds__(kThreads)
gemm_simt_tiled_kernel(const SimtParams p) {
  __shared__ __align__(16) float As[2][kTK][kTM + kPad];
  __shared__ __align__(16) float Bs[2][kTK][kTN + kPad];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  const int b = blockIdx.z;
  const long long a0 = static_cast<long long>(b) * p.strideA, b0 = static_cast<long long>(b) * p.strideB;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  // staging registers: 8 elements of A and 8 of B per thread (as 2 float4 each in the vector form)
  float ra[8], rb[8];
  auto fetch = [&](int k0) {
    if constexpr (kVec) {
      const float* A = reinterpret_cast<const float*>(p.A) + a0;
      const float* B = reinterpret_cast<const float*>(p.B) + b0;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int idx = tid + i * kThreads;                    // 512 float4 per operand tile
        float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vb = va;
        if (p.a_mn) { const int k = idx >> 5, m = (idx & 31) * 4;   // [k][m..m+3]
          if (k0 + k < p.K && m0 + m < p.M) va = *reinterpret_cast<const float4*>(A + static_cast<long long>(k0 + k) * p.lda + m0 + m);
        } else      { const int m = idx >> 2, k = (idx & 3) * 4;    // [m][k..k+3]
          if (m0 + m < p.M && k0 + k < p.K) va = *reinterpret_cast<const float4*>(A + static_cast<long long>(m0 + m) * p.lda + k0 + k);
        }
        if (p.b_mn) { const int k = idx >> 5, n = (idx & 31) * 4;
          if (k0 + k < p.K && n0 + n < p.N) vb = *reinterpret_cast<const float4*>(B + static_cast<long long>(k0 + k) * p.ldb + n0 + n);
        } else      { const int n = idx >> 2, k = (idx & 3) * 4;
          if (n0 + n < p.N && k0 + k < p.K) vb = *reinterpret_cast<const float4*>(B + static_cast<long long>(n0 + n) * p.ldb + k0 + k);
        }
        ra[4 * i] = va.x; ra[4 * i + 1] = va.y; ra[4 * i + 2] = va.z; ra[4 * i + 3] = va.w;
        rb[4 * i] = vb.x; rb[4 * i + 1] = vb.y; rb[4 * i + 2] = vb.z; rb[4 * i + 3] = vb.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + i * kThreads;
        int m, k;
        if (p.a_mn) { m = idx & (kTM - 1); k = idx >> 7; } else { k = idx & (kTK - 1); m = idx >> 4; }
        const int gm = m0 + m, gk = k0 + k;
        ra[i] = (gm < p.M && gk < p.K)
                    ? load_as_f32(p.A, a0 + (p.a_mn ? static_cast<long long>(gk) * p.lda + gm
                                                    : static_cast<long long>(gm) * p.lda + gk), p.in_dtype)
                    : 0.f;
        int n, kk;
        if (p.b_mn) { n = idx & (kTN - 1); kk = idx >> 7; } else { kk = idx & (kTK - 1); n = idx >> 4; }
        const int gn = n0 + n, gkb = k0 + kk;
        rb[i] = (gn < p.N && gkb < p.K)
                    ? load_as_f32(p.B, b0 + (p.b_mn ? static_cast<long long>(gkb) * p.ldb + gn
                                                    : static_cast<long long>(gn) * p.ldb + gkb), p.in_dtype)
                    : 0.f;
      }
    }
  };
  auto stash = [&](int buf) {
    if constexpr (kVec) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int idx = tid + i * kThreads;
        if (p.a_mn) { const int k = idx >> 5, m = (idx & 31) * 4;
          *reinterpret_cast<float4*>(&As[buf][k][m]) = make_float4(ra[4 * i], ra[4 * i + 1], ra[4 * i + 2], ra[4 * i + 3]);
        } else      { const int m = idx >> 2, k = (idx & 3) * 4;
#pragma unroll
          for (int t = 0; t < 4; ++t) As[buf][k + t][m] = ra[4 * i + t];
        }
        if (p.b_mn) { const int k = idx >> 5, n = (idx & 31) * 4;
          *reinterpret_cast<float4*>(&Bs[buf][k][n]) = make_float4(rb[4 * i], rb[4 * i + 1], rb[4 * i + 2], rb[4 * i + 3]);
        } else      { const int n = idx >> 2, k = (idx & 3) * 4;
#pragma unroll
          for (int t = 0; t < 4; ++t) Bs[buf][k + t][n] = rb[4 * i + t];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + i * kThreads;
        int m, k;
        if (p.a_mn) { m = idx & (kTM - 1); k = idx >> 7; } else { k = idx & (kTK - 1); m = idx >> 4; }
        As[buf][k][m] = ra[i];
        int n, kk;
        if (p.b_mn) { n = idx & (kTN - 1); kk = idx >> 7; } else { kk = idx & (kTK - 1); n = idx >> 4; }
        Bs[buf][kk][n] = rb[i];
      }
    }
  };

  const int k_tiles = (p.K + kTK - 1) / kTK;
  fetch(0);
  stash(0);
  __syncthreads();
  for (int kt = 0; kt < k_tiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < k_tiles) fetch((kt + 1) * kTK);
#pragma unroll
    for (int k = 0; k < kTK; ++k) {
      const float4 a_lo = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a_hi = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b_lo = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b_hi = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
      const float w[8] = {b_lo.x, b_lo.y, b_lo.z, b_lo.w, b_hi.x, b_hi.y, b_hi.z, b_hi.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    if (kt + 1 < k_tiles) stash(buf ^ 1);
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (n < p.N) simt_epilogue(p, b, m, n, acc[i][j]);
    }
  }
}

}  // namespace

cudaError_t launch_gemm_simt(const GemmProblem& g, cudaStream_t s) {
  if (g.M < 1 || g.N < 1 || g.K < 1 || g.batch < 1) return cudaErrorInvalidValue;
  SimtParams p{};
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.A = g.A; p.lda = g.lda; p.strideA = g.strideA; p.a_mn = g.a_mn ? 1 : 0;
  p.B = g.B; p.ldb = g.ldb; p.strideB = g.strideB; p.b_mn = g.b_mn ? 1 : 0;
  p.in_dtype = g.in_dtype;
  p.epi = g.epi;
  const bool tiny = (static_cast<long long>(g.M) * g.N < 4096) || (g.K < 8);
  if (tiny) {
    dim3 block(16, 16), grid((g.N + 15) / 16, (g.M + 15) / 16, g.batch);
    gemm_simt_small_kernel<<<grid, block, 0, s>>>(p);
  } else {
    dim3 grid((g.N + kTN - 1) / kTN, (g.M + kTM - 1) / kTM, g.batch);
    auto mult4 = [](long long v) { return (v & 3) == 0; };
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    const bool vec = g.in_dtype == kF32 && al16(g.A) && al16(g.B) && mult4(g.lda) && mult4(g.ldb) &&
                     mult4(g.strideA) && mult4(g.strideB) && mult4(g.a_mn ? g.M : g.K) && mult4(g.b_mn ? g.N : g.K);
    if (vec) gemm_simt_tiled_kernel<true><<<grid, kThreads, 0, s>>>(p);
    else     gemm_simt_tiled_kernel<false><<<grid, kThreads, 0, s>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace ge2b
