// TEST INFRASTRUCTURE ONLY.  Exposes the reference's OWN epilogue math, compiled for the host through its
// AI_SHIM_TEST_ON_HOST switch (backends/cuda/ops/_common/shim/ai_defs.hpp:28-34), behind a C interface so that
// Python can (a) validate oracle/dense_oracle.c against it and (b) generate tests/golden/*.npz.
// The reference headers are included from the mounted reference tree at build time (see oracle/Makefile);
// nothing of them is copied here.  The GEMM core below is this file's own plain loop in the summation order of
// the reference kernels (one fmaf chain per output, k ascending).
#define AI_SHIM_TEST_ON_HOST 1
#include "backends/cuda/ops/_common/shim/activations.hpp"
#include "backends/cuda/ops/_common/shim/bias.hpp"
#include "backends/cuda/ops/_common/shim/epilogue_functors.hpp"

#include <cmath>
#include <cstddef>

namespace rs = ai::cuda::shim;

extern "C" {

float ref_act_runtime(int kind, float x, float leaky) {
  return rs::apply_act_runtime(x, static_cast<rs::ActKind>(kind), leaky);
}

// Template (compile-time) derivative: the one the reference's backward kernel instantiates.
float ref_act_deriv(int kind, float x, float leaky) {
  switch (static_cast<rs::ActKind>(kind)) {
    case rs::ActKind::ReLU:      return rs::act_deriv<rs::ActKind::ReLU>(x, leaky);
    case rs::ActKind::LeakyReLU: return rs::act_deriv<rs::ActKind::LeakyReLU>(x, leaky);
    case rs::ActKind::GELU:      return rs::act_deriv<rs::ActKind::GELU>(x, leaky);
    case rs::ActKind::Sigmoid:   return rs::act_deriv<rs::ActKind::Sigmoid>(x, leaky);
    case rs::ActKind::Tanh:      return rs::act_deriv<rs::ActKind::Tanh>(x, leaky);
    default:                     return rs::act_deriv<rs::ActKind::None>(x, leaky);
  }
}

// Y = act(alpha*A.B + beta*C + bias) with optional Z stash; epilogue = reference apply_epilogue_scalar.
void ref_dense_forward_f32(const float* A, int lda, const float* B, int ldb, const float* C, int ldc,
                           const float* bias, int bias_kind, float* D, int ldd, float* Z, int ldz,
                           int M, int N, int K, float alpha, float beta, int act, float leaky) {
  rs::EpilogueCtx e;
  e.alpha = alpha; e.beta = beta;
  e.bias = bias; e.bias_kind = static_cast<rs::BiasKind>(bias_kind);
  e.act = static_cast<rs::ActKind>(act); e.leaky_slope = leaky;
  e.C = C; e.ldc = ldc;
  e.Z = Z; e.ldZ = ldz; e.save_preact = Z ? 1 : 0;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc = std::fmaf(A[(std::size_t)m * lda + k], B[(std::size_t)k * ldb + n], acc);
      D[(std::size_t)m * ldd + n] = rs::apply_epilogue_scalar(acc, m, n, M, N, e);
    }
}

// gZ = gY * act'(Z) with the reference's template derivative.
void ref_dense_bwd_gz_f32(const float* gY, int ldgY, const float* Z, int ldz, float* gZ, int M, int N, int act,
                          float leaky) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n)
      gZ[(std::size_t)m * N + n] = gY[(std::size_t)m * ldgY + n] * ref_act_deriv(act, Z[(std::size_t)m * ldz + n], leaky);
}

}  // extern "C"
