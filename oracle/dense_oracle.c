/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's dense-layer path, used as the checker in
 * tests/, in __graft_entry__.smoke() and as bench.py's cpu_baseline.  Nothing in the product links or calls it.
 *
 * Parity pin: checked in tests/test_oracle.py against tests/golden/*.npz, which were produced by the
 * reference's own host-compilable epilogue headers (oracle/_ref, built by oracle/Makefile from the mounted
 * reference tree) on the seeds and shapes of the reference's GEMM tests.
 *
 * What it follows:
 *   summation order   one fmaf chain per output, k ascending, fp32
 *                     (backends/cuda/ops/gemm/kernels/regemm_gemm_bias_act.cu:226-252 and :319-355; the plain
 *                     CPU loop the reference keeps as a checker is GPU_test/ge_v2_gemm/gemm_tiled_test.cu:195-207)
 *   epilogue          pre = alpha*acc (skipped when alpha == 1); pre = fmaf(beta, C, pre); pre += bias;
 *                     Z = pre; D = act(pre)            (backends/cuda/ops/_common/shim/traits.hpp:30-73)
 *   activations       backends/cuda/ops/_common/shim/activations.hpp:11-120 (tanh-form GELU, two-branch sigmoid,
 *                     GELU derivative with tanh clamped to +-0.999999, ReLU' = 0 at 0)
 *   bias kinds        None / Scalar / PerM / PerN      (backends/cuda/ops/_common/shim/bias.hpp:33-66)
 *   backward          gZ = gY*act'(Z); gC = beta*gZ; gBias = sum of gZ over rows / columns / all;
 *                     gA = alpha*gZ.B^T; gB = alpha*A^T.gZ
 *                     (backends/cuda/ops/gemm/kernels/regemm_backward.cu:92-130,183-197,265-291)
 * Host libm (expf, tanhf) stands where the device uses __expf / tanhf, so sigmoid/GELU/tanh agree with the
 * device to a few ulp, not bitwise.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_LEAKY = 2, ACT_GELU = 3, ACT_SIGMOID = 4, ACT_TANH = 5 };
enum { BIAS_NONE = 0, BIAS_SCALAR = 1, BIAS_PER_M = 2, BIAS_PER_N = 3 };

static float gelu_inner(float x) {
  const float c = 0.7978845608f, k1 = 0.044715f;
  const float x2 = x * x, x3 = x2 * x;
  return fmaf(c * k1, x3, c * x);
}

static float sigmoid_stable(float x) {
  if (x >= 0.f) { const float z = expf(-x); return 1.f / (1.f + z); }
  const float z = expf(x);
  return z / (1.f + z);
}

float oracle_act(int kind, float x, float leaky) {
  switch (kind) {
    case ACT_RELU:    return x > 0.f ? x : 0.f;
    case ACT_LEAKY:   return x > 0.f ? x : leaky * x;
    case ACT_GELU:    return 0.5f * x * (1.f + tanhf(gelu_inner(x)));
    case ACT_SIGMOID: return sigmoid_stable(x);
    case ACT_TANH:    return tanhf(x);
    default:          return x;
  }
}

float oracle_act_deriv(int kind, float x, float leaky) {
  switch (kind) {
    case ACT_RELU:  return x > 0.f ? 1.f : 0.f;
    case ACT_LEAKY: return x > 0.f ? 1.f : leaky;
    case ACT_GELU: {
      const float c = 0.7978845608f, k1 = 0.044715f;
      const float x2 = x * x;
      float th = tanhf(gelu_inner(x));
      if (th > 0.999999f) th = 0.999999f;
      if (th < -0.999999f) th = -0.999999f;
      const float sech2 = 1.f - th * th;
      const float dt = c * (1.f + 3.f * k1 * x2);
      return 0.5f * (1.f + th) + 0.5f * x * sech2 * dt;
    }
    case ACT_SIGMOID: { const float s = sigmoid_stable(x); return s * (1.f - s); }
    case ACT_TANH:    { const float th = tanhf(x); return 1.f - th * th; }
    default:          return 1.f;
  }
}

static float bias_at(const float* bias, int kind, int m, int n) {
  if (!bias) return 0.f;
  switch (kind) {
    case BIAS_SCALAR: return bias[0];
    case BIAS_PER_M:  return bias[m];
    case BIAS_PER_N:  return bias[n];
    default:          return 0.f;
  }
}

/* Forward.  B is [K,N] row-major, or [N,K] row-major when trans_b != 0.  Z may be NULL.  Rows are
 * independent, so the OpenMP split over rows does not change any result. */
void oracle_dense_forward_f32(const float* A, int lda, const float* B, int ldb, int trans_b,
                              const float* C, int ldc, const float* bias, int bias_kind,
                              float* D, int ldd, float* Z, int ldz,
                              int M, int N, int K, float alpha, float beta, int act, float leaky) {
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
      if (trans_b) {
        for (int k = 0; k < K; ++k) acc = fmaf(A[(size_t)m * lda + k], B[(size_t)n * ldb + k], acc);
      } else {
        for (int k = 0; k < K; ++k) acc = fmaf(A[(size_t)m * lda + k], B[(size_t)k * ldb + n], acc);
      }
      float pre = (alpha == 1.f) ? acc : alpha * acc;
      if (C && beta != 0.f) pre = fmaf(beta, C[(size_t)m * ldc + n], pre);
      if (bias && bias_kind != BIAS_NONE) pre += bias_at(bias, bias_kind, m, n);
      if (Z) Z[(size_t)m * ldz + n] = pre;
      D[(size_t)m * ldd + n] = oracle_act(act, pre, leaky);
    }
  }
}

/* gZ = gY * act'(Z)  (contiguous, ld = N), optional gC = beta*gZ, optional bias gradient.
 * The bias gradient is summed in double and rounded once: the reference sums it with fp32 atomics in an
 * unspecified order, so no fp32 order is "the" reference order. */
void oracle_dense_bwd_prologue_f32(const float* gY, int ldgY, const float* Z, int ldz, float* gZ,
                                   float* gC, int ldgC, float beta, float* gBias, int bias_kind,
                                   int M, int N, int act, float leaky) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const float gz = gY[(size_t)m * ldgY + n] * oracle_act_deriv(act, Z[(size_t)m * ldz + n], leaky);
      gZ[(size_t)m * N + n] = gz;
      if (gC) gC[(size_t)m * ldgC + n] = beta * gz;
    }
  if (!gBias || bias_kind == BIAS_NONE) return;
  if (bias_kind == BIAS_PER_N) {
    for (int n = 0; n < N; ++n) {
      double s = 0.0;
      for (int m = 0; m < M; ++m) s += gZ[(size_t)m * N + n];
      gBias[n] = (float)s;
    }
  } else if (bias_kind == BIAS_PER_M) {
    for (int m = 0; m < M; ++m) {
      double s = 0.0;
      for (int n = 0; n < N; ++n) s += gZ[(size_t)m * N + n];
      gBias[m] = (float)s;
    }
  } else {
    double s = 0.0;
    for (size_t i = 0; i < (size_t)M * N; ++i) s += gZ[i];
    gBias[0] = (float)s;
  }
}

/* gA[M,K] = alpha * gZ[M,N] . B[K,N]^T   and   gB[K,N] = alpha * A[M,K]^T . gZ[M,N], fp32 fmaf chains in
 * ascending order of the reduction index.  Either output may be NULL. */
void oracle_dense_bwd_gemms_f32(const float* A, int lda, const float* B, int ldb, const float* gZ,
                                float* gA, int ldgA, float* gB, int ldgB, int M, int N, int K, float alpha) {
  if (gA) {
    for (int m = 0; m < M; ++m)
      for (int k = 0; k < K; ++k) {
        float acc = 0.f;
        for (int n = 0; n < N; ++n) acc = fmaf(gZ[(size_t)m * N + n], B[(size_t)k * ldb + n], acc);
        gA[(size_t)m * ldgA + k] = (alpha == 1.f) ? acc : alpha * acc;
      }
  }
  if (gB) {
    for (int k = 0; k < K; ++k)
      for (int n = 0; n < N; ++n) {
        float acc = 0.f;
        for (int m = 0; m < M; ++m) acc = fmaf(A[(size_t)m * lda + k], gZ[(size_t)m * N + n], acc);
        gB[(size_t)k * ldgB + n] = (alpha == 1.f) ? acc : alpha * acc;
      }
  }
}

/* Element-wise helpers over arrays (used to check the activation math on its own). */
void oracle_act_array(int kind, const float* x, float* y, size_t n, float leaky) {
  for (size_t i = 0; i < n; ++i) y[i] = oracle_act(kind, x[i], leaky);
}
void oracle_act_deriv_array(int kind, const float* x, float* y, size_t n, float leaky) {
  for (size_t i = 0; i < n; ++i) y[i] = oracle_act_deriv(kind, x[i], leaky);
}
