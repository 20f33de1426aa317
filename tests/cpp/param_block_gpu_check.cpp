// GPU check of the C++ layers under the Tensor API: gemm_bias_act_f32 / _f32_ex / _bwd_f32 called with the reference's
// parameter blocks, and ai::ops::gemm_run_ex / gemm_bwd_run through the registry.  The expected values come from a
// plain loop in this file that accumulates with fmaf in ascending k, which is the order the exact-fp32 kernel uses,
// so Z and the ReLU output must match bit for bit; the gradients are compared to 1e-5 relative.
// Prints "ok" or the first failing line; exit code 0 / 1.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "ge2_dispatch.hpp"

namespace shim = ai::cuda::shim;

#define CHECK(cond) do { if (!(cond)) { std::printf("FAILED line %d: %s\n", __LINE__, #cond); return 1; } } while (0)

static float lcg(unsigned& s) { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xffff) / 32768.f - 1.f; }

template <class T> static T* to_dev(const std::vector<T>& h) {
  T* d = nullptr;
  cudaMalloc(&d, h.size() * sizeof(T));
  cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}
static std::vector<float> to_host(const float* d, size_t n) {
  std::vector<float> h(n);
  cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost);
  return h;
}
static bool same_bits(const std::vector<float>& a, const std::vector<float>& b) {
  return a.size() == b.size() && std::memcmp(a.data(), b.data(), a.size() * sizeof(float)) == 0;
}
static bool close(const std::vector<float>& a, const std::vector<float>& b, float rel) {
  double num = 0, den = 0;
  for (size_t i = 0; i < a.size(); ++i) { num += double(a[i] - b[i]) * (a[i] - b[i]); den += double(b[i]) * b[i]; }
  return std::sqrt(num) <= rel * std::sqrt(den) + 1e-12;
}

int main() {
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no CUDA device\n"); return 2; }
  const int M = 67, N = 40, K = 53;
  unsigned seed = 12345u;
  std::vector<float> A(M * K), B(K * N), bias(N), gY(M * N);
  for (auto& v : A) v = lcg(seed);
  for (auto& v : B) v = lcg(seed);
  for (auto& v : bias) v = lcg(seed);
  for (auto& v : gY) v = lcg(seed);

  // expected forward: Z = A.B + bias (ascending-k fmaf), Y = relu(Z)
  std::vector<float> Z(M * N), Y(M * N);
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc = std::fmaf(A[m * K + k], B[k * N + n], acc);
      Z[m * N + n] = acc + bias[n];
      Y[m * N + n] = Z[m * N + n] > 0.f ? Z[m * N + n] : 0.f;
    }
  // expected backward
  std::vector<float> gZ(M * N), gA(M * K, 0.f), gB(K * N, 0.f), gBias(N, 0.f);
  for (int i = 0; i < M * N; ++i) gZ[i] = gY[i] * (Z[i] > 0.f ? 1.f : 0.f);   // keeps the sign of a zero product
  for (int m = 0; m < M; ++m)
    for (int k = 0; k < K; ++k) { double s = 0; for (int n = 0; n < N; ++n) s += double(gZ[m * N + n]) * B[k * N + n]; gA[m * K + k] = float(s); }
  for (int k = 0; k < K; ++k)
    for (int n = 0; n < N; ++n) { double s = 0; for (int m = 0; m < M; ++m) s += double(A[m * K + k]) * gZ[m * N + n]; gB[k * N + n] = float(s); }
  for (int n = 0; n < N; ++n) { double s = 0; for (int m = 0; m < M; ++m) s += gZ[m * N + n]; gBias[n] = float(s); }

  float *dA = to_dev(A), *dB = to_dev(B), *dbias = to_dev(bias), *dgY = to_dev(gY);
  float *dY, *dZ, *dgA, *dgB, *dgBias, *dscratch;
  cudaMalloc(&dY, M * N * 4); cudaMalloc(&dZ, M * N * 4); cudaMalloc(&dgA, M * K * 4); cudaMalloc(&dgB, K * N * 4);
  cudaMalloc(&dgBias, N * 4); cudaMalloc(&dscratch, M * N * 4);

  // ---- parameter-block forward with the Z stash ----
  shim::GemmBiasActParamsEx p{};
  p.M = M; p.N = N; p.K = K; p.A = dA; p.lda = K; p.B = dB; p.ldb = N; p.C = nullptr; p.ldc = 0; p.D = dY; p.ldd = N;
  p.alpha = 1.f; p.beta = 0.f; p.bias = dbias; p.bias_kind = shim::BiasKind::PerN; p.act = shim::ActKind::ReLU;
  p.leaky_slope = 0.01f; p.Z = dZ; p.ldZ = 0; p.save_preact = 1;
  shim::gemm_bias_act_f32_ex(p, nullptr);
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  CHECK(same_bits(to_host(dZ, M * N), Z));
  CHECK(same_bits(to_host(dY, M * N), Y));

  // ---- the block without a stash ----
  cudaMemset(dY, 0, M * N * 4);
  shim::GemmBiasActParams q{};
  q.M = M; q.N = N; q.K = K; q.A = dA; q.lda = K; q.B = dB; q.ldb = N; q.C = nullptr; q.ldc = 0; q.D = dY; q.ldd = N;
  q.alpha = 1.f; q.beta = 0.f; q.bias = dbias; q.bias_kind = shim::BiasKind::PerN; q.act = shim::ActKind::ReLU; q.leaky_slope = 0.01f;
  shim::gemm_bias_act_f32(q, nullptr);
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  CHECK(same_bits(to_host(dY, M * N), Y));

  // ---- parameter-block backward with caller scratch ----
  shim::GemmBiasActBwdParams b{};
  b.M = M; b.N = N; b.K = K; b.A = dA; b.lda = K; b.B = dB; b.ldb = N; b.C = nullptr; b.ldc = 0; b.Z = dZ; b.ldZ = N;
  b.gY = dgY; b.ldgY = N; b.gA = dgA; b.ldgA = K; b.gB = dgB; b.ldgB = N; b.gC = nullptr; b.ldgC = 0; b.gBias = dgBias;
  b.gZ_scratch = dscratch; b.ldgZ = N; b.bias_kind = shim::BiasKind::PerN; b.act = shim::ActKind::ReLU;
  shim::gemm_bias_act_bwd_f32(b, nullptr);
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  CHECK(close(to_host(dgA, M * K), gA, 1e-5f));
  CHECK(close(to_host(dgB, K * N), gB, 1e-5f));
  CHECK(close(to_host(dgBias, N), gBias, 1e-5f));
  CHECK(same_bits(to_host(dscratch, M * N), gZ));
  bool threw = false;
  b.gY = nullptr;
  try { shim::gemm_bias_act_bwd_f32(b, nullptr); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw);

  // ---- registry run layer ----
  ai::register_b200_gemm_kernels();
  cudaMemset(dY, 0, M * N * 4); cudaMemset(dZ, 0, M * N * 4);
  cudaMemset(dgA, 0, M * K * 4); cudaMemset(dgB, 0, K * N * 4); cudaMemset(dgBias, 0, N * 4);
  ai::Tensor tA = shim::make_tensor2d(dA, M, K), tB = shim::make_tensor2d(dB, K, N), tY = shim::make_tensor2d(dY, M, N);
  ai::Tensor tZ = shim::make_tensor2d(dZ, M, N), tgY = shim::make_tensor2d(dgY, M, N);
  ai::Tensor tgA = shim::make_tensor2d(dgA, M, K), tgB = shim::make_tensor2d(dgB, K, N);
  ai::Tensor tbias; tbias.data = dbias; tbias.desc.shape = {N}; tbias.desc.stride = {1};
  ai::Tensor tgBias; tgBias.data = dgBias; tgBias.desc.shape = {N}; tgBias.desc.stride = {1};
  ai::GemmAttrs at{};
  at.act = shim::ActKind::ReLU; at.with_bias = true; at.save_z = true;
  CHECK(ai::ops::gemm_run_ex(tA, tB, &tbias, tY, at, nullptr, &tZ) == 0);
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  CHECK(same_bits(to_host(dZ, M * N), Z));
  CHECK(same_bits(to_host(dY, M * N), Y));
  CHECK(ai::ops::gemm_bwd_run(tA, tB, nullptr, tgY, tZ, &tgA, &tgB, nullptr, &tgBias, at, nullptr) == 0);
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  CHECK(close(to_host(dgA, M * K), gA, 1e-5f));
  CHECK(close(to_host(dgB, K * N), gB, 1e-5f));
  CHECK(close(to_host(dgBias, N), gBias, 1e-5f));
  std::printf("ok\n");
  return 0;
}
