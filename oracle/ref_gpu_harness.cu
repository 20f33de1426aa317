// TEST INFRASTRUCTURE ONLY.  C interface over the reference's own GPU operator API
// (backends/cuda/ops/gemm/api.hpp:124-188), linked with the reference's three GEMM sources compiled for
// sm_100a from the mounted reference tree (see oracle/Makefile).  Lets GPU tests and the benchmark run the
// reference kernels on the same device buffers as the new library.  All tensors fp32 row-major, contiguous.
#include "backends/cuda/ops/gemm/api.hpp"

namespace rs = ai::cuda::shim;

static rs::Tensor t2d(const void* p, long long r, long long c) {
  return rs::make_tensor2d(const_cast<void*>(p), r, c, rs::DType::F32);
}

extern "C" {

// bias_len selects the bias shape: 0 none, else a 1-D tensor of that length.  Returns the Status as int.
int ref_gpu_forward(const float* A, const float* B, const float* bias, long long bias_len, float* Y, float* Z,
                    int M, int K, int N, int act, float leaky, void* stream) {
  rs::Tensor tA = t2d(A, M, K), tB = t2d(B, K, N), tY = t2d(Y, M, N), tZ = t2d(Z, M, N), tBias;
  if (bias && bias_len > 0) {
    tBias.data = const_cast<float*>(bias);
    tBias.desc.shape = {bias_len};
    tBias.desc.stride = {1};
  }
  rs::GemmAttrs at;
  at.act = static_cast<rs::ActKind>(act);
  at.with_bias = bias != nullptr;
  at.leaky_slope = leaky;
  at.save_z = Z != nullptr;
  return static_cast<int>(rs::GemmCudaLaunch(tA, tB, bias ? &tBias : nullptr, tY, at,
                                             reinterpret_cast<cudaStream_t>(stream), Z ? &tZ : nullptr, nullptr));
}

int ref_gpu_backward(const float* A, const float* B, const float* gY, const float* Z, float* gA, float* gB,
                     float* gBias, long long bias_len, float* scratch, int M, int K, int N, int act, float leaky,
                     void* stream) {
  rs::Tensor tA = t2d(A, M, K), tB = t2d(B, K, N), tgY = t2d(gY, M, N), tZ = t2d(Z, M, N);
  rs::Tensor tgA = t2d(gA, M, K), tgB = t2d(gB, K, N), tgBias;
  if (gBias && bias_len > 0) {
    tgBias.data = gBias;
    tgBias.desc.shape = {bias_len};
    tgBias.desc.stride = {1};
  }
  rs::GemmAttrs at;
  at.act = static_cast<rs::ActKind>(act);
  at.leaky_slope = leaky;
  rs::GemmWorkspace ws;
  ws.scratch = scratch;
  try {
    return static_cast<int>(rs::GemmCudaBackward(tA, tB, nullptr, tgY, tZ, gA ? &tgA : nullptr, gB ? &tgB : nullptr,
                                                 nullptr, gBias ? &tgBias : nullptr, at,
                                                 reinterpret_cast<cudaStream_t>(stream), scratch ? &ws : nullptr));
  } catch (...) {
    return 3;   // Status::RuntimeError
  }
}

}  // extern "C"
