// Host-side description of one dense-layer forward or backward call, independent of which public
// surface (C ABI, C++ operator API) it came through, and the two functions that route it to kernels.
#pragma once
#include <cuda_runtime.h>

#include "ge2_internal.hpp"

namespace ge2b {

struct DenseForward {
  int M = 0, N = 0, K = 0, batch = 1;
  int dtype = kF32, z_dtype = kF32;
  int math = 0;                         // fp32 tensors: 0 exact FMA, 1 TF32 tensor cores
  bool trans_a = false;                 // A given as [K,M]
  bool trans_b = false;                 // B given as [N,K]
  const void* A = nullptr; long long lda = 0, strideA = 0;
  const void* B = nullptr; long long ldb = 0, strideB = 0;
  const void* C = nullptr; long long ldc = 0, strideC = 0;
  void* D = nullptr;       long long ldd = 0, strideD = 0;
  void* Z = nullptr;       long long ldz = 0, strideZ = 0;   // null: no stash
  const float* bias = nullptr; int bias_kind = kBiasNone;
  int act = kActNone; float leaky = 0.01f;
  float alpha = 1.f, beta = 0.f;
};

struct DenseBackward {
  int M = 0, N = 0, K = 0;
  int dtype = kF32, z_dtype = kF32;
  int math = 0;
  const void* A = nullptr; long long lda = 0;
  const void* B = nullptr; long long ldb = 0;
  const void* C = nullptr; long long ldc = 0;
  const void* gY = nullptr; long long ldgY = 0;
  const void* Z = nullptr;  long long ldZ = 0;
  void* gA = nullptr; long long ldgA = 0;
  void* gB = nullptr; long long ldgB = 0;
  void* gC = nullptr; long long ldgC = 0;
  float* gBias = nullptr; int bias_kind = kBiasNone;
  int act = kActNone; float leaky = 0.01f;
  float alpha = 1.f, beta = 0.f;
  void* scratch = nullptr; size_t scratch_bytes = 0;   // gZ; null: stream-ordered allocation
  bool reuse_gz = false;   // scratch already holds gZ of this (gY, Z): skip the prologue (and leave gC / gBias alone)
};

enum : int { kOk = 0, kBadArgs = -1, kCudaError = -2, kUnimplemented = -99 };

// Which kernel family a call was routed to (for tests and launch counting).
enum : int { kRouteNone = 0, kRouteSimt = 1, kRouteTensor = 2 };
int last_route();                 // thread-local: route of the most recent GEMM launch of this thread
long long launches_total();       // process-wide count of kernels launched by this library
void note_tensor_launch(int kernels);   // a tensor-core kernel outside run_gemm (the implicit convolution) was launched

int dense_forward(const DenseForward& f, cudaStream_t s);
// Routes a fully described problem (used by the convolution, which needs the batch-reducing form).  A problem with
// reduce_batch that the tensor-core path cannot take (exact fp32, unaligned pitch) returns kUnimplemented.
int run_gemm_problem(const GemmProblem& g, cudaStream_t s);
int dense_backward(const DenseBackward& b, cudaStream_t s);

// One tensor of a multi-tensor SGD launch: fp32 master `p`, gradient `g` of `g_dtype`, optional low-precision copy.
struct SgdTensor {
  float* p; const void* g; void* low; long long n; int g_dtype; int low_dtype;
};
constexpr int kSgdMaxTensors = 16;

// fp32 tensors default to exact arithmetic; GE2B_FP32_MATH=tf32 in the environment opts the operator API
// (which has no field for it) into TF32 tensor cores.
int default_fp32_math();

}  // namespace ge2b
