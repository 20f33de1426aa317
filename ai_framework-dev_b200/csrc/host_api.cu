// Host-buffer plan: one dense-layer forward + backward per call with inputs and results in HOST memory.
//
// Counterpart of the reference's GemmPlan (graph_executor_v2/src/bindings/py_api.cpp:403-523): device buffers
// are allocated once when the plan is created; every step copies the inputs up, launches, and copies the
// results back.  Here a step is pipelined over three streams so that PCIe traffic in both directions overlaps
// the kernels: inputs (X, W, bias, then dY) go up on the copy-in stream; the forward kernel starts as soon as
// X and W are up; Y goes down while the backward runs; dW is computed first and goes down while dX is computed.
// The step returns when all requested results are in host memory.  Pass page-locked host buffers for full
// copy speed; pageable ones work but serialise.
#include <cuda_runtime.h>

#include <new>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"

using namespace ge2b;

struct ge2b_dense_plan {
  int M, K, N, dtype, act, has_bias, math;
  float leaky;
  int device;
  size_t esz;
  void *X, *W, *dY, *Y, *Z, *gZ, *dX, *dW;
  float *bias, *db;
  cudaStream_t s_in, s_compute, s_out;
  cudaEvent_t e_xw, e_dy, e_fwd, e_dw, e_dx;
};

namespace {

bool ok(cudaError_t e) { return e == cudaSuccess; }

void destroy(ge2b_dense_plan* p) {
  if (!p) return;
  void* bufs[] = {p->X, p->W, p->dY, p->Y, p->Z, p->gZ, p->dX, p->dW, p->bias, p->db};
  for (void* b : bufs)
    if (b) cudaFree(b);
  cudaStream_t ss[] = {p->s_in, p->s_compute, p->s_out};
  for (cudaStream_t s : ss)
    if (s) cudaStreamDestroy(s);
  cudaEvent_t es[] = {p->e_xw, p->e_dy, p->e_fwd, p->e_dw, p->e_dx};
  for (cudaEvent_t e : es)
    if (e) cudaEventDestroy(e);
  delete p;
}

}  // namespace

extern "C" {

int ge2b_dense_plan_create(ge2b_dense_plan** out, int M, int K, int N, ge2_dtype_t dtype, ge2_act_kind_t act,
                           float leaky_slope, int has_bias, ge2_math_t math) {
  if (!out || M <= 0 || K <= 0 || N <= 0) return kBadArgs;
  if (dtype != GE2_DT_F32 && dtype != GE2_DT_F16 && dtype != GE2_DT_BF16) return kBadArgs;
  ge2b_dense_plan* p = new (std::nothrow) ge2b_dense_plan();
  if (!p) return kCudaError;
  p->M = M; p->K = K; p->N = N; p->dtype = dtype; p->act = act; p->has_bias = has_bias; p->leaky = leaky_slope;
  p->math = (dtype == GE2_DT_F32) ? (math == GE2_MATH_TENSOR ? 1 : 0) : 1;
  p->esz = dtype_bytes(dtype);
  const size_t mk = (size_t)M * K * p->esz, kn = (size_t)K * N * p->esz, mn = (size_t)M * N * p->esz;
  bool good = ok(cudaGetDevice(&p->device));
  good = good && ok(cudaMalloc(&p->X, mk)) && ok(cudaMalloc(&p->W, kn)) && ok(cudaMalloc(&p->dY, mn)) &&
         ok(cudaMalloc(&p->Y, mn)) && ok(cudaMalloc(&p->Z, mn)) && ok(cudaMalloc(&p->gZ, mn)) &&
         ok(cudaMalloc(&p->dX, mk)) && ok(cudaMalloc(&p->dW, kn)) &&
         ok(cudaMalloc(reinterpret_cast<void**>(&p->bias), (size_t)N * 4)) &&
         ok(cudaMalloc(reinterpret_cast<void**>(&p->db), (size_t)N * 4));
  good = good && ok(cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking)) &&
         ok(cudaStreamCreateWithFlags(&p->s_compute, cudaStreamNonBlocking)) &&
         ok(cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking));
  cudaEvent_t* evs[] = {&p->e_xw, &p->e_dy, &p->e_fwd, &p->e_dw, &p->e_dx};
  for (cudaEvent_t* e : evs) good = good && ok(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
  if (!good) { destroy(p); return kCudaError; }
  *out = p;
  return kOk;
}

void ge2b_dense_plan_destroy(ge2b_dense_plan* plan) { destroy(plan); }

int ge2b_dense_plan_step(ge2b_dense_plan* p, const void* X, const void* W, const float* bias, const void* dY,
                         void* Y, void* dX, void* dW, float* db) {
  if (!p || !X || !W || !dY) return kBadArgs;
  if (p->has_bias && !bias) return kBadArgs;
  const size_t mk = (size_t)p->M * p->K * p->esz, kn = (size_t)p->K * p->N * p->esz, mn = (size_t)p->M * p->N * p->esz;
  const auto H2D = cudaMemcpyHostToDevice;
  const auto D2H = cudaMemcpyDeviceToHost;

  // copy-in stream
  bool good = ok(cudaMemcpyAsync(p->X, X, mk, H2D, p->s_in)) && ok(cudaMemcpyAsync(p->W, W, kn, H2D, p->s_in));
  if (p->has_bias) good = good && ok(cudaMemcpyAsync(p->bias, bias, (size_t)p->N * 4, H2D, p->s_in));
  good = good && ok(cudaEventRecord(p->e_xw, p->s_in));
  good = good && ok(cudaMemcpyAsync(p->dY, dY, mn, H2D, p->s_in)) && ok(cudaEventRecord(p->e_dy, p->s_in));
  if (!good) return kCudaError;

  // compute stream: forward, then dW (+ db), then dX
  DenseForward f;
  f.M = p->M; f.N = p->N; f.K = p->K;
  f.dtype = p->dtype; f.z_dtype = p->dtype; f.math = p->math;
  f.A = p->X; f.lda = p->K; f.B = p->W; f.ldb = p->N; f.D = p->Y; f.ldd = p->N; f.Z = p->Z; f.ldz = p->N;
  f.bias = p->has_bias ? p->bias : nullptr; f.bias_kind = p->has_bias ? kBiasPerN : kBiasNone;
  f.act = p->act; f.leaky = p->leaky;
  if (!ok(cudaStreamWaitEvent(p->s_compute, p->e_xw, 0))) return kCudaError;
  int rc = dense_forward(f, p->s_compute);
  if (rc != kOk) return rc;
  if (!ok(cudaEventRecord(p->e_fwd, p->s_compute)) || !ok(cudaStreamWaitEvent(p->s_compute, p->e_dy, 0)))
    return kCudaError;

  DenseBackward b;
  b.M = p->M; b.N = p->N; b.K = p->K;
  b.dtype = p->dtype; b.z_dtype = p->dtype; b.math = p->math;
  b.A = p->X; b.lda = p->K; b.B = p->W; b.ldb = p->N;
  b.gY = p->dY; b.ldgY = p->N; b.Z = p->Z; b.ldZ = p->N;
  b.act = p->act; b.leaky = p->leaky;
  b.scratch = p->gZ; b.scratch_bytes = mn;
  b.gB = p->dW; b.ldgB = p->N;
  b.gBias = p->has_bias ? p->db : nullptr; b.bias_kind = p->has_bias ? kBiasPerN : kBiasNone;
  rc = dense_backward(b, p->s_compute);                 // prologue (gZ, db) + dW
  if (rc != kOk) return rc;
  if (!ok(cudaEventRecord(p->e_dw, p->s_compute))) return kCudaError;
  b.gB = nullptr; b.gBias = nullptr; b.bias_kind = kBiasNone;
  b.gA = p->dX; b.ldgA = p->K; b.reuse_gz = true;
  rc = dense_backward(b, p->s_compute);                 // dX from the gZ already in the scratch
  if (rc != kOk) return rc;
  if (!ok(cudaEventRecord(p->e_dx, p->s_compute))) return kCudaError;

  // copy-out stream
  good = ok(cudaStreamWaitEvent(p->s_out, p->e_fwd, 0));
  if (Y) good = good && ok(cudaMemcpyAsync(Y, p->Y, mn, D2H, p->s_out));
  good = good && ok(cudaStreamWaitEvent(p->s_out, p->e_dw, 0));
  if (dW) good = good && ok(cudaMemcpyAsync(dW, p->dW, kn, D2H, p->s_out));
  if (db && p->has_bias) good = good && ok(cudaMemcpyAsync(db, p->db, (size_t)p->N * 4, D2H, p->s_out));
  good = good && ok(cudaStreamWaitEvent(p->s_out, p->e_dx, 0));
  if (dX) good = good && ok(cudaMemcpyAsync(dX, p->dX, mk, D2H, p->s_out));
  if (!good) return kCudaError;
  return ok(cudaStreamSynchronize(p->s_out)) ? kOk : kCudaError;
}

}  // extern "C"
