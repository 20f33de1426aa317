// Host-buffer plan: one dense-layer forward + backward per call with inputs and results in HOST memory.
//
// Counterpart of the reference's GemmPlan (graph_executor_v2/src/bindings/py_api.cpp:403-523): device buffers
// are allocated once when the plan is created; every step copies the inputs up, launches, and copies the
// results back.  Here a step is pipelined over three streams so that PCIe traffic in both directions overlaps
// the kernels: inputs (X, W, bias, then dY) go up on the copy-in stream; the forward kernel starts as soon as
// X and W are up; Y goes down while the backward runs; dW is computed first and goes down while dX is computed.
// `step` returns when all requested results are in host memory.  `submit` / `wait` split it so that a caller
// with two sets of host result buffers keeps two steps in flight (the plan owns two sets of device buffers):
// step i+1's inputs go up while step i computes and its results come down, which hides the dependency chain
// X,W -> forward -> ... -> dX of a single step behind the neighbouring steps' copies.  Pass page-locked host
// buffers for full copy speed; pageable ones work but serialise.
#include <cuda_runtime.h>

#include <new>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"

using namespace ge2b;

constexpr int kSlots = 2;   // two device buffer sets: step i+1 is copied in while step i computes / copies out

struct PlanSlot {
  void *X, *W, *dY, *Y, *Z, *gZ, *dX, *dW;
  float *bias, *db;
  cudaEvent_t e_xw, e_dy, e_fwd, e_dw, e_dx, e_out;   // e_out: this slot's results have reached the host
  bool busy;
};

struct ge2b_dense_plan {
  int M, K, N, dtype, act, has_bias, math;
  float leaky;
  int device;
  size_t esz;
  PlanSlot slot[kSlots];
  cudaStream_t s_in, s_compute, s_out;
  unsigned long long submitted, waited;
};

namespace {

bool ok(cudaError_t e) { return e == cudaSuccess; }

void destroy(ge2b_dense_plan* p) {
  if (!p) return;
  for (PlanSlot& sl : p->slot) {
    void* bufs[] = {sl.X, sl.W, sl.dY, sl.Y, sl.Z, sl.gZ, sl.dX, sl.dW, sl.bias, sl.db};
    for (void* b : bufs)
      if (b) cudaFree(b);
    cudaEvent_t es[] = {sl.e_xw, sl.e_dy, sl.e_fwd, sl.e_dw, sl.e_dx, sl.e_out};
    for (cudaEvent_t e : es)
      if (e) cudaEventDestroy(e);
  }
  cudaStream_t ss[] = {p->s_in, p->s_compute, p->s_out};
  for (cudaStream_t s : ss)
    if (s) cudaStreamDestroy(s);
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
  p->math = (dtype == GE2_DT_F32) ? (math == GE2_MATH_TENSOR ? 1 : (math == GE2_MATH_FP32X3 ? 2 : 0)) : 1;
  p->esz = dtype_bytes(dtype);
  const size_t mk = (size_t)M * K * p->esz, kn = (size_t)K * N * p->esz, mn = (size_t)M * N * p->esz;
  bool good = ok(cudaGetDevice(&p->device));
  for (PlanSlot& sl : p->slot) {
    good = good && ok(cudaMalloc(&sl.X, mk)) && ok(cudaMalloc(&sl.W, kn)) && ok(cudaMalloc(&sl.dY, mn)) &&
           ok(cudaMalloc(&sl.Y, mn)) && ok(cudaMalloc(&sl.Z, mn)) && ok(cudaMalloc(&sl.gZ, mn)) &&
           ok(cudaMalloc(&sl.dX, mk)) && ok(cudaMalloc(&sl.dW, kn)) &&
           ok(cudaMalloc(reinterpret_cast<void**>(&sl.bias), (size_t)N * 4)) &&
           ok(cudaMalloc(reinterpret_cast<void**>(&sl.db), (size_t)N * 4));
    cudaEvent_t* evs[] = {&sl.e_xw, &sl.e_dy, &sl.e_fwd, &sl.e_dw, &sl.e_dx, &sl.e_out};
    for (cudaEvent_t* e : evs) good = good && ok(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
  }
  good = good && ok(cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking)) &&
         ok(cudaStreamCreateWithFlags(&p->s_compute, cudaStreamNonBlocking)) &&
         ok(cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking));
  if (!good) { destroy(p); return kCudaError; }
  *out = p;
  return kOk;
}

void ge2b_dense_plan_destroy(ge2b_dense_plan* plan) {
  if (plan) cudaStreamSynchronize(plan->s_out);
  destroy(plan);
}

int ge2b_dense_plan_wait(ge2b_dense_plan* p) {
  if (!p) return kBadArgs;
  if (p->waited == p->submitted) return kOk;
  PlanSlot& sl = p->slot[p->waited % kSlots];
  const bool good = ok(cudaEventSynchronize(sl.e_out));
  sl.busy = false;
  ++p->waited;
  return good ? kOk : kCudaError;
}

int ge2b_dense_plan_submit(ge2b_dense_plan* p, const void* X, const void* W, const float* bias, const void* dY,
                           void* Y, void* dX, void* dW, float* db) {
  if (!p || !X || !W || !dY) return kBadArgs;
  if (p->has_bias && !bias) return kBadArgs;
  if (p->submitted - p->waited >= kSlots) {           // both buffer sets in flight: retire the oldest first
    const int rc = ge2b_dense_plan_wait(p);
    if (rc != kOk) return rc;
  }
  PlanSlot& sl = p->slot[p->submitted % kSlots];
  const size_t mk = (size_t)p->M * p->K * p->esz, kn = (size_t)p->K * p->N * p->esz, mn = (size_t)p->M * p->N * p->esz;
  const auto H2D = cudaMemcpyHostToDevice;
  const auto D2H = cudaMemcpyDeviceToHost;

  // copy-in stream (the slot's previous occupant has been waited for, so its buffers are free)
  bool good = ok(cudaMemcpyAsync(sl.X, X, mk, H2D, p->s_in)) && ok(cudaMemcpyAsync(sl.W, W, kn, H2D, p->s_in));
  if (p->has_bias) good = good && ok(cudaMemcpyAsync(sl.bias, bias, (size_t)p->N * 4, H2D, p->s_in));
  good = good && ok(cudaEventRecord(sl.e_xw, p->s_in));
  good = good && ok(cudaMemcpyAsync(sl.dY, dY, mn, H2D, p->s_in)) && ok(cudaEventRecord(sl.e_dy, p->s_in));
  if (!good) return kCudaError;

  // compute stream: forward, then dW (+ db), then dX
  DenseForward f;
  f.M = p->M; f.N = p->N; f.K = p->K;
  f.dtype = p->dtype; f.z_dtype = p->dtype; f.math = p->math;
  f.A = sl.X; f.lda = p->K; f.B = sl.W; f.ldb = p->N; f.D = sl.Y; f.ldd = p->N; f.Z = sl.Z; f.ldz = p->N;
  f.bias = p->has_bias ? sl.bias : nullptr; f.bias_kind = p->has_bias ? kBiasPerN : kBiasNone;
  f.act = p->act; f.leaky = p->leaky;
  if (!ok(cudaStreamWaitEvent(p->s_compute, sl.e_xw, 0))) return kCudaError;
  int rc = dense_forward(f, p->s_compute);
  if (rc != kOk) return rc;
  if (!ok(cudaEventRecord(sl.e_fwd, p->s_compute)) || !ok(cudaStreamWaitEvent(p->s_compute, sl.e_dy, 0)))
    return kCudaError;

  DenseBackward b;
  b.M = p->M; b.N = p->N; b.K = p->K;
  b.dtype = p->dtype; b.z_dtype = p->dtype; b.math = p->math;
  b.A = sl.X; b.lda = p->K; b.B = sl.W; b.ldb = p->N;
  b.gY = sl.dY; b.ldgY = p->N; b.Z = sl.Z; b.ldZ = p->N;
  b.act = p->act; b.leaky = p->leaky;
  b.scratch = sl.gZ; b.scratch_bytes = mn;
  b.gB = sl.dW; b.ldgB = p->N;
  b.gBias = p->has_bias ? sl.db : nullptr; b.bias_kind = p->has_bias ? kBiasPerN : kBiasNone;
  rc = dense_backward(b, p->s_compute);                 // prologue (gZ, db) + dW
  if (rc != kOk) return rc;
  if (!ok(cudaEventRecord(sl.e_dw, p->s_compute))) return kCudaError;
  b.gB = nullptr; b.gBias = nullptr; b.bias_kind = kBiasNone;
  b.gA = sl.dX; b.ldgA = p->K; b.reuse_gz = true;
  rc = dense_backward(b, p->s_compute);                 // dX from the gZ already in the scratch
  if (rc != kOk) return rc;
  if (!ok(cudaEventRecord(sl.e_dx, p->s_compute))) return kCudaError;

  // copy-out stream
  good = ok(cudaStreamWaitEvent(p->s_out, sl.e_fwd, 0));
  if (Y) good = good && ok(cudaMemcpyAsync(Y, sl.Y, mn, D2H, p->s_out));
  good = good && ok(cudaStreamWaitEvent(p->s_out, sl.e_dw, 0));
  if (dW) good = good && ok(cudaMemcpyAsync(dW, sl.dW, kn, D2H, p->s_out));
  if (db && p->has_bias) good = good && ok(cudaMemcpyAsync(db, sl.db, (size_t)p->N * 4, D2H, p->s_out));
  good = good && ok(cudaStreamWaitEvent(p->s_out, sl.e_dx, 0));
  if (dX) good = good && ok(cudaMemcpyAsync(dX, sl.dX, mk, D2H, p->s_out));
  good = good && ok(cudaEventRecord(sl.e_out, p->s_out));
  if (!good) return kCudaError;
  sl.busy = true;
  ++p->submitted;
  return kOk;
}

int ge2b_dense_plan_step(ge2b_dense_plan* p, const void* X, const void* W, const float* bias, const void* dY,
                         void* Y, void* dX, void* dW, float* db) {
  int rc = ge2b_dense_plan_submit(p, X, W, bias, dY, Y, dX, dW, db);
  if (rc != kOk) return rc;
  while (p->waited < p->submitted) {
    rc = ge2b_dense_plan_wait(p);
    if (rc != kOk) return rc;
  }
  return kOk;
}

}  // extern "C"
