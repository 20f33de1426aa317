// TEST INFRASTRUCTURE ONLY.  C interface over the reference's own cross-entropy and optimizer ops
// (backends/cuda/ops/cross_entropy/api.hpp:22-60, backends/cuda/ops/optimizer/api.hpp:24-28), linked with those ops'
// sources compiled unmodified for sm_100a from the mounted reference tree (see oracle/Makefile).  All tensors fp32,
// contiguous; labels int32.
#include <cuda_runtime.h>

#include "backends/cuda/ops/cross_entropy/api.hpp"
#include "backends/cuda/ops/optimizer/api.hpp"

namespace {

ai::Tensor t2(const void* p, long long r, long long c) {
  ai::Tensor t;
  t.data = const_cast<void*>(p);
  t.device = ai::Device::CUDA;
  t.device_index = 0;
  t.desc.dtype = ai::DType::F32;
  t.desc.layout = ai::Layout::RowMajor;
  t.desc.shape = {r, c};
  t.desc.stride = {c, 1};
  return t;
}

ai::Tensor t1(const void* p, long long n, ai::DType dt) {
  ai::Tensor t;
  t.data = const_cast<void*>(p);
  t.device = ai::Device::CUDA;
  t.device_index = 0;
  t.desc.dtype = dt;
  t.desc.layout = ai::Layout::RowMajor;
  t.desc.shape = {n};
  t.desc.stride = {1};
  return t;
}

}  // namespace

extern "C" {

// reduction: 0 none (loss has M elements), 1 mean, 2 sum (loss has 1 element); loss may be null
int ref_ce_fused(const float* logits, const int* labels, float* dlogits, float* loss, int M, int C, int reduction,
                 void* stream) {
  ai::Tensor L = t2(logits, M, C), D = t2(dlogits, M, C), T = t1(labels, M, ai::DType::I32);
  ai::Tensor lo = t1(loss, reduction == 0 ? M : 1, ai::DType::F32);
  ai::SCEFuseAttrs a;
  a.reduction = static_cast<ai::SCEFuseAttrs::Reduction>(reduction);
  a.stable = true;
  return static_cast<int>(ai::SoftmaxCEFusedForwardBackwardCudaLaunch(L, T, D, loss ? &lo : nullptr, a,
                                                                       reinterpret_cast<ai::StreamHandle>(stream)));
}

// the separate forward (loss) and backward (dX) ops, which know ignore_index and label smoothing
int ref_ce_forward(const float* logits, const int* labels, float* loss, int M, int C, int reduction, int ignore_index,
                   float ls_eps, void* stream) {
  ai::Tensor L = t2(logits, M, C), T = t1(labels, M, ai::DType::I32);
  ai::Tensor lo = t1(loss, reduction == 0 ? M : 1, ai::DType::F32);
  ai::CrossEntropyAttrs a;
  a.from_logits = true;
  a.reduction = static_cast<ai::Reduction>(reduction);
  a.ignore_index = ignore_index;
  a.ls_eps = ls_eps;
  return static_cast<int>(ai::CrossEntropyCudaLaunch(L, T, lo, a, reinterpret_cast<ai::StreamHandle>(stream)));
}

int ref_ce_backward(const float* logits, const int* labels, float* dX, int M, int C, int reduction, int ignore_index,
                    float ls_eps, void* stream) {
  ai::Tensor L = t2(logits, M, C), D = t2(dX, M, C), T = t1(labels, M, ai::DType::I32);
  ai::CrossEntropyAttrs a;
  a.from_logits = true;
  a.reduction = static_cast<ai::Reduction>(reduction);
  a.ignore_index = ignore_index;
  a.ls_eps = ls_eps;
  return static_cast<int>(ai::CrossEntropyCudaBackwardLaunch(L, T, D, a, reinterpret_cast<ai::StreamHandle>(stream)));
}

int ref_sgd(float* P, const float* G, float* V, long long n, float lr, float momentum, float dampening, int nesterov,
            float weight_decay, void* stream) {
  ai::Tensor p = t1(P, n, ai::DType::F32), g = t1(G, n, ai::DType::F32), v = t1(V, n, ai::DType::F32);
  ai::SGDAttrs a;
  a.lr = lr; a.momentum = momentum; a.dampening = dampening; a.nesterov = nesterov != 0; a.weight_decay = weight_decay;
  return static_cast<int>(ai::SGDCudaUpdateLaunch(p, g, V ? &v : nullptr, a, reinterpret_cast<ai::StreamHandle>(stream)));
}

}  // extern "C"
