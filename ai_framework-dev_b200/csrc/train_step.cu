// The two HBM-bound passes that sit either side of the dense layers inside a training step:
//   * fused softmax + cross-entropy forward/backward from logits, one warp per row:
//       loss_row = logsumexp(x) - x[label],  dlogits = (softmax(x) - onehot(label)) * grad_scale
//     Restates softmax_ce_fused_fwd_bwd_kernel (backends/cuda/ops/cross_entropy/kernels.cu:287-372): max-shifted
//     exponentials with __expf, logf of the denominator, the scalar loss accumulated with atomicAdd into a zeroed
//     word (Mean divides by the number of rows, ignored rows included, as the native op does:
//     cross_entropy/launcher.cu:114-115).  Additions: 16-bit logits / gradients, a row is read once into registers
//     when it has at most 2048 classes, `grad_scale` folds the 1/batch of a mean loss (or 1/global batch under data
//     parallelism) into the gradient, an ignore_index row yields zero loss and zero gradient, and label smoothing
//     follows the reference's separate forward / backward ops (kernels.cu:96-101, 188-195):
//     loss_row = (1-ls)(logZ - x_t) + ls (logZ - mean(x)),  target = (1-ls) onehot + ls / C.
//   * SGD update on fp32 master weights with an optional low-precision copy for the next forward:
//       g' = grad_scale * g (+ wd * p when decay is L2);  v = mu * v + (1 - damp) * g';  step = nesterov ? g' + mu * v : v
//       p -= lr * step (+ lr * wd * p when decay is decoupled)
//     L2 form: backends/cuda/ops/optimizer/kernels.cu:33-66; decoupled form: python/graph_executor_v2/optim/sgd.py:16-34.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"
#include "epilogue_math.cuh"

using namespace ge2b;

namespace {

constexpr int kRowsPerBlock = 8;      // one warp per row

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct CeParams {
  const void* logits; long long ld_x; int x_dtype;
  const int* labels;
  void* dlogits; long long ld_d; int d_dtype;
  float* loss;                 // null, [M] (reduction none) or [1]
  int M, C, reduction, ignore_index;
  float grad_scale, loss_scale;
  float ls;                    // label smoothing: target = (1 - ls) * onehot + ls / C
};

// kCache > 0: a lane keeps kCache values of its row in registers (rows of up to 32*kCache classes are read once);
// kCache == 0: any row length, three passes over the row.
template <int kCache>
__global__ void __launch_bounds__(32 * kRowsPerBlock)
softmax_ce_fused_kernel(const CeParams p) {
  constexpr bool kCached = kCache > 0;
  constexpr int kMaxCached = kCached ? kCache : 1;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);
  if (row >= p.M) return;
  const long long xo = static_cast<long long>(row) * p.ld_x, dox = static_cast<long long>(row) * p.ld_d;
  const int t = p.labels[row];
  const bool ignored = (t == p.ignore_index) || t < 0 || t >= p.C;

  float cache[kMaxCached];
  float m = -CUDART_INF_F;
  float sumx = 0.f;            // sum of the row's logits, for the smoothed target's uniform part
  if constexpr (kCached) {
#pragma unroll
    for (int i = 0; i < kMaxCached; ++i) {
      const int c = lane + 32 * i;
      cache[i] = (c < p.C) ? load_as_f32(p.logits, xo + c, p.x_dtype) : -CUDART_INF_F;
      m = fmaxf(m, cache[i]);
      if (c < p.C) sumx += cache[i];
    }
  } else {
    for (int c = lane; c < p.C; c += 32) {
      const float x = load_as_f32(p.logits, xo + c, p.x_dtype);
      m = fmaxf(m, x);
      sumx += x;
    }
  }
  m = warp_max(m);
  if (p.ls != 0.f) sumx = warp_sum(sumx);

  float s = 0.f;
  if constexpr (kCached) {
#pragma unroll
    for (int i = 0; i < kMaxCached; ++i) {
      cache[i] = __expf(cache[i] - m);       // exp(-inf) = 0 for the padding
      s += cache[i];
    }
  } else {
    for (int c = lane; c < p.C; c += 32) s += __expf(load_as_f32(p.logits, xo + c, p.x_dtype) - m);
  }
  s = warp_sum(s);

  if (lane == 0 && p.loss != nullptr) {
    float loss_row = 0.f;
    if (!ignored) {
      const float logZ = m + logf(s);
      loss_row = logZ - load_as_f32(p.logits, xo + t, p.x_dtype);
      if (p.ls != 0.f) loss_row = (1.f - p.ls) * loss_row + p.ls * (logZ - sumx / static_cast<float>(p.C));
    }
    if (p.reduction == 0) p.loss[row] = loss_row;
    else if (!ignored)    atomicAdd(p.loss, loss_row * p.loss_scale);
  }

  const float inv = ignored ? 0.f : p.grad_scale / s;
  const float hot = ignored ? 0.f : p.grad_scale * (1.f - p.ls);
  const float uni = ignored ? 0.f : p.grad_scale * p.ls / static_cast<float>(p.C);
  if constexpr (kCached) {
#pragma unroll
    for (int i = 0; i < kMaxCached; ++i) {
      const int c = lane + 32 * i;
      if (c < p.C) store_from_f32(p.dlogits, dox + c, p.d_dtype, cache[i] * inv - (c == t ? hot : 0.f) - uni);
    }
  } else {
    for (int c = lane; c < p.C; c += 32) {
      const float e = __expf(load_as_f32(p.logits, xo + c, p.x_dtype) - m);
      store_from_f32(p.dlogits, dox + c, p.d_dtype, e * inv - (c == t ? hot : 0.f) - uni);
    }
  }
}

struct SgdParams {
  float* p; const void* g; int g_dtype; float* v; void* p_low; int low_dtype;
  long long n;
  float lr, momentum, dampening, weight_decay, grad_scale;
  int nesterov, decay_mode;     // decay_mode: 0 none, 1 L2 (added to the gradient), 2 decoupled
};

__global__ void __launch_bounds__(256)
sgd_update_kernel(const SgdParams a) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    float p = a.p[i];
    float g = a.grad_scale * load_as_f32(a.g, i, a.g_dtype);
    if (a.decay_mode == 1 && a.weight_decay != 0.f) g += a.weight_decay * p;
    float step = g;
    if (a.momentum > 0.f && a.v != nullptr) {
      const float v = a.momentum * a.v[i] + (1.f - a.dampening) * g;
      a.v[i] = v;
      step = a.nesterov ? (g + a.momentum * v) : v;
    }
    const float decay = (a.decay_mode == 2) ? a.lr * a.weight_decay * p : 0.f;
    p = p - a.lr * step - decay;
    a.p[i] = p;
    if (a.p_low != nullptr) store_from_f32(a.p_low, i, a.low_dtype, p);
  }
}

bool dtype_ok(int d) { return d == GE2_DT_F32 || d == GE2_DT_F16 || d == GE2_DT_BF16; }

// Plain SGD (p -= lr * g) on up to 16 tensors in ONE launch: a training step updates every weight and bias of the
// stack, and one launch per tensor costs more in launch gaps than the update itself once the tensors are small.
// Block b works on a 4096-element chunk; `first_block[t]` says where tensor t's chunks begin.  Four elements per
// thread and access (16-byte master loads / stores, 8- or 16-byte gradient loads) when the tensor's element count
// and addresses allow, else scalar.
constexpr int kSgdChunk = 4096;
struct SgdMultiParams {
  SgdTensor t[kSgdMaxTensors];
  int first_block[kSgdMaxTensors + 1];
  int n_tensors;
  float lr;
};

__device__ __forceinline__ void load4(const void* g, long long i, int dt, float (&v)[4]) {
  if (dt == kF32) {
    const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(g) + i);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const unsigned short*>(g) + i);
    if (dt == kBF16) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
  }
}

__global__ void __launch_bounds__(256) sgd_multi_kernel(const SgdMultiParams a) {
  int ti = 0;
  while (ti + 1 < a.n_tensors && static_cast<int>(blockIdx.x) >= a.first_block[ti + 1]) ++ti;
  const SgdTensor t = a.t[ti];
  const long long begin = static_cast<long long>(blockIdx.x - a.first_block[ti]) * kSgdChunk;
  const long long end = begin + kSgdChunk < t.n ? begin + kSgdChunk : t.n;
  const bool vec = (t.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) |
                                       reinterpret_cast<uintptr_t>(t.low)) % 16 == 0);
  if (vec) {
    for (long long i = begin + 4ll * threadIdx.x; i < end; i += 4 * 256) {
      float4 p = *reinterpret_cast<float4*>(t.p + i);
      float g[4];
      load4(t.g, i, t.g_dtype, g);
      p.x -= a.lr * g[0]; p.y -= a.lr * g[1]; p.z -= a.lr * g[2]; p.w -= a.lr * g[3];
      *reinterpret_cast<float4*>(t.p + i) = p;
      if (t.low != nullptr) {
        if (t.low_dtype == kBF16) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
          *reinterpret_cast<uint2*>(static_cast<unsigned short*>(t.low) + i) =
              make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
        } else if (t.low_dtype == kF16) {
          __half2 lo = __floats2half2_rn(p.x, p.y), hi = __floats2half2_rn(p.z, p.w);
          *reinterpret_cast<uint2*>(static_cast<unsigned short*>(t.low) + i) =
              make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
        } else {
          *reinterpret_cast<float4*>(static_cast<float*>(t.low) + i) = p;
        }
      }
    }
  } else {
    for (long long i = begin + threadIdx.x; i < end; i += 256) {
      const float p = t.p[i] - a.lr * load_as_f32(t.g, i, t.g_dtype);
      t.p[i] = p;
      if (t.low != nullptr) store_from_f32(t.low, i, t.low_dtype, p);
    }
  }
}

}  // namespace

namespace ge2b {
int launch_sgd_multi(const SgdTensor* t, int n, float lr, cudaStream_t s) {
  if (!t || n < 1 || n > kSgdMaxTensors) return kBadArgs;
  SgdMultiParams a{};
  int blocks = 0;
  for (int i = 0; i < n; ++i) {
    if (!t[i].p || !t[i].g || t[i].n <= 0) return kBadArgs;
    a.t[i] = t[i];
    a.first_block[i] = blocks;
    blocks += static_cast<int>((t[i].n + kSgdChunk - 1) / kSgdChunk);
  }
  a.first_block[n] = blocks;
  a.n_tensors = n;
  a.lr = lr;
  sgd_multi_kernel<<<blocks, 256, 0, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}
}  // namespace ge2b

extern "C" {

int ge2_launch_softmax_ce_fused(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 5) return kBadArgs;
  const auto* q = reinterpret_cast<const ge2_softmax_ce_params_t*>(bufs[n - 1]);
  if (!q || q->M <= 0 || q->C <= 0 || !bufs[0] || !bufs[1] || !bufs[2]) return kBadArgs;
  if (!dtype_ok(q->dtype) || !dtype_ok(q->grad_dtype) || q->reduction < 0 || q->reduction > 2) return kBadArgs;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  CeParams p{};
  p.logits = reinterpret_cast<const void*>(bufs[0]); p.ld_x = q->ld_logits > 0 ? q->ld_logits : q->C; p.x_dtype = q->dtype;
  p.labels = reinterpret_cast<const int*>(bufs[1]);
  p.dlogits = reinterpret_cast<void*>(bufs[2]); p.ld_d = q->ld_dlogits > 0 ? q->ld_dlogits : q->C; p.d_dtype = q->grad_dtype;
  p.loss = reinterpret_cast<float*>(bufs[3]);
  p.M = q->M; p.C = q->C; p.reduction = q->reduction; p.ignore_index = q->ignore_index;
  p.grad_scale = q->grad_scale;
  p.ls = q->label_smoothing;
  if (!(p.ls >= 0.f && p.ls < 1.f)) return kBadArgs;
  // Mean: divide by the stated denominator (the global batch under data parallelism), default the row count
  p.loss_scale = q->reduction == 1 ? 1.f / static_cast<float>(q->mean_denominator > 0 ? q->mean_denominator : q->M) : 1.f;
  if (p.loss && q->reduction != 0 && cudaMemsetAsync(p.loss, 0, sizeof(float), s) != cudaSuccess) return kCudaError;
  const int grid = (q->M + kRowsPerBlock - 1) / kRowsPerBlock;
  if (q->C <= 1024)      softmax_ce_fused_kernel<32><<<grid, 32 * kRowsPerBlock, 0, s>>>(p);
  else if (q->C <= 2048) softmax_ce_fused_kernel<64><<<grid, 32 * kRowsPerBlock, 0, s>>>(p);
  else                   softmax_ce_fused_kernel<0><<<grid, 32 * kRowsPerBlock, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int ge2_launch_sgd_update(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 5) return kBadArgs;
  const auto* q = reinterpret_cast<const ge2_sgd_params_t*>(bufs[n - 1]);
  if (!q || q->n <= 0 || !bufs[0] || !bufs[1]) return kBadArgs;
  if (!dtype_ok(q->grad_dtype) || !dtype_ok(q->low_dtype) || q->decay_mode < 0 || q->decay_mode > 2) return kBadArgs;
  SgdParams a{};
  a.p = reinterpret_cast<float*>(bufs[0]);
  a.g = reinterpret_cast<const void*>(bufs[1]); a.g_dtype = q->grad_dtype;
  a.v = reinterpret_cast<float*>(bufs[2]);
  a.p_low = reinterpret_cast<void*>(bufs[3]); a.low_dtype = q->low_dtype;
  a.n = q->n;
  a.lr = q->lr; a.momentum = q->momentum; a.dampening = q->dampening; a.weight_decay = q->weight_decay;
  a.grad_scale = q->grad_scale == 0.f ? 1.f : q->grad_scale;
  a.nesterov = q->nesterov; a.decay_mode = q->decay_mode;
  long long blocks = (q->n + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  sgd_update_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // extern "C"
