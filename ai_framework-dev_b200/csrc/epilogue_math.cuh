// Device-side activation math of the dense-layer epilogue and of its derivative.
//
// Restates the formulas of the reference's GEMM path
// (backends/cuda/ops/_common/shim/activations.hpp:11-120, math_compat.hpp:12-28):
//   GELU is the tanh form with c = 0.7978845608f, k1 = 0.044715f and t = fmaf(c*k1, x^3, c*x);
//   sigmoid is the two-branch overflow-safe form evaluated with __expf on the device;
//   tanh is tanhf; the GELU derivative clamps tanh to +-0.999999 before forming sech^2;
//   ReLU' is 0 at x == 0; LeakyReLU uses the slope carried in the attributes.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include "ge2_internal.hpp"

namespace ge2b {

__device__ __forceinline__ float gelu_inner(float x) {
  const float c = 0.7978845608f, k1 = 0.044715f;
  const float x2 = x * x, x3 = x2 * x;
  return fmaf(c * k1, x3, c * x);
}

__device__ __forceinline__ float sigmoid_stable(float x) {
  if (x >= 0.f) { const float z = __expf(-x); return 1.f / (1.f + z); }
  const float z = __expf(x);
  return z / (1.f + z);
}

// kFast selects exp-based forms of tanh and sigmoid (two special-function instructions and no branches, absolute
// error about 1e-7).  It is used only where the result is rounded to a 16-bit type afterwards; fp32 results keep
// tanhf and the two-branch sigmoid so that they match the reference's device code.
__device__ __forceinline__ float tanh_fast(float x) {
#ifdef GE2B_TANH_EXP
  return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x));      // exp -> inf gives 1, exp -> 0 gives -1
#else
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));        // one special-function instruction, rel. error 2^-11
  return y;
#endif
}
__device__ __forceinline__ float sigmoid_fast(float x) {
#ifdef GE2B_TANH_EXP
  return __fdividef(1.f, 1.f + __expf(-x));
#else
  return fmaf(0.5f, tanh_fast(0.5f * x), 0.5f);
#endif
}

template <int ACT, bool kFast = false>
__device__ __forceinline__ float act_fwd(float x, float leaky) {
  if constexpr (ACT == kActReLU)         return x > 0.f ? x : 0.f;
  else if constexpr (ACT == kActLeaky)   return x > 0.f ? x : leaky * x;
  else if constexpr (ACT == kActGELU) {
    if constexpr (kFast) {
      const float c = 0.7978845608f, k1 = 0.044715f;
      const float w = fmaf(x * x, c * k1, c);               // t = x * (c + c*k1*x^2)
      const float h = 0.5f * x;
      return fmaf(h, tanh_fast(x * w), h);
    } else {
      return 0.5f * x * (1.f + tanhf(gelu_inner(x)));
    }
  }
  else if constexpr (ACT == kActSigmoid) return kFast ? sigmoid_fast(x) : sigmoid_stable(x);
  else if constexpr (ACT == kActTanh)    return kFast ? tanh_fast(x) : tanhf(x);
  else                                   return x;
}

template <int ACT, bool kFast = false>
__device__ __forceinline__ float act_bwd(float x, float leaky) {
  if constexpr (ACT == kActReLU)       return x > 0.f ? 1.f : 0.f;
  else if constexpr (ACT == kActLeaky) return x > 0.f ? 1.f : leaky;
  else if constexpr (ACT == kActGELU) {
    const float c = 0.7978845608f, k1 = 0.044715f;
    const float x2 = x * x;
    if constexpr (kFast) {
      // tanh.approx stays inside [-1, 1], so 1 - th^2 cannot go negative and the clamp is not needed
      const float th = tanh_fast(x * fmaf(x2, c * k1, c));
      const float sech2 = fmaf(-th, th, 1.f);
      const float hxdt = (0.5f * x) * fmaf(x2, 3.f * c * k1, c);
      return fmaf(hxdt, sech2, fmaf(0.5f, th, 0.5f));
    }
    float th = tanhf(gelu_inner(x));
    th = fminf(fmaxf(th, -0.999999f), 0.999999f);
    const float sech2 = 1.f - th * th;
    const float dt = c * (1.f + 3.f * k1 * x2);
    return 0.5f * (1.f + th) + 0.5f * x * sech2 * dt;
  } else if constexpr (ACT == kActSigmoid) {
    const float s = kFast ? sigmoid_fast(x) : sigmoid_stable(x);
    return s * (1.f - s);
  } else if constexpr (ACT == kActTanh) {
    const float th = kFast ? tanh_fast(x) : tanhf(x);
    return 1.f - th * th;
  } else {
    return 1.f;
  }
}

__device__ __forceinline__ float act_fwd_rt(float x, int act, float leaky) {
  switch (act) {
    case kActReLU:    return act_fwd<kActReLU>(x, leaky);
    case kActLeaky:   return act_fwd<kActLeaky>(x, leaky);
    case kActGELU:    return act_fwd<kActGELU>(x, leaky);
    case kActSigmoid: return act_fwd<kActSigmoid>(x, leaky);
    case kActTanh:    return act_fwd<kActTanh>(x, leaky);
    default:          return x;
  }
}

__device__ __forceinline__ float act_bwd_rt(float x, int act, float leaky) {
  switch (act) {
    case kActReLU:    return act_bwd<kActReLU>(x, leaky);
    case kActLeaky:   return act_bwd<kActLeaky>(x, leaky);
    case kActGELU:    return act_bwd<kActGELU>(x, leaky);
    case kActSigmoid: return act_bwd<kActSigmoid>(x, leaky);
    case kActTanh:    return act_bwd<kActTanh>(x, leaky);
    default:          return 1.f;
  }
}

// ---- typed element access used by the generic (any dtype) code paths ----
__device__ __forceinline__ float load_as_f32(const void* p, long long i, int dt) {
  if (dt == kF32)  return reinterpret_cast<const float*>(p)[i];
  if (dt == kBF16) return __uint_as_float(static_cast<unsigned>(reinterpret_cast<const unsigned short*>(p)[i]) << 16);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ unsigned short f32_to_bf16_bits(float f) {
  // round to nearest even, NaN kept quiet
  unsigned u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<unsigned short>((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<unsigned short>(u >> 16);
}

__device__ __forceinline__ void store_from_f32(void* p, long long i, int dt, float v) {
  if (dt == kF32)       reinterpret_cast<float*>(p)[i] = v;
  else if (dt == kBF16) reinterpret_cast<unsigned short*>(p)[i] = f32_to_bf16_bits(v);
  else                  reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

}  // namespace ge2b
