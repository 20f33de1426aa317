// TEST INFRASTRUCTURE ONLY.  C interface over the reference's own convolution op
// (backends/cuda/ops/conv2d/api.hpp:44-64), linked with the reference's conv2d and GEMM sources compiled for sm_100a
// from the mounted reference tree (see oracle/Makefile).  Allocates the workspaces the reference asks for
// (api.hpp:20-41) with cudaMalloc, runs the op, frees them.  All tensors fp32, contiguous.
#include <cuda_runtime.h>

#include <algorithm>
#include <vector>

#include "backends/cuda/ops/conv2d/api.hpp"

namespace {

ai::Tensor t4(const void* p, long long a, long long b, long long c, long long d) {
  ai::Tensor t;
  t.data = const_cast<void*>(p);
  t.device = ai::Device::CUDA;
  t.device_index = 0;
  t.desc.dtype = ai::DType::F32;
  t.desc.layout = ai::Layout::RowMajor;
  t.desc.shape = {a, b, c, d};
  t.desc.stride = {b * c * d, c * d, d, 1};
  return t;
}

struct Bufs {
  std::vector<void*> ptrs;
  float* get(size_t elems) {
    void* p = nullptr;
    if (cudaMalloc(&p, std::max<size_t>(elems, 1) * sizeof(float)) != cudaSuccess) return nullptr;
    ptrs.push_back(p);
    return static_cast<float*>(p);
  }
  ~Bufs() { for (void* p : ptrs) cudaFree(p); }
};

ai::Conv2DAttrs attrs_of(int sh, int sw, int ph, int pw, int dh, int dw, int act, float leaky, bool bias, bool save_z) {
  ai::Conv2DAttrs a;
  a.stride_h = sh; a.stride_w = sw; a.pad_h = ph; a.pad_w = pw; a.dil_h = dh; a.dil_w = dw;
  a.groups = 1;
  a.act = static_cast<ai::ActKind>(act);
  a.leaky_slope = leaky;
  a.with_bias = bias;
  a.save_z = save_z;
  return a;
}

}  // namespace

extern "C" {

int ref_conv_forward(const float* X, const float* W, const float* bias, float* Y, float* Z, int N, int Cin, int H, int Wd,
                     int Cout, int Kh, int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int act, float leaky,
                     void* stream) {
  const int Ho = (H + 2 * ph - dh * (Kh - 1) - 1) / sh + 1, Wo = (Wd + 2 * pw - dw * (Kw - 1) - 1) / sw + 1;
  const size_t HWo = static_cast<size_t>(Ho) * Wo, K = static_cast<size_t>(Cin) * Kh * Kw;
  Bufs b;
  ai::Conv2DWorkspaceFwd ws;
  ws.dCol = b.get(HWo * K); ws.W_KC = b.get(K * Cout); ws.Y_tmp = b.get(HWo * Cout); ws.Z_rows = b.get(HWo * Cout);
  if (!ws.dCol || !ws.W_KC || !ws.Y_tmp || !ws.Z_rows) return -2;
  ai::Tensor tX = t4(X, N, Cin, H, Wd), tW = t4(W, Cout, Cin, Kh, Kw), tY = t4(Y, N, Cout, Ho, Wo), tZ = t4(Z, N, Cout, Ho, Wo);
  ai::Tensor tB;
  if (bias) { tB.data = const_cast<float*>(bias); tB.desc.shape = {Cout}; tB.desc.stride = {1}; }
  const ai::Conv2DAttrs a = attrs_of(sh, sw, ph, pw, dh, dw, act, leaky, bias != nullptr, Z != nullptr);
  const int st = static_cast<int>(ai::Conv2DCudaLaunch(tX, tW, bias ? &tB : nullptr, tY, a,
                                                       reinterpret_cast<cudaStream_t>(stream), Z ? &tZ : nullptr, &ws));
  cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream));
  return st;
}

int ref_conv_backward(const float* X, const float* W, const float* dY, const float* Z, float* dW, float* dB, float* dX,
                      int N, int Cin, int H, int Wd, int Cout, int Kh, int Kw, int sh, int sw, int ph, int pw, int dh,
                      int dw, int act, float leaky, void* stream) {
  const int Ho = (H + 2 * ph - dh * (Kh - 1) - 1) / sh + 1, Wo = (Wd + 2 * pw - dw * (Kw - 1) - 1) / sw + 1;
  const size_t HWo = static_cast<size_t>(Ho) * Wo, K = static_cast<size_t>(Cin) * Kh * Kw;
  Bufs b;
  ai::Conv2DWorkspaceBwd ws;
  ws.dCol = b.get(HWo * K); ws.dTmp = b.get(std::max(K * Cout, HWo * K)); ws.W_CK = b.get(K * Cout);
  ws.dY_HT = b.get(HWo * Cout); ws.dWpack = b.get(K * Cout); ws.gy_rows = b.get(HWo * Cout); ws.Z_rows = b.get(HWo * Cout);
  if (!ws.dCol || !ws.dTmp || !ws.W_CK || !ws.dY_HT || !ws.dWpack || !ws.gy_rows || !ws.Z_rows) return -2;
  ai::Tensor tX = t4(X, N, Cin, H, Wd), tW = t4(W, Cout, Cin, Kh, Kw), tdY = t4(dY, N, Cout, Ho, Wo), tZ = t4(Z, N, Cout, Ho, Wo);
  ai::Tensor tdW = t4(dW, Cout, Cin, Kh, Kw), tdX = t4(dX, N, Cin, H, Wd), tdB;
  if (dB) { tdB.data = dB; tdB.desc.shape = {Cout}; tdB.desc.stride = {1}; }
  const ai::Conv2DAttrs a = attrs_of(sh, sw, ph, pw, dh, dw, act, leaky, dB != nullptr, false);
  int st;
  try {
    st = static_cast<int>(ai::Conv2DCudaBackwardLaunch(tX, tW, tdY, tZ, dW ? &tdW : nullptr, dB ? &tdB : nullptr,
                                                       dX ? &tdX : nullptr, a, reinterpret_cast<cudaStream_t>(stream), &ws));
  } catch (...) {
    st = 3;
  }
  cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream));
  return st;
}

}  // extern "C"
