// C++ operator API of the convolution, with the reference's signatures (backends/cuda/ops/conv2d/api.hpp:6-64) so that
// its binding (src/bindings/conv2d_pybind.cpp) links against this library.  The workspace structs are kept for source
// compatibility; their buffers are not used (scratch is stream-ordered) and a null workspace is accepted.
// Differences from the reference, all additive: tensors may be BF16 / F16 as well as F32; dB sums over the whole batch.
#pragma once
#include "ge2_op_api.hpp"

namespace ai {

using cuda::shim::ActKind;
using cuda::shim::Status;
using cuda::shim::StreamHandle;
using cuda::shim::Tensor;

struct Conv2DAttrs {
  int stride_h{1}, stride_w{1};
  int pad_h{0}, pad_w{0};
  int dil_h{1}, dil_w{1};
  int groups{1};
  ActKind act{ActKind::None};
  float leaky_slope{0.01f};
  bool with_bias{false};
  bool save_z{false};
};

struct Conv2DWorkspaceFwd {
  float* dCol{nullptr};
  float* W_KC{nullptr};
  float* Y_tmp{nullptr};
  float* Z_rows{nullptr};
};

struct Conv2DWorkspaceBwd {
  float* dCol{nullptr};
  float* dTmp{nullptr};
  float* W_CK{nullptr};
  float* dY_HT{nullptr};
  float* dWpack{nullptr};
  float* gy_rows{nullptr};
  float* Z_rows{nullptr};
};

Status Conv2DCudaLaunch(const Tensor& X, const Tensor& W, const Tensor* B, Tensor& Y, const Conv2DAttrs& attrs,
                        StreamHandle stream, Tensor* Z_saved = nullptr, const Conv2DWorkspaceFwd* ws_fwd = nullptr);

Status Conv2DCudaBackwardLaunch(const Tensor& X, const Tensor& W, const Tensor& dY, const Tensor& Z, Tensor* dW,
                                Tensor* dB, Tensor* dX, const Conv2DAttrs& attrs, StreamHandle stream,
                                const Conv2DWorkspaceBwd* ws_bwd = nullptr);

}  // namespace ai
