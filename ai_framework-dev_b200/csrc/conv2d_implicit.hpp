// Host-side description of one implicit-GEMM convolution launch (conv2d_implicit.cu): the forward pass of a
// convolution and the input gradient of a unit-stride convolution are both expressed with it.
#pragma once
#include <cuda_runtime.h>

#include "dense_ops.hpp"

namespace ge2b {

constexpr int kConvMaxTaps = 128;        // Kh * Kw the kernel's tap table holds

struct ImplicitConv {
  int dtype = kBF16;                     // of input, weight and output (bf16 or f16)
  // input planes [image][channel][row][column]
  const void* X = nullptr;
  long long img_pitch = 0, plane_pitch = 0; int row_pitch = 0;     // in elements
  int H = 0, W = 0;                      // extent of one input plane (reads outside it are zero)
  // output planes [image][Cout][Ho][Wo]
  int Ho = 0, Wo = 0;
  long long P = 0;                       // images * Ho * Wo
  long long out_img_pitch = 0;           // elements from image to image (Cout * Ho * Wo when dense)
  int sh = 1, sw = 1;                    // input row / column = output row * sh + tap_row[t], column likewise
  int taps = 0;
  int tap_row[kConvMaxTaps] = {}, tap_col[kConvMaxTaps] = {};
  // weight matrix [Cout][K], K = channels * taps with the tap index fastest, pitch ldw elements
  const void* Wm = nullptr; long long ldw = 0;
  int K = 0, Cout = 0;
  const float* bias = nullptr;           // per output channel, may be null
  int act = kActNone; float leaky = 0.01f;
  void* Y = nullptr;
  void* Z = nullptr; int z_dtype = kBF16;  // optional pre-activation stash (dtype or fp32)
  bool force_general = false;            // tests: take the element-wise gather even where the aligned one applies
};

// Weight gradient dW[Cout][K] = sum over images and positions of gZ . Col: `in` describes the gathered input exactly as
// for the forward pass (X, pitches, extents, strides, taps, K, Cout, dtype; its weight / output fields are unused).
struct ImplicitWgrad {
  ImplicitConv in;
  int imgs = 0;
  const void* G = nullptr;               // gZ planes [image][Cout][Ho * Wo], 16-bit
  long long g_plane_pitch = 0, g_img_pitch = 0;
  void* dW = nullptr;                    // [Cout][K] dense, dtype of the input
  float* part = nullptr; size_t part_bytes = 0;   // scratch for the slices' partial sums (conv_wgrad_plan says how much)
};

bool conv_implicit_supported(const ImplicitConv& d);
// How many slices the reduction is cut into for this shape and the scratch they need; false: shape not taken.
bool conv_wgrad_plan(const ImplicitWgrad& w, int* split, size_t* part_bytes);
int conv_wgrad_launch(const ImplicitWgrad& w, cudaStream_t s);
// kUnimplemented when the shape is outside what the kernel takes (the caller then uses the column-matrix route).
int conv_implicit_launch(const ImplicitConv& d, cudaStream_t s);
// Wt[ci][co * taps + t] = W[co][ci][t]: the weight as the input-gradient convolution reads it (pitch ldt elements).
cudaError_t launch_transpose_weight(const void* W, void* Wt, int Cout, int Cin, int taps, long long ldt, cudaStream_t s);

// ---- unit-stride convolution from a position-major input patch in shared memory (conv2d_patch.cu) ----
// Y[n][co][ho][wo] = act(bias[co] + sum over c, kh, kw of X[n][c][ho + kh*dh - ph][wo + kw*dw - pw] . Wt(co, c, kh, kw))
// with Wt(co, c, tap) = W[co * w_row_stride + c * w_chan_stride + tap'] and tap' = tap, or the mirrored tap when
// flip_taps is set (the input-gradient form).
struct PatchConv {
  int dtype = kBF16;
  const void* X = nullptr;
  long long img_pitch = 0, plane_pitch = 0; int row_pitch = 0;
  int imgs = 0, Cin = 0, H = 0, W = 0;
  int ph = 0, pw = 0, Kh = 1, Kw = 1, dh = 1, dw = 1;
  const void* W_ = nullptr;              // weight elements as described above
  long long w_row_stride = 0, w_chan_stride = 0;
  bool flip_taps = false;
  void* Wr = nullptr;                    // scratch of conv_patch_weight_bytes(): the weight as the kernel reads it
  int Cout = 0;
  const float* bias = nullptr;
  int act = kActNone; float leaky = 0.01f;
  void* Y = nullptr;                     // dense planes of Ho x Wo
  void* Z = nullptr; int z_dtype = kBF16;
  long long out_img_pitch = 0;
  // Optional generalisations (zero: the plain convolution described above).
  // A list of taps instead of the Kh x Kw grid: tap i reads the padded pixel (ho + tap_r[i], wq + tap_c[i]) and uses
  // the weight's tap tap_src[i]; Kh, Kw, dh, dw and flip_taps are then unused.
  int n_taps = 0;
  int tap_r[kConvMaxTaps] = {}, tap_c[kConvMaxTaps] = {}, tap_src[kConvMaxTaps] = {};
  int Wp = 0;                            // padded row width (>= W + pw and >= out_W + largest tap_c)
  int out_H = 0, out_W = 0;              // output extent
  // Output position (ho, wq) of channel co is written to Y[n*out_img_pitch + co*out_plane + ho*osh*out_row_pitch +
  // wq*osw + out_off] (defaults: dense planes of out_H x out_W).
  long long out_plane = 0; int out_row_pitch = 0, osh = 0, osw = 0, out_off = 0;
};
size_t conv_patch_weight_bytes(const PatchConv& d);
bool conv_patch_supported(const PatchConv& d);
int conv_patch_launch(const PatchConv& d, cudaStream_t s);

}  // namespace ge2b
