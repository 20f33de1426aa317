// 2-D convolution (NCHW tensors, OIHW weights, groups = 1) on the dense-layer GEMM kernels.
//
// The reference (backends/cuda/ops/conv2d/launcher.cu:115-462, kernels.cu:12-167) loops over the images of a batch
// and, per image, runs im2col -> GEMM -> transpose, after packing the weight into [K, Cout]; its backward adds
// two more transposes, a per-image GemmCudaBackward, col2im and an atomic transpose-add into the packed weight
// gradient.  Here the whole batch takes
//   forward   one im2col pass into Col[K][N][HWp] (output positions contiguous), then ONE strided-batched GEMM launch
//             Y[n] (Cout x HWo) = act(W (Cout x K) . Col[n] (K x HWo) + bias[co]) that writes NCHW directly: the OIHW
//             weight is already the row-major Cout x K matrix, the per-channel bias is the kernel's per-row bias, and
//             the pre-activation stash is the same launch's second output.  No weight packing, no transposes.
//   backward  gZ = dY * act'(Z) with per-(image, channel) row sums folded into dB; dW (Cout x K) as ONE launch whose
//             reduction runs over the output positions of every image (no atomics, no per-image partial results);
//             dCol[n] = W^T . gZ[n] as one batched launch into the Col buffer, then a gather-form col2im into dX.
//   1x1, stride 1, no padding: Col[n] is X[n] itself, so neither pass materialises anything.
// fp32 tensors run the exact fp32 kernel (same ascending-k fmaf chain per output as the reference's GEMM, so Z is
// bit-identical) unless math = tensor asks for TF32; bf16 / f16 tensors run on the tcgen05 kernel.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "../../include/ge2_b200.h"
#include "../../include/ge2_conv2d_api.hpp"
#include "conv2d_implicit.hpp"
#include "dense_ops.hpp"
#include "epilogue_math.cuh"

#include <cstdlib>
#include <cstring>
#include <vector>

namespace ge2b {
namespace {

struct ConvGeom {
  int N, Cin, H, W, Cout, Kh, Kw;
  int sh, sw, ph, pw, dh, dw;
  int Ho, Wo, HWo, HWp, K;      // HWp: HWo rounded up so that every Col / gZ row starts on a 32-byte boundary
};

constexpr int kColRows = 4;      // (k, n) rows per block: one warp each

// Col[k][n][hw] = X[n][c][ho*sh - ph + kh*dh][wo*sw - pw + kw*dw] (zero outside the image and in the padding columns
// hw >= HWo).  One warp per (k, n) row; a lane gathers 16 bytes' worth of consecutive output positions and writes
// them with one store.  T is the element's storage type: values are copied bit for bit.
template <typename T>
__global__ void __launch_bounds__(32 * kColRows)
im2col_batched_kernel(const T* __restrict__ X, T* __restrict__ Col, const ConvGeom g, const long long rows) {
  constexpr int V = 16 / sizeof(T);
  const long long kn = static_cast<long long>(blockIdx.x) * kColRows + threadIdx.y;
  if (kn >= rows) return;
  const int k = static_cast<int>(kn / g.N), n = static_cast<int>(kn - static_cast<long long>(k) * g.N);
  const int kw = k % g.Kw;
  const int t = k / g.Kw;
  const int kh = t % g.Kh, c = t / g.Kh;
  const T* __restrict__ xc = X + (static_cast<long long>(n) * g.Cin + c) * g.H * g.W;
  T* __restrict__ col = Col + kn * g.HWp;
  const int h_off = kh * g.dh - g.ph, w_off = kw * g.dw - g.pw;
  for (int v = threadIdx.x; v < g.HWp / V; v += 32) {
    const int hw0 = v * V;
    int ho = hw0 / g.Wo, wo = hw0 - ho * g.Wo;
    alignas(16) T vals[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
      T val = T(0);
      const int hi = ho * g.sh + h_off, wi = wo * g.sw + w_off;
      if (hw0 + j < g.HWo && static_cast<unsigned>(hi) < static_cast<unsigned>(g.H) &&
          static_cast<unsigned>(wi) < static_cast<unsigned>(g.W))
        val = __ldg(xc + hi * g.W + wi);
      vals[j] = val;
      if (++wo == g.Wo) { wo = 0; ++ho; }
    }
    *reinterpret_cast<uint4*>(col + hw0) = *reinterpret_cast<const uint4*>(vals);
  }
}

// dX[n][c][h][w] = sum over the (kh, kw) taps whose output position exists of dCol[(c,kh,kw)][n][ho*Wo + wo];
// fp32 accumulation in tap order (kh outer, kw inner), one thread per input pixel, plain store (no atomics).
// grid.x = (n, c) plane, grid.y covers the plane's pixels.  kUnit: stride 1 in both directions (no divisions per tap).
// KS: compile-time square kernel size (0: taken from the geometry).  With unit stride every tap's load is issued
// whether or not the tap exists (from a clamped address, its value then dropped), so that the loads of one pixel do
// not wait for one another: with a branch around each load the kernel ran at the latency of Kh*Kw dependent loads.
template <bool kUnit, int KS>
__global__ void __launch_bounds__(256)
col2im_batched_kernel(const void* __restrict__ dCol, void* __restrict__ dX, const ConvGeom g, const int dt) {
  const int plane = blockIdx.x;
  const int n = plane / g.Cin, c = plane - n * g.Cin;
  const int HW = g.H * g.W;
  const int Kh = KS ? KS : g.Kh, Kw = KS ? KS : g.Kw;
  const long long out_base = static_cast<long long>(plane) * HW;
  const long long row_stride = static_cast<long long>(g.N) * g.HWp;          // from tap k to tap k + 1
  const long long tap0 = (static_cast<long long>(c) * Kh * Kw * g.N + n) * g.HWp;
  for (int pix = blockIdx.y * 256 + threadIdx.x; pix < HW; pix += gridDim.y * 256) {
    const int h = pix / g.W, w = pix - h * g.W;
    float acc = 0.f;
#pragma unroll
    for (int kh = 0; kh < Kh; ++kh) {
      const int hn = h + g.ph - kh * g.dh;
      if constexpr (kUnit) {
        const int ho = hn;
        const bool hok = static_cast<unsigned>(ho) < static_cast<unsigned>(g.Ho);
#pragma unroll 4
        for (int kw = 0; kw < Kw; ++kw) {
          const int wo = w + g.pw - kw * g.dw;
          const bool ok = hok && static_cast<unsigned>(wo) < static_cast<unsigned>(g.Wo);
          const long long idx = ok ? tap0 + (kh * Kw + kw) * row_stride + ho * g.Wo + wo : tap0;
          const float x = load_as_f32(dCol, idx, dt);
          acc += ok ? x : 0.f;
        }
      } else {
        // strided: most taps have no output position for a given pixel (1 in sh*sw does), so they are skipped
        if (hn < 0 || hn % g.sh) continue;
        const int ho = hn / g.sh;
        if (ho >= g.Ho) continue;
        for (int kw = 0; kw < Kw; ++kw) {
          const int wn = w + g.pw - kw * g.dw;
          if (wn < 0 || wn % g.sw) continue;
          const int wo = wn / g.sw;
          if (wo >= g.Wo) continue;
          acc += load_as_f32(dCol, tap0 + (kh * Kw + kw) * row_stride + ho * g.Wo + wo, dt);
        }
      }
    }
    store_from_f32(dX, out_base + pix, dt, acc);
  }
}

// out[i] = sum_n part[n][i] in image order (the exact-fp32 route of the weight gradient: per-image products first,
// then this fixed-order sum).
__global__ void sum_images_kernel(const float* __restrict__ part, float* __restrict__ out, long long elems, int n_img,
                                  int first) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < elems; i += gridDim.x * 256ll) {
    float acc = first ? 0.f : out[i];
    for (int n = 0; n < n_img; ++n) acc += part[static_cast<long long>(n) * elems + i];
    out[i] = acc;
  }
}

// dB[co] = sum_n rows[n * Cout + co]  (rows: per-(image, channel) sums of gZ left by the prologue kernel)
__global__ void fold_db_kernel(const float* __restrict__ rows, float* __restrict__ dB, int N, int Cout) {
  const int co = blockIdx.x * blockDim.x + threadIdx.x;
  if (co >= Cout) return;
  float acc = 0.f;
  for (int n = 0; n < N; ++n) acc += rows[static_cast<long long>(n) * Cout + co];
  dB[co] = acc;
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

bool make_geom(const ge2b_conv2d_params_t& p, ConvGeom& g) {
  g.N = p.N; g.Cin = p.Cin; g.H = p.H; g.W = p.W; g.Cout = p.Cout; g.Kh = p.Kh; g.Kw = p.Kw;
  g.sh = p.stride_h; g.sw = p.stride_w; g.ph = p.pad_h; g.pw = p.pad_w; g.dh = p.dil_h; g.dw = p.dil_w;
  if (g.N <= 0 || g.Cin <= 0 || g.H <= 0 || g.W <= 0 || g.Cout <= 0 || g.Kh <= 0 || g.Kw <= 0) return false;
  if (g.sh <= 0 || g.sw <= 0 || g.dh <= 0 || g.dw <= 0 || g.ph < 0 || g.pw < 0) return false;
  // output size as in conv2d/launcher.cu:137-138
  g.Ho = (g.H + 2 * g.ph - g.dh * (g.Kh - 1) - 1) / g.sh + 1;
  g.Wo = (g.W + 2 * g.pw - g.dw * (g.Kw - 1) - 1) / g.sw + 1;
  if (g.Ho <= 0 || g.Wo <= 0) return false;
  const long long hwo = static_cast<long long>(g.Ho) * g.Wo, k = static_cast<long long>(g.Cin) * g.Kh * g.Kw;
  if (hwo > (1ll << 30) || k > (1ll << 30)) return false;
  g.HWo = static_cast<int>(hwo);
  g.HWp = round_up(g.HWo, 8);
  g.K = static_cast<int>(k);
  return true;
}

// A 1x1 / stride-1 / unpadded convolution reads X[n] (Cin x HW) as its column matrix; taken when the rows of that
// matrix start on 16-byte boundaries (otherwise the padded copy is what lets the tensor-core path run).
bool pointwise(const ConvGeom& g, int esz) {
  return g.Kh == 1 && g.Kw == 1 && g.sh == 1 && g.sw == 1 && g.ph == 0 && g.pw == 0 &&
         (static_cast<long long>(g.H) * g.W * esz) % 16 == 0;
}

cudaError_t launch_im2col(const void* X, void* Col, const ConvGeom& g, int dt, cudaStream_t s) {
  const long long rows = static_cast<long long>(g.K) * g.N;
  const long long blocks = (rows + kColRows - 1) / kColRows;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  const dim3 block(32, kColRows);
  if (dtype_bytes(dt) == 4)
    im2col_batched_kernel<float><<<static_cast<unsigned>(blocks), block, 0, s>>>(
        static_cast<const float*>(X), static_cast<float*>(Col), g, rows);
  else
    im2col_batched_kernel<unsigned short><<<static_cast<unsigned>(blocks), block, 0, s>>>(
        static_cast<const unsigned short*>(X), static_cast<unsigned short*>(Col), g, rows);
  return cudaGetLastError();
}

}  // namespace

namespace {

int dtype_ok(int dt) { return dt == kF32 || dt == kF16 || dt == kBF16; }

// Stream-ordered scratch that frees itself on every return path.
struct AsyncBuf {
  void* p = nullptr;
  cudaStream_t s;
  explicit AsyncBuf(cudaStream_t st) : s(st) {}
  bool alloc(size_t bytes) {
    keep_async_pool_cached();
    return cudaMallocAsync(&p, bytes ? bytes : 16, s) == cudaSuccess;
  }
  ~AsyncBuf() { if (p) cudaFreeAsync(p, s); }
  AsyncBuf(const AsyncBuf&) = delete;
  AsyncBuf& operator=(const AsyncBuf&) = delete;
};

// The OIHW weight is the row-major Cout x K matrix of the GEMMs.  When its rows do not start on 16-byte boundaries
// (K * element size not a multiple of 16, e.g. a 7x7 stem on 3 channels) the tensor-core path could not address it:
// a copy with padded pitch (a few hundred KB at most) keeps those layers on it.  Returns the matrix to use and its
// pitch in elements.
const void* aligned_weight(AsyncBuf& buf, const void* W, const ConvGeom& g, int dtype, int math, long long& ld,
                           cudaStream_t s, bool& failed) {
  const int esz = dtype_bytes(dtype);
  ld = g.K;
  failed = false;
  const bool tensor_path = dtype != kF32 || math == 1;
  if (!tensor_path || (static_cast<long long>(g.K) * esz) % 16 == 0) return W;
  const long long kp = (g.K + 7) / 8 * 8;
  if (!buf.alloc(static_cast<size_t>(g.Cout) * kp * esz) ||
      cudaMemcpy2DAsync(buf.p, kp * esz, W, static_cast<size_t>(g.K) * esz, static_cast<size_t>(g.K) * esz, g.Cout,
                        cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
    failed = true;
    return W;
  }
  ld = kp;
  return buf.p;
}

// GE2B_CONV in the environment picks the route of 16-bit convolutions (read on every call so that one process can
// compare them): "explicit" = column matrix in memory; "gather" = the kernels that gather column tiles from global
// memory, wherever they apply; "general" = the same with their element-wise gather only; unset = by shape: the
// shared-memory patch kernel for unit-stride forward / input-gradient passes, the gathering kernel for the weight
// gradient where its aligned gather applies, the column matrix for the rest.
enum : int { kConvAuto = 0, kConvExplicit = 1, kConvGather = 2, kConvGatherGeneral = 3 };
int conv_route() {
  const char* e = std::getenv("GE2B_CONV");
  if (!e) return kConvAuto;
  if (std::strcmp(e, "explicit") == 0) return kConvExplicit;
  if (std::strcmp(e, "gather") == 0) return kConvGather;
  if (std::strcmp(e, "general") == 0) return kConvGatherGeneral;
  return kConvAuto;
}

// The patch kernel pads the channels of a block to 64 and copies 128 + (Kh-1)*dil_h*Wp + (Kw-1)*dil_w pixels per
// 128 output positions: taken when the padding costs at most twice the arithmetic and the halo at most twice the tile
// (on wide images, e.g. 3 x 3 at 224 x 224, the gathering kernel measured faster).
bool patch_worthwhile(int channels, int kh, int kw, int dh, int dw, int padded_width) {
  const long long halo = static_cast<long long>(kh - 1) * dh * padded_width + static_cast<long long>(kw - 1) * dw;
  return (channels + 63) / 64 * 64 <= 2 * channels && halo <= 256;
}

}  // namespace

int conv2d_forward(const ge2b_conv2d_params_t& p, const void* X, const void* W, const float* bias, void* Y, void* Z,
                   cudaStream_t s) {
  ConvGeom g;
  if (!X || !W || !Y || !dtype_ok(p.dtype) || !make_geom(p, g)) return kBadArgs;
  if (p.groups != 1) return kUnimplemented;
  const int zdt = Z ? p.z_dtype : p.dtype;
  if (Z && !(zdt == p.dtype || zdt == kF32)) return kBadArgs;
  const int esz = dtype_bytes(p.dtype);

  AsyncBuf wpad(s);
  long long ldw = g.K;
  bool failed = false;
  const void* Wm = aligned_weight(wpad, W, g, p.dtype, p.math, ldw, s, failed);
  if (failed) return kCudaError;

  const int route = conv_route();
  const bool sixteen = p.dtype != kF32 && !pointwise(g, esz) && g.Kh * g.Kw <= kConvMaxTaps;
  if (route == kConvAuto && sixteen && g.sh == 1 && g.sw == 1 &&
      patch_worthwhile(g.Cin, g.Kh, g.Kw, g.dh, g.dw, g.W + 2 * g.pw)) {
    // unit stride: operand tiles are windows of one input patch in shared memory
    PatchConv d;
    d.dtype = p.dtype;
    d.X = X; d.img_pitch = static_cast<long long>(g.Cin) * g.H * g.W; d.plane_pitch = static_cast<long long>(g.H) * g.W;
    d.row_pitch = g.W; d.imgs = g.N; d.Cin = g.Cin; d.H = g.H; d.W = g.W;
    d.ph = g.ph; d.pw = g.pw; d.Kh = g.Kh; d.Kw = g.Kw; d.dh = g.dh; d.dw = g.dw;
    d.W_ = W; d.w_row_stride = g.K; d.w_chan_stride = static_cast<long long>(g.Kh) * g.Kw;
    d.Cout = g.Cout;
    d.bias = (bias && p.with_bias) ? bias : nullptr;
    d.act = p.act_kind; d.leaky = p.leaky_slope;
    d.Y = Y; d.Z = Z; d.z_dtype = zdt;
    d.out_img_pitch = static_cast<long long>(g.Cout) * g.HWo;
    AsyncBuf wr(s);
    if (conv_patch_supported(d) && wr.alloc(conv_patch_weight_bytes(d))) {
      d.Wr = wr.p;
      const int rc = conv_patch_launch(d, s);
      if (rc != kUnimplemented) return rc;
    }
  }
  const bool gather_aligned = g.sw == 1 && g.W % 8 == 0 && g.Wo % 8 == 0;
  if (sixteen && (route == kConvGather || route == kConvGatherGeneral || (route == kConvAuto && gather_aligned))) {
    // column tiles gathered from global memory inside the kernel (by shape only where its aligned gather applies:
    // the other shapes measured faster through the column matrix)
    ImplicitConv d;
    d.dtype = p.dtype;
    d.X = X; d.img_pitch = static_cast<long long>(g.Cin) * g.H * g.W; d.plane_pitch = static_cast<long long>(g.H) * g.W;
    d.row_pitch = g.W; d.H = g.H; d.W = g.W;
    d.Ho = g.Ho; d.Wo = g.Wo; d.P = static_cast<long long>(g.N) * g.HWo;
    d.out_img_pitch = static_cast<long long>(g.Cout) * g.HWo;
    d.sh = g.sh; d.sw = g.sw;
    d.taps = g.Kh * g.Kw;
    for (int kh = 0; kh < g.Kh; ++kh)
      for (int kw = 0; kw < g.Kw; ++kw) {
        d.tap_row[kh * g.Kw + kw] = kh * g.dh - g.ph;
        d.tap_col[kh * g.Kw + kw] = kw * g.dw - g.pw;
      }
    d.Wm = Wm; d.ldw = ldw; d.K = g.K; d.Cout = g.Cout;
    d.bias = (bias && p.with_bias) ? bias : nullptr;
    d.act = p.act_kind; d.leaky = p.leaky_slope;
    d.Y = Y; d.Z = Z; d.z_dtype = zdt;
    d.force_general = route == kConvGatherGeneral;
    const int rc = conv_implicit_launch(d, s);
    if (rc != kUnimplemented) return rc;
  }

  AsyncBuf col(s);
  const void* B = X;
  long long ldb = static_cast<long long>(g.H) * g.W, strideB = static_cast<long long>(g.Cin) * g.H * g.W;
  if (!pointwise(g, esz)) {
    if (!col.alloc(static_cast<size_t>(g.K) * g.N * g.HWp * esz)) return kCudaError;
    if (launch_im2col(X, col.p, g, p.dtype, s) != cudaSuccess) return kCudaError;
    B = col.p; ldb = static_cast<long long>(g.N) * g.HWp; strideB = g.HWp;
  }
  DenseForward f;
  f.M = g.Cout; f.N = g.HWo; f.K = g.K; f.batch = g.N;
  f.dtype = p.dtype; f.z_dtype = zdt; f.math = p.math;
  f.A = Wm; f.lda = ldw; f.strideA = 0;                      // the weight is shared by every image
  f.B = B; f.ldb = ldb; f.strideB = strideB;
  f.D = Y; f.ldd = g.HWo; f.strideD = static_cast<long long>(g.Cout) * g.HWo;
  f.Z = Z; f.ldz = g.HWo; f.strideZ = f.strideD;
  f.bias = (bias && p.with_bias) ? bias : nullptr; f.bias_kind = f.bias ? kBiasPerM : kBiasNone;
  f.act = p.act_kind; f.leaky = p.leaky_slope;
  return dense_forward(f, s);
}

int conv2d_backward(const ge2b_conv2d_params_t& p, const void* X, const void* W, const void* dY, const void* Z,
                    void* dW, float* dB, void* dX, cudaStream_t s) {
  ConvGeom g;
  if (!X || !W || !dY || !Z || !dtype_ok(p.dtype) || !make_geom(p, g)) return kBadArgs;
  if (p.groups != 1) return kUnimplemented;
  if (!(p.z_dtype == p.dtype || p.z_dtype == kF32)) return kBadArgs;
  const int esz = dtype_bytes(p.dtype);
  const long long img_rows = static_cast<long long>(g.N) * g.Cout;
  if (img_rows > 0x7fffffffll) return kBadArgs;

  // ---- gZ = dY * act'(Z), rows = (image, channel), columns = output positions; row sums feed dB ----
  AsyncBuf gz(s), rows(s);
  if (!gz.alloc(static_cast<size_t>(img_rows) * g.HWp * esz)) return kCudaError;
  const bool want_db = dB != nullptr;
  if (want_db) {
    if (!rows.alloc(static_cast<size_t>(img_rows) * sizeof(float))) return kCudaError;
    if (cudaMemsetAsync(rows.p, 0, static_cast<size_t>(img_rows) * sizeof(float), s) != cudaSuccess) return kCudaError;
  }
  BwdPrologueArgs pa{};
  pa.M = static_cast<int>(img_rows); pa.N = g.HWo;
  pa.gY = dY; pa.ldgY = g.HWo; pa.gy_dtype = p.dtype;
  pa.Z = Z; pa.ldZ = g.HWo; pa.z_dtype = p.z_dtype;
  pa.gZ = gz.p; pa.ldgZ = g.HWp; pa.gz_dtype = p.dtype;
  pa.gBias = want_db ? static_cast<float*>(rows.p) : nullptr; pa.bias_kind = want_db ? kBiasPerM : kBiasNone;
  pa.act = p.act_kind; pa.leaky = p.leaky_slope;
  if (launch_bwd_prologue(pa, s) != cudaSuccess) return kCudaError;
  if (want_db) {
    fold_db_kernel<<<(g.Cout + 127) / 128, 128, 0, s>>>(static_cast<const float*>(rows.p), dB, g.N, g.Cout);
    if (cudaGetLastError() != cudaSuccess) return kCudaError;
  }
  if (!dW && !dX) return kOk;

  const bool pw = pointwise(g, esz);
  AsyncBuf col(s);
  const long long gz_stride = static_cast<long long>(g.Cout) * g.HWp;
  const void* B = X;
  long long ldb = static_cast<long long>(g.H) * g.W, strideB = static_cast<long long>(g.Cin) * g.H * g.W;
  // the column matrix of the batch (also the home of dCol), taken when a step first needs it
  auto need_col = [&]() {
    if (pw || col.p) return true;
    if (!col.alloc(static_cast<size_t>(g.K) * g.N * g.HWp * esz)) return false;
    B = col.p; ldb = static_cast<long long>(g.N) * g.HWp; strideB = g.HWp;
    return true;
  };

  const int route = conv_route();
  bool dw_done = false;
  const bool sixteen = p.dtype != kF32 && !pw && g.Kh * g.Kw <= kConvMaxTaps;
  // (by shape: where the aligned 16-byte gather applies; other shapes measured faster through the column matrix)
  const bool wgrad_aligned = g.sw == 1 && g.W % 8 == 0 && g.Wo % 8 == 0;
  // (small planes, 14 x 14 and below, also measured faster gathered than through a column matrix of short rows)
  const bool wgrad_gather = wgrad_aligned || g.HWo <= 256;
  if (dW && sixteen && (route == kConvGather || route == kConvGatherGeneral || (route == kConvAuto && wgrad_gather))) {
    // weight gradient with the column tiles gathered inside the kernel (no Col), slices summed in fixed order
    ImplicitWgrad w;
    ImplicitConv& d = w.in;
    d.dtype = p.dtype;
    d.X = X; d.img_pitch = static_cast<long long>(g.Cin) * g.H * g.W; d.plane_pitch = static_cast<long long>(g.H) * g.W;
    d.row_pitch = g.W; d.H = g.H; d.W = g.W;
    d.Ho = g.Ho; d.Wo = g.Wo;
    d.sh = g.sh; d.sw = g.sw;
    d.taps = g.Kh * g.Kw;
    for (int kh = 0; kh < g.Kh; ++kh)
      for (int kw = 0; kw < g.Kw; ++kw) {
        d.tap_row[kh * g.Kw + kw] = kh * g.dh - g.ph;
        d.tap_col[kh * g.Kw + kw] = kw * g.dw - g.pw;
      }
    d.K = g.K; d.Cout = g.Cout;
    d.force_general = route == kConvGatherGeneral;
    w.imgs = g.N; w.G = gz.p; w.g_plane_pitch = g.HWp; w.g_img_pitch = gz_stride;
    w.dW = dW;
    int split = 0; size_t bytes = 0;
    AsyncBuf part(s);
    if (conv_wgrad_plan(w, &split, &bytes) && part.alloc(bytes)) {
      w.part = static_cast<float*>(part.p); w.part_bytes = bytes;
      const int rc = conv_wgrad_launch(w, s);
      if (rc == kOk) dw_done = true;
      else if (rc != kUnimplemented) return rc;
    }
  }

  if (dW && !dw_done) {
    if (!need_col()) return kCudaError;
    if (!pw && launch_im2col(X, col.p, g, p.dtype, s) != cudaSuccess) return kCudaError;
    // dW (Cout x K) = sum_n gZ[n] (Cout x HWo) . Col[n]^T (HWo x K)
    GemmProblem q{};
    q.M = g.Cout; q.N = g.K; q.K = g.HWo; q.batch = g.N;
    q.in_dtype = p.dtype; q.math = p.math;
    q.a_mn = false; q.b_mn = false;                            // both operands have the reduction index contiguous
    q.A = gz.p; q.lda = g.HWp; q.strideA = gz_stride;
    q.B = B; q.ldb = ldb; q.strideB = strideB;
    q.reduce_batch = true;
    q.epi.D = dW; q.epi.ldd = g.K; q.epi.d_dtype = p.dtype; q.epi.z_dtype = p.dtype;
    q.epi.alpha = 1.f; q.epi.act = kActNone; q.epi.bias_kind = kBiasNone;
    int rc = run_gemm_problem(q, s);
    if (rc == kUnimplemented) {
      // Route without the batch-reducing kernel (exact fp32, or a pitch TMA cannot address): the images' products
      // as ONE batched launch into a scratch [group][Cout][K], then a sum over the group in image order; groups keep
      // the scratch under 256 MiB.  fp32 tensors only (a 16-bit scratch would round the partial sums).
      if (p.dtype == kF32) {
        const long long elems = static_cast<long long>(g.Cout) * g.K;
        long long group = (256ll << 20) / (elems * 4);
        if (group < 1) group = 1;
        if (group > g.N) group = g.N;
        AsyncBuf part(s);
        if (!part.alloc(static_cast<size_t>(group) * elems * 4)) return kCudaError;
        for (int n0 = 0; n0 < g.N; n0 += static_cast<int>(group)) {
          const int cnt = static_cast<int>(std::min<long long>(group, g.N - n0));
          DenseForward f;
          f.M = g.Cout; f.N = g.K; f.K = g.HWo; f.batch = cnt;
          f.dtype = p.dtype; f.z_dtype = p.dtype; f.math = p.math;
          f.trans_b = true;
          f.A = static_cast<const uint8_t*>(gz.p) + static_cast<size_t>(n0) * gz_stride * esz; f.lda = g.HWp; f.strideA = gz_stride;
          f.B = static_cast<const uint8_t*>(B) + static_cast<size_t>(n0) * strideB * esz; f.ldb = ldb; f.strideB = strideB;
          f.D = part.p; f.ldd = g.K; f.strideD = elems;
          rc = dense_forward(f, s);
          if (rc != kOk) return rc;
          long long blocks = (elems + 255) / 256;
          if (blocks > 4096) blocks = 4096;
          sum_images_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const float*>(part.p),
                                                                        static_cast<float*>(dW), elems, cnt, n0 == 0);
          if (cudaGetLastError() != cudaSuccess) return kCudaError;
        }
      } else {
      // 16-bit tensors whose pitch TMA cannot address: one launch per image, accumulating into dW
      for (int n = 0; n < g.N; ++n) {
        DenseForward f;
        f.M = g.Cout; f.N = g.K; f.K = g.HWo; f.batch = 1;
        f.dtype = p.dtype; f.z_dtype = p.dtype; f.math = p.math;
        f.trans_b = true;
        f.A = static_cast<const uint8_t*>(gz.p) + static_cast<size_t>(n) * gz_stride * esz; f.lda = g.HWp;
        f.B = static_cast<const uint8_t*>(B) + static_cast<size_t>(n) * strideB * esz; f.ldb = ldb;
        f.C = dW; f.ldc = g.K; f.beta = n > 0 ? 1.f : 0.f;
        f.D = dW; f.ldd = g.K;
        rc = dense_forward(f, s);
        if (rc != kOk) return rc;
      }
      }
    } else if (rc != kOk) {
      return rc;
    }
  }

  bool dx_done = false;
  // (1 x 1 layers measured faster through the batched GEMM: their dCol is dX itself or one small copy)
  if (dX && sixteen && route == kConvAuto && g.sh == 1 && g.sw == 1 && g.Kh * g.Kw > 1 && g.Cin >= 16 &&
      g.ph <= (g.Kh - 1) * g.dh && g.pw <= (g.Kw - 1) * g.dw &&
      patch_worthwhile(g.Cout, g.Kh, g.Kw, g.dh, g.dw, g.Wo + 2 * ((g.Kw - 1) * g.dw - g.pw))) {
    // Input gradient of a unit-stride convolution = convolution of gZ (border dil*(K-1) - pad) with the taps mirrored
    // and the weight read as [Cin][tap][Cout]: the patch kernel again, no dCol and no col2im.
    PatchConv d;
    d.dtype = p.dtype;
    d.X = gz.p; d.img_pitch = gz_stride; d.plane_pitch = g.HWp; d.row_pitch = g.Wo;
    d.imgs = g.N; d.Cin = g.Cout; d.H = g.Ho; d.W = g.Wo;
    d.ph = (g.Kh - 1) * g.dh - g.ph; d.pw = (g.Kw - 1) * g.dw - g.pw;
    d.Kh = g.Kh; d.Kw = g.Kw; d.dh = g.dh; d.dw = g.dw;
    d.W_ = W; d.w_row_stride = static_cast<long long>(g.Kh) * g.Kw; d.w_chan_stride = g.K; d.flip_taps = true;
    d.Cout = g.Cin;
    d.Y = dX;
    d.out_img_pitch = static_cast<long long>(g.Cin) * g.H * g.W;
    AsyncBuf wr(s);
    if (conv_patch_supported(d) && wr.alloc(conv_patch_weight_bytes(d))) {
      d.Wr = wr.p;
      const int rc = conv_patch_launch(d, s);
      if (rc == kOk) dx_done = true;
      else if (rc != kUnimplemented) return rc;
    }
  }
  // (not for layers with a handful of input channels, e.g. an RGB stem: the kernel's narrowest output tile is 64 wide)
  if (dX && !dx_done && sixteen && route == kConvAuto && (g.sh > 1 || g.sw > 1) && g.sh <= 4 && g.sw <= 4 &&
      (g.Cout + 63) / 64 * 64 <= 2 * g.Cout && g.Cin >= 16) {
    // Strided convolution: the input pixels (h, w) with h % sh == a and w % sw == b receive only the taps with
    // (a + ph - kh*dh) % sh == 0 and (b + pw - kw*dw) % sw == 0, and for those dX[a + sh*i][b + sw*j] is a UNIT-stride
    // correlation of gZ: sum of gZ[i + (a + ph - kh*dh)/sh][j + (b + pw - kw*dw)/sw] . W[.., kh, kw].  One patch-kernel
    // launch per phase (a, b), each writing its own pixels of dX; no dCol, no col2im.
    struct Phase { PatchConv d; bool empty; };
    std::vector<Phase> phases;
    bool all_ok = true, any_empty = false;
    for (int a = 0; a < g.sh && all_ok; ++a)
      for (int b = 0; b < g.sw && all_ok; ++b) {
        Phase ph{};
        PatchConv& d = ph.d;
        const int Hph = (g.H - a + g.sh - 1) / g.sh, Wph = (g.W - b + g.sw - 1) / g.sw;
        if (Hph <= 0 || Wph <= 0) continue;
        int qh[kConvMaxTaps], qw[kConvMaxTaps], kh_of[kConvMaxTaps], kw_of[kConvMaxTaps], nh = 0, nw = 0;
        for (int kh = 0; kh < g.Kh; ++kh) {
          const int num = a + g.ph - kh * g.dh;
          if (((num % g.sh) + g.sh) % g.sh == 0) { qh[nh] = (num - (((num % g.sh) + g.sh) % g.sh)) / g.sh; kh_of[nh++] = kh; }
        }
        for (int kw = 0; kw < g.Kw; ++kw) {
          const int num = b + g.pw - kw * g.dw;
          if (((num % g.sw) + g.sw) % g.sw == 0) { qw[nw] = (num - (((num % g.sw) + g.sw) % g.sw)) / g.sw; kw_of[nw++] = kw; }
        }
        ph.empty = nh == 0 || nw == 0;
        any_empty = any_empty || ph.empty;
        if (!ph.empty) {
          int top = 0, left = 0;                       // zero border so that every tap offset is >= 0
          for (int i = 0; i < nh; ++i) top = std::max(top, -qh[i]);
          for (int i = 0; i < nw; ++i) left = std::max(left, -qw[i]);
          int max_tc = 0;
          d.n_taps = nh * nw;
          for (int i = 0; i < nh; ++i)
            for (int j = 0; j < nw; ++j) {
              const int t = i * nw + j;
              d.tap_r[t] = qh[i] + top; d.tap_c[t] = qw[j] + left;
              d.tap_src[t] = kh_of[i] * g.Kw + kw_of[j];
              max_tc = std::max(max_tc, d.tap_c[t]);
            }
          d.dtype = p.dtype;
          d.X = gz.p; d.img_pitch = gz_stride; d.plane_pitch = g.HWp; d.row_pitch = g.Wo;
          d.imgs = g.N; d.Cin = g.Cout; d.H = g.Ho; d.W = g.Wo;
          d.ph = top; d.pw = left;
          d.Wp = std::max(g.Wo + left, Wph + max_tc);
          d.out_H = Hph; d.out_W = Wph;
          d.W_ = W; d.w_row_stride = static_cast<long long>(g.Kh) * g.Kw; d.w_chan_stride = g.K;
          d.Cout = g.Cin;
          d.Y = dX;
          d.out_img_pitch = static_cast<long long>(g.Cin) * g.H * g.W;
          d.out_plane = static_cast<long long>(g.H) * g.W; d.out_row_pitch = g.W;
          d.osh = g.sh; d.osw = g.sw; d.out_off = a * g.W + b;
          all_ok = conv_patch_supported(d);
        }
        phases.push_back(ph);
      }
    if (all_ok && !phases.empty()) {
      size_t wbytes = 0;
      for (const Phase& ph : phases) if (!ph.empty) wbytes = std::max(wbytes, conv_patch_weight_bytes(ph.d));
      AsyncBuf wr(s);
      if (wr.alloc(wbytes)) {
        // pixels of a phase without taps (kernel smaller than the stride) get no contribution at all
        if (any_empty && cudaMemsetAsync(dX, 0, static_cast<size_t>(g.N) * g.Cin * g.H * g.W * esz, s) != cudaSuccess)
          return kCudaError;
        dx_done = true;
        for (Phase& ph : phases) {
          if (ph.empty) continue;
          ph.d.Wr = wr.p;
          const int rc = conv_patch_launch(ph.d, s);
          if (rc != kOk) return rc == kUnimplemented ? kCudaError : rc;
        }
      }
    }
  }

  // (gZ rows are Wo wide and dX rows W wide: the aligned gather needs both to be multiples of 8)
  if (dX && !dx_done && sixteen && g.sh == 1 && g.sw == 1 &&
      (route == kConvGather || route == kConvGatherGeneral || (route == kConvAuto && wgrad_aligned))) {
    // the same through the gathering kernel
    const int taps = g.Kh * g.Kw;
    const long long kt = static_cast<long long>(g.Cout) * taps, ldt = (kt + 7) / 8 * 8;
    AsyncBuf wt(s);
    if (kt <= (1 << 24) && wt.alloc(static_cast<size_t>(g.Cin) * ldt * esz) &&
        launch_transpose_weight(W, wt.p, g.Cout, g.Cin, taps, ldt, s) == cudaSuccess) {
      ImplicitConv d;
      d.dtype = p.dtype;
      d.X = gz.p; d.img_pitch = gz_stride; d.plane_pitch = g.HWp; d.row_pitch = g.Wo; d.H = g.Ho; d.W = g.Wo;
      d.Ho = g.H; d.Wo = g.W; d.P = static_cast<long long>(g.N) * g.H * g.W;
      d.out_img_pitch = static_cast<long long>(g.Cin) * g.H * g.W;
      d.sh = 1; d.sw = 1;
      d.taps = taps;
      for (int kh = 0; kh < g.Kh; ++kh)
        for (int kw = 0; kw < g.Kw; ++kw) {
          d.tap_row[kh * g.Kw + kw] = g.ph - kh * g.dh;
          d.tap_col[kh * g.Kw + kw] = g.pw - kw * g.dw;
        }
      d.Wm = wt.p; d.ldw = ldt; d.K = static_cast<int>(kt); d.Cout = g.Cin;
      d.Y = dX;
      d.force_general = route == kConvGatherGeneral;
      const int rc = conv_implicit_launch(d, s);
      if (rc == kOk) dx_done = true;
      else if (rc != kUnimplemented) return rc;
    }
  }

  if (dX && !dx_done) {
    // dCol[n] (K x HWo) = W^T (K x Cout) . gZ[n] (Cout x HWo); for a pointwise convolution dCol[n] is dX[n]
    if (!need_col()) return kCudaError;
    DenseForward f;
    f.M = g.K; f.N = g.HWo; f.K = g.Cout; f.batch = g.N;
    f.dtype = p.dtype; f.z_dtype = p.dtype; f.math = p.math;
    f.trans_a = true;                                          // W is stored Cout x K: reduction index outermost
    AsyncBuf wpad(s);
    long long ldw = g.K;
    bool failed = false;
    f.A = aligned_weight(wpad, W, g, p.dtype, p.math, ldw, s, failed);
    if (failed) return kCudaError;
    f.lda = ldw; f.strideA = 0;
    f.B = gz.p; f.ldb = g.HWp; f.strideB = gz_stride;
    if (pw) { f.D = dX; f.ldd = g.HWo; f.strideD = static_cast<long long>(g.Cin) * g.HWo; }
    else    { f.D = col.p; f.ldd = static_cast<long long>(g.N) * g.HWp; f.strideD = g.HWp; }
    const int rc = dense_forward(f, s);
    if (rc != kOk) return rc;
    if (!pw) {
      const long long planes = static_cast<long long>(g.N) * g.Cin;
      if (planes > 0x7fffffffll) return kBadArgs;
      int gy = (g.H * g.W + 255) / 256;
      if (gy > 4096) gy = 4096;
      const dim3 grid(static_cast<unsigned>(planes), gy);
      const bool unit = g.sh == 1 && g.sw == 1;
      // compile-time kernel sizes pay off only in the unit-stride form (all taps unrolled, loads in flight together)
      const int ks = (unit && g.Kh == g.Kw && (g.Kh == 3 || g.Kh == 5 || g.Kh == 7)) ? g.Kh : 0;
#define GE2B_COL2IM(KS_)                                                                              \
      do {                                                                                            \
        if (unit) col2im_batched_kernel<true, KS_><<<grid, 256, 0, s>>>(col.p, dX, g, p.dtype);       \
        else      col2im_batched_kernel<false, KS_><<<grid, 256, 0, s>>>(col.p, dX, g, p.dtype);      \
      } while (0)
      switch (ks) {
        case 3:  GE2B_COL2IM(3); break;
        case 5:  GE2B_COL2IM(5); break;
        case 7:  GE2B_COL2IM(7); break;
        default: GE2B_COL2IM(0); break;
      }
#undef GE2B_COL2IM
      if (cudaGetLastError() != cudaSuccess) return kCudaError;
    }
  }
  return kOk;
}

}  // namespace ge2b

extern "C" {

int ge2b_conv2d_forward(const ge2b_conv2d_params_t* p, const void* X, const void* W, const float* bias, void* Y, void* Z,
                        void* stream) {
  if (!p) return ge2b::kBadArgs;
  return ge2b::conv2d_forward(*p, X, W, bias, Y, (p->save_z ? Z : nullptr), reinterpret_cast<cudaStream_t>(stream));
}

int ge2b_conv2d_backward(const ge2b_conv2d_params_t* p, const void* X, const void* W, const void* dY, const void* Z,
                         void* dW, float* dB, void* dX, void* stream) {
  if (!p) return ge2b::kBadArgs;
  return ge2b::conv2d_backward(*p, X, W, dY, Z, dW, dB, dX, reinterpret_cast<cudaStream_t>(stream));
}

int ge2b_conv2d_output_size(const ge2b_conv2d_params_t* p, int* Ho, int* Wo) {
  ge2b::ConvGeom g;
  if (!p || !ge2b::make_geom(*p, g)) return ge2b::kBadArgs;
  if (Ho) *Ho = g.Ho;
  if (Wo) *Wo = g.Wo;
  return ge2b::kOk;
}

}  // extern "C"

// ---- C++ operator API (validation order and Status codes of conv2d/launcher.cu:115-158, 236-280) ----
namespace ai {
namespace {

namespace shim = cuda::shim;

bool is4(const Tensor& t, shim::DType dt) {
  return t.device == shim::Device::CUDA && t.desc.dtype == dt && t.desc.layout == shim::Layout::RowMajor &&
         t.desc.shape.size() == 4;
}
bool float_dtype(shim::DType d) { return d == shim::DType::F32 || d == shim::DType::F16 || d == shim::DType::BF16; }
bool shape_is(const Tensor& t, std::int64_t a, std::int64_t b, std::int64_t c, std::int64_t d) {
  return t.desc.shape[0] == a && t.desc.shape[1] == b && t.desc.shape[2] == c && t.desc.shape[3] == d;
}
Status from_rc(int rc) {
  switch (rc) {
    case ge2b::kOk:            return Status::Ok;
    case ge2b::kBadArgs:       return Status::Invalid;
    case ge2b::kUnimplemented: return Status::Unimplemented;
    default:                   return Status::CUDA_ERROR;
  }
}
bool fill_params(const Tensor& X, const Tensor& W, const Conv2DAttrs& a, ge2b_conv2d_params_t& p) {
  for (int i = 0; i < 4; ++i)
    if (X.desc.shape[i] <= 0 || X.desc.shape[i] > 0x7fffffff || W.desc.shape[i] <= 0 || W.desc.shape[i] > 0x7fffffff)
      return false;
  p.N = static_cast<int>(X.desc.shape[0]); p.Cin = static_cast<int>(X.desc.shape[1]);
  p.H = static_cast<int>(X.desc.shape[2]); p.W = static_cast<int>(X.desc.shape[3]);
  p.Cout = static_cast<int>(W.desc.shape[0]); p.Kh = static_cast<int>(W.desc.shape[2]); p.Kw = static_cast<int>(W.desc.shape[3]);
  p.stride_h = a.stride_h; p.stride_w = a.stride_w; p.pad_h = a.pad_h; p.pad_w = a.pad_w; p.dil_h = a.dil_h; p.dil_w = a.dil_w;
  p.groups = a.groups;
  p.act_kind = static_cast<int>(a.act); p.leaky_slope = a.leaky_slope;
  p.with_bias = a.with_bias ? 1 : 0; p.save_z = a.save_z ? 1 : 0;
  p.dtype = static_cast<int>(X.desc.dtype); p.z_dtype = p.dtype;
  p.math = (X.desc.dtype == shim::DType::F32) ? ge2b::default_fp32_math() : 1;
  return true;
}

}  // namespace

Status Conv2DCudaLaunch(const Tensor& X, const Tensor& W, const Tensor* B, Tensor& Y, const Conv2DAttrs& a,
                        StreamHandle stream, Tensor* Z_saved, const Conv2DWorkspaceFwd* /*ws_fwd*/) {
  const shim::DType dt = X.desc.dtype;
  if (!float_dtype(dt) || !is4(X, dt) || !is4(Y, dt)) return Status::Invalid;
  if (!is4(W, dt)) return Status::Invalid;
  if (a.groups != 1) return Status::Unimplemented;
  if (W.desc.shape[1] != X.desc.shape[1]) return Status::ShapeMismatch;
  ge2b_conv2d_params_t p{};
  if (!fill_params(X, W, a, p)) return Status::Invalid;
  if (a.stride_h <= 0 || a.stride_w <= 0) return Status::Invalid;
  // output size and the order of the two checks as in conv2d/launcher.cu:137-146
  const int Ho = (p.H + 2 * p.pad_h - p.dil_h * (p.Kh - 1) - 1) / p.stride_h + 1;
  const int Wo = (p.W + 2 * p.pad_w - p.dil_w * (p.Kw - 1) - 1) / p.stride_w + 1;
  if (!shape_is(Y, p.N, p.Cout, Ho, Wo)) return Status::ShapeMismatch;
  if (Ho <= 0 || Wo <= 0 || ge2b_conv2d_output_size(&p, nullptr, nullptr) != 0) return Status::Invalid;
  const bool want_z = a.save_z && Z_saved != nullptr;
  if (want_z) {
    const shim::DType zdt = Z_saved->desc.dtype;
    if (!(zdt == dt || zdt == shim::DType::F32) || !is4(*Z_saved, zdt)) return Status::Invalid;
    if (!shape_is(*Z_saved, p.N, p.Cout, Ho, Wo)) return Status::ShapeMismatch;
    p.z_dtype = static_cast<int>(zdt);
  }
  p.save_z = want_z ? 1 : 0;
  const float* bias = (B && B->data && a.with_bias) ? static_cast<const float*>(B->data) : nullptr;
  if (bias && B->desc.dtype != shim::DType::F32) return Status::Invalid;
  p.with_bias = bias ? 1 : 0;
  return from_rc(ge2b_conv2d_forward(&p, X.data, W.data, bias, Y.data, want_z ? Z_saved->data : nullptr, stream));
}

Status Conv2DCudaBackwardLaunch(const Tensor& X, const Tensor& W, const Tensor& dY, const Tensor& Z, Tensor* dW,
                                Tensor* dB, Tensor* dX, const Conv2DAttrs& a, StreamHandle stream,
                                const Conv2DWorkspaceBwd* /*ws_bwd*/) {
  const shim::DType dt = X.desc.dtype;
  const shim::DType zdt = Z.desc.dtype;
  if (!float_dtype(dt) || !is4(X, dt) || !is4(W, dt) || !is4(dY, dt) || !(zdt == dt || zdt == shim::DType::F32) ||
      !is4(Z, zdt))
    return Status::Invalid;
  if (a.groups != 1) return Status::Unimplemented;
  if (W.desc.shape[1] != X.desc.shape[1]) return Status::ShapeMismatch;
  ge2b_conv2d_params_t p{};
  if (!fill_params(X, W, a, p)) return Status::Invalid;
  p.z_dtype = static_cast<int>(zdt);
  if (a.stride_h <= 0 || a.stride_w <= 0) return Status::Invalid;
  const int Ho = (p.H + 2 * p.pad_h - p.dil_h * (p.Kh - 1) - 1) / p.stride_h + 1;
  const int Wo = (p.W + 2 * p.pad_w - p.dil_w * (p.Kw - 1) - 1) / p.stride_w + 1;
  const bool geom_ok = Ho > 0 && Wo > 0 && ge2b_conv2d_output_size(&p, nullptr, nullptr) == 0;
  if (!shape_is(dY, p.N, p.Cout, Ho, Wo) || !shape_is(Z, p.N, p.Cout, Ho, Wo)) return Status::ShapeMismatch;
  if (dW && (!is4(*dW, dt) || !shape_is(*dW, p.Cout, p.Cin, p.Kh, p.Kw))) return Status::ShapeMismatch;
  if (dB && !(dB->device == shim::Device::CUDA && dB->desc.dtype == shim::DType::F32 && dB->desc.shape.size() == 1 &&
              dB->desc.shape[0] == p.Cout))
    return Status::ShapeMismatch;
  if (dX && (!is4(*dX, dt) || !shape_is(*dX, p.N, p.Cin, p.H, p.W))) return Status::ShapeMismatch;
  if (!geom_ok) return Status::Invalid;
  // the bias gradient is produced only when the layer has a bias (launcher.cu:412-418)
  float* db = (dB && a.with_bias) ? static_cast<float*>(dB->data) : nullptr;
  return from_rc(ge2b_conv2d_backward(&p, X.data, W.data, dY.data, Z.data, dW ? dW->data : nullptr, db,
                                      dX ? dX->data : nullptr, stream));
}

}  // namespace ai
