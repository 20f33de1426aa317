// C++ operator API of the dense-layer path, source- and link-compatible with the reference's
// `ai::cuda::shim` GEMM op so that its callers (the pybind module of src/bindings/gemm_pybind.cpp, the conv2d
// and rnn launchers) can be linked against libge2_b200.so unchanged.
//
// The types below are declared in the same namespace, with the same member order and the same enumerator
// values as the reference's headers, because they cross the library boundary by reference:
//   Status                 backends/cuda/ops/_common/shim/ai_status.hpp:14-39
//   Device, DType, Layout  backends/cuda/ops/_common/shim/ai_device.hpp:14-16
//   ActKind, BiasKind      backends/cuda/ops/_common/shim/enums.hpp:10-24
//   TensorDesc, Tensor     backends/cuda/ops/_common/shim/ai_tensor.hpp:13-63
//   GemmAttrs              backends/cuda/ops/_common/shim/ai_ops_base.hpp:9-18
//   GemmWorkspace          backends/cuda/ops/gemm/api.hpp:97-104
//   GemmCudaLaunch / GemmCudaBackward / GemmCudaBackwardInto   backends/cuda/ops/gemm/api.hpp:124-188
// Do not include this header together with the reference's own headers in one translation unit.
//
// Behaviour kept from the reference launcher (backends/cuda/ops/gemm/launcher.cu:147-383): order of the
// validation checks and the Status each returns; Z may alias Y; bias kind inferred from the bias tensor's
// shape; attrs.alpha / attrs.beta are accepted and ignored (alpha = 1, beta = 0 unless C and gC are given).
// Added: every tensor of a call may be BF16 or F16 instead of F32 (bias and bias gradient stay F32, Z may be
// F32 or the operand dtype); those calls run on the tcgen05 kernels.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

struct CUstream_st;

namespace ai::cuda::shim {

enum class Status : int {
  Ok = 0,
  Invalid = 1, Unimplemented = 2, RuntimeError = 3, InvalidArgument = 4,
  MissingInput = 10, MissingOutput = 11,
  DeviceMismatch = 100, DtypeMismatch = 101, LayoutMismatch = 102, ShapeMismatch = 103, StrideMismatch = 104,
  TransposeNotSupported = 105,
  CUDA_ERROR = 130,
  Unknown = 999
};

enum class Device : int { CPU = 0, CUDA = 1 };
enum class DType : int { F32 = 0, F16 = 1, BF16 = 2, I32 = 3, I8 = 4 };
enum class Layout : int { RowMajor = 0, ColMajor = 1 };
enum class ActKind : int { None = 0, ReLU = 1, LeakyReLU = 2, GELU = 3, Sigmoid = 4, Tanh = 5 };
enum class BiasKind : int { None = 0, Scalar = 1, PerM = 2, PerN = 3 };

struct TensorDesc {
  DType dtype{DType::F32};
  Layout layout{Layout::RowMajor};
  std::vector<std::int64_t> shape;
  std::vector<std::int64_t> stride;   // in elements
};

// Non-owning view of device memory.
struct Tensor {
  void* data{nullptr};
  TensorDesc desc{};
  Device device{Device::CUDA};
  int device_index{0};
};

struct GemmAttrs {
  bool trans_a{false};
  bool trans_b{false};
  ActKind act{ActKind::None};
  bool with_bias{false};
  float leaky_slope{0.01f};
  bool save_z{false};
  float alpha{1.0f};
  float beta{0.0f};
};

struct alignas(256) GemmWorkspace {
  void* lt_workspace = nullptr;          // 256-byte aligned; lent to the launch for split-K partial sums when >= 2 MiB
  std::size_t lt_workspace_bytes = 0;
  void* scratch = nullptr;               // gZ of the backward pass, row-major with ld = N
  std::size_t scratch_bytes = 0;         // 0 = not stated
};

using StreamHandle = CUstream_st*;

inline Tensor make_tensor2d(void* ptr, std::int64_t rows, std::int64_t cols, DType dt = DType::F32) {
  Tensor t;
  t.data = ptr;
  t.desc.dtype = dt;
  t.desc.shape = {rows, cols};
  t.desc.stride = {cols, 1};
  return t;
}

constexpr std::size_t GemmRequiredBackwardScratchBytes(std::int64_t M, std::int64_t N) noexcept {
  return (M <= 0 || N <= 0) ? 0 : static_cast<std::size_t>(M) * static_cast<std::size_t>(N) * sizeof(float);
}

// ---- parameter blocks of the layer below the Tensor API (backends/cuda/ops/gemm/api.hpp:19-93); the legacy C ABI
//      adapters fill these and call the three functions declared after them.  fp32, row-major, device pointers. ----
struct GemmBiasActParams {
  int M, N, K;
  const void* A; int lda;
  const void* B; int ldb;
  const void* C; int ldc;           // optional addend, used when beta != 0
  void* D; int ldd;
  float alpha, beta;                // D = act(alpha * A.B + beta * C + bias)
  const void* bias;
  BiasKind bias_kind;
  ActKind act;
  float leaky_slope;
};

struct GemmBiasActParamsEx {
  int M, N, K;
  const void* A; int lda;
  const void* B; int ldb;
  const void* C; int ldc;
  void* D; int ldd;
  float alpha, beta;
  const void* bias;
  BiasKind bias_kind;
  ActKind act;
  float leaky_slope;
  void* Z; int ldZ;                 // pre-activation stash; ldZ == 0 means ldd
  int save_preact;
  void* lt_workspace{nullptr};      // carried, unused
  std::size_t lt_workspace_bytes{0};
};

struct GemmBiasActBwdParams {
  int M, N, K;
  const void* A; int lda;
  const void* B; int ldb;
  const void* C; int ldc;
  const void* Z; int ldZ;
  const void* gY; int ldgY;
  void* gA; int ldgA;
  void* gB; int ldgB;
  void* gC; int ldgC;
  void* gBias;
  float* gZ_scratch; int ldgZ;      // row-major with ld = N; null: stream-ordered allocation
  float alpha{1.f};
  float beta{0.f};
  BiasKind bias_kind{BiasKind::None};
  ActKind act{ActKind::None};
  float leaky_slope{0.01f};
  void* lt_workspace{nullptr};
  std::size_t lt_workspace_bytes{0};
};

// Replace regemm_gemm_bias_act.cu:516-526 and regemm_backward.cu:151-301.  As in the reference they return nothing;
// launch errors surface through cudaGetLastError(), and the backward throws std::invalid_argument on bad sizes
// or null gY / Z.
void gemm_bias_act_f32(const GemmBiasActParams& p, CUstream_st* stream);
void gemm_bias_act_f32_ex(const GemmBiasActParamsEx& p, CUstream_st* stream);
void gemm_bias_act_bwd_f32(const GemmBiasActBwdParams& p, CUstream_st* stream);
void launch_gemm_bias_act_f32_smoke_ex(const GemmBiasActParamsEx& p, CUstream_st* stream);

// Y[M,N] = act(A[M,K] . B[K,N] + bias); with attrs.save_z the pre-activation is written to *Z_saved.
Status GemmCudaLaunch(const Tensor& A, const Tensor& B, const Tensor* Bias, Tensor& Y, const GemmAttrs& attrs,
                      StreamHandle stream, Tensor* Z_saved = nullptr, const GemmWorkspace* ws = nullptr);

inline Status GemmCudaLaunch(const Tensor& A, const Tensor& B, Tensor& Y, const GemmAttrs& attrs, StreamHandle stream,
                             Tensor* Z_saved = nullptr, const GemmWorkspace* ws = nullptr) {
  return GemmCudaLaunch(A, B, nullptr, Y, attrs, stream, Z_saved, ws);
}

// (A, B, C, gY, Z) -> (gA, gB, gC, gBias); any output may be null.  With ws->scratch nothing is allocated.
Status GemmCudaBackward(const Tensor& A, const Tensor& B, const Tensor* C, const Tensor& gY, const Tensor& Z,
                        Tensor* gA, Tensor* gB, Tensor* gC, Tensor* gBias, const GemmAttrs& attrs, StreamHandle stream,
                        const GemmWorkspace* ws = nullptr);

inline Status GemmCudaBackwardInto(const Tensor& A, const Tensor& B, const Tensor* C, const Tensor& gY,
                                   const Tensor& Z, Tensor* gA, Tensor* gB, Tensor* gC, Tensor* gBias,
                                   const GemmAttrs& attrs, StreamHandle stream, float* dZ, void* lt_ws = nullptr,
                                   std::size_t lt_ws_bytes = 0) {
  GemmWorkspace ws{};
  ws.scratch = dZ;
  ws.scratch_bytes = 0;
  ws.lt_workspace = lt_ws;
  ws.lt_workspace_bytes = lt_ws_bytes;
  return GemmCudaBackward(A, B, C, gY, Z, gA, gB, gC, gBias, attrs, stream, &ws);
}

}  // namespace ai::cuda::shim

// Registry-style function-pointer signatures of the reference's dispatch table
// (graph_executor_v2/include/ai/dispatch.hpp:9-111).
namespace ge2b {
using KernelFn = ai::cuda::shim::Status (*)(const ai::cuda::shim::Tensor&, const ai::cuda::shim::Tensor&,
                                            const ai::cuda::shim::Tensor*, ai::cuda::shim::Tensor&,
                                            const ai::cuda::shim::GemmAttrs&, ai::cuda::shim::StreamHandle,
                                            ai::cuda::shim::Tensor*);
using GemmBwdFn = ai::cuda::shim::Status (*)(const ai::cuda::shim::Tensor&, const ai::cuda::shim::Tensor&,
                                             const ai::cuda::shim::Tensor*, const ai::cuda::shim::Tensor&,
                                             const ai::cuda::shim::Tensor&, ai::cuda::shim::Tensor*,
                                             ai::cuda::shim::Tensor*, ai::cuda::shim::Tensor*,
                                             ai::cuda::shim::Tensor*, const ai::cuda::shim::GemmAttrs&,
                                             ai::cuda::shim::StreamHandle);
KernelFn gemm_forward_kernel_fn();     // entry suitable for OpRegistry::reg
GemmBwdFn gemm_backward_kernel_fn();   // entry suitable for BwdOpRegistry::reg
}  // namespace ge2b
