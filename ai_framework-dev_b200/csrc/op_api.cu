// ai::cuda::shim::GemmCudaLaunch / GemmCudaBackward over the B200 kernels.
// Validation order and Status codes follow backends/cuda/ops/gemm/launcher.cu:147-383 of the reference;
// the kernels behind it are this library's.
#include <cuda_runtime.h>

#include <limits>
#include <stdexcept>

#include "../../include/ge2_op_api.hpp"
#include "dense_ops.hpp"

namespace ai::cuda::shim {
namespace {

using ge2b::kBiasNone;
using ge2b::kBiasPerM;
using ge2b::kBiasPerN;
using ge2b::kBiasScalar;

bool float_dtype(DType d) { return d == DType::F32 || d == DType::F16 || d == DType::BF16; }

// Reference rule: CUDA, row-major, rank 2, fp32 (ai_validate.hpp:137-142); here also f16 / bf16.
bool is_cuda_rowmajor_2d(const Tensor& t, DType want) {
  return t.device == Device::CUDA && t.desc.dtype == want && t.desc.layout == Layout::RowMajor &&
         t.desc.shape.size() == 2;
}

// stride[0] when positive, otherwise the row length (tensor_layout.hpp:12-19).
std::int64_t infer_ld(const Tensor& t) {
  if (t.desc.shape.size() != 2) return 0;
  if (t.desc.stride.size() >= 2 && t.desc.stride[0] > 0) return t.desc.stride[0];
  return t.desc.shape[1];
}

bool fits_i32(std::int64_t v) { return v >= 0 && v <= std::numeric_limits<int>::max(); }

// Bias kind from the tensor's shape: 1-D length 1 / N / M first, then (1,N), (M,1), (1,1), then element count
// (launcher.cu:47-77, bias.hpp:69-78).
int decide_bias_kind(const Tensor* b, std::int64_t M, std::int64_t N) {
  if (!b || !b->data) return kBiasNone;
  const auto& s = b->desc.shape;
  if (s.size() == 1) {
    if (s[0] == 1) return kBiasScalar;
    if (s[0] == N) return kBiasPerN;
    if (s[0] == M) return kBiasPerM;
  }
  std::int64_t numel = 1;
  for (auto v : s) {
    if (v < 0) return kBiasNone;
    numel *= v;
  }
  if (numel == 0) return kBiasNone;
  if (s.size() == 2 && s[0] == 1 && s[1] == N) return kBiasPerN;
  if (s.size() == 2 && s[0] == M && s[1] == 1) return kBiasPerM;
  if (s.size() == 2 && s[0] == 1 && s[1] == 1) return kBiasScalar;
  if (numel == N) return kBiasPerN;
  if (numel == M) return kBiasPerM;
  if (numel == 1) return kBiasScalar;
  return kBiasNone;
}

bool bias_buffer_ok(const Tensor* b, int kind) {
  if (!b || !b->data || kind == kBiasNone) return true;
  return b->desc.dtype == DType::F32;
}

bool ws_lt_ok(const GemmWorkspace* ws) {
  return !ws || !ws->lt_workspace || (reinterpret_cast<std::uintptr_t>(ws->lt_workspace) % 256u) == 0;
}

Status from_rc(int rc) {
  switch (rc) {
    case ge2b::kOk:            return Status::Ok;
    case ge2b::kBadArgs:       return Status::Invalid;
    case ge2b::kUnimplemented: return Status::Unimplemented;
    default:                   return Status::CUDA_ERROR;
  }
}

}  // namespace

Status GemmCudaLaunch(const Tensor& A, const Tensor& B, const Tensor* Bias, Tensor& Y, const GemmAttrs& attrs,
                      StreamHandle stream, Tensor* Z_saved, const GemmWorkspace* ws) {
  const DType dt = A.desc.dtype;
  if (!float_dtype(dt)) return Status::DeviceMismatch;
  if (!is_cuda_rowmajor_2d(A, dt) || !is_cuda_rowmajor_2d(B, dt) || !is_cuda_rowmajor_2d(Y, dt))
    return Status::DeviceMismatch;
  if (attrs.trans_a || attrs.trans_b) return Status::TransposeNotSupported;

  const std::int64_t M = A.desc.shape[0], K = A.desc.shape[1], Kb = B.desc.shape[0], N = B.desc.shape[1];
  if (K != Kb || Y.desc.shape[0] != M || Y.desc.shape[1] != N) return Status::ShapeMismatch;

  const std::int64_t lda = infer_ld(A), ldb = infer_ld(B), ldd = infer_ld(Y);
  if (lda < K || ldb < N || ldd < N) return Status::StrideMismatch;
  if (!fits_i32(M) || !fits_i32(N) || !fits_i32(K) || !fits_i32(lda) || !fits_i32(ldb) || !fits_i32(ldd))
    return Status::Invalid;

  if (attrs.save_z && Z_saved == nullptr) return Status::MissingOutput;
  const bool want_z = attrs.save_z && Z_saved != nullptr;
  std::int64_t ldz = 0;
  DType zdt = dt;
  if (want_z) {
    zdt = Z_saved->desc.dtype;
    if (!(zdt == dt || zdt == DType::F32) || !is_cuda_rowmajor_2d(*Z_saved, zdt)) return Status::DeviceMismatch;
    if (Z_saved->desc.shape[0] != M || Z_saved->desc.shape[1] != N) return Status::ShapeMismatch;
    const bool alias = Z_saved->data == Y.data;
    ldz = alias ? ldd : infer_ld(*Z_saved);
    if (ldz < N) return Status::StrideMismatch;
    if (!fits_i32(ldz)) return Status::Invalid;
  }
  if (!ws_lt_ok(ws)) return Status::Invalid;

  const int bias_kind = decide_bias_kind(Bias, M, N);
  if (!bias_buffer_ok(Bias, bias_kind)) return Status::Invalid;
  if (M == 0 || N == 0) return Status::Ok;   // nothing to write
  if (K == 0) return Status::Invalid;

  ge2b::DenseForward f;
  f.M = static_cast<int>(M); f.N = static_cast<int>(N); f.K = static_cast<int>(K);
  f.dtype = static_cast<int>(dt); f.z_dtype = static_cast<int>(zdt);
  f.math = (dt == DType::F32) ? ge2b::default_fp32_math() : 1;
  f.A = A.data; f.lda = lda;
  f.B = B.data; f.ldb = ldb;
  f.D = Y.data; f.ldd = ldd;
  f.Z = want_z ? Z_saved->data : nullptr; f.ldz = ldz;
  f.bias = (Bias && Bias->data && bias_kind != kBiasNone) ? static_cast<const float*>(Bias->data) : nullptr;
  f.bias_kind = bias_kind;
  f.act = static_cast<int>(attrs.act);
  f.leaky = attrs.leaky_slope;
  f.alpha = 1.f; f.beta = 0.f;
  // the caller's lt_workspace (which the reference plumbs through and never reads) holds split-K partial sums
  ge2b::ScopedLease lease(ws ? ws->lt_workspace : nullptr, ws ? ws->lt_workspace_bytes : 0, false);
  return from_rc(ge2b::dense_forward(f, reinterpret_cast<cudaStream_t>(stream)));
}

Status GemmCudaBackward(const Tensor& A, const Tensor& B, const Tensor* C, const Tensor& gY, const Tensor& Z,
                        Tensor* gA, Tensor* gB, Tensor* gC, Tensor* gBias, const GemmAttrs& attrs, StreamHandle stream,
                        const GemmWorkspace* ws) {
  const DType dt = A.desc.dtype;
  if (!float_dtype(dt)) return Status::DeviceMismatch;
  const DType zdt = Z.desc.dtype;
  if (!is_cuda_rowmajor_2d(A, dt) || !is_cuda_rowmajor_2d(B, dt) || !is_cuda_rowmajor_2d(gY, dt) ||
      !(zdt == dt || zdt == DType::F32) || !is_cuda_rowmajor_2d(Z, zdt))
    return Status::DeviceMismatch;
  if (gA && !is_cuda_rowmajor_2d(*gA, dt)) return Status::DeviceMismatch;
  if (gB && !is_cuda_rowmajor_2d(*gB, dt)) return Status::DeviceMismatch;
  if (gC && !is_cuda_rowmajor_2d(*gC, dt)) return Status::DeviceMismatch;
  if (C && !is_cuda_rowmajor_2d(*C, dt)) return Status::DeviceMismatch;
  if (attrs.trans_a || attrs.trans_b) return Status::TransposeNotSupported;

  const std::int64_t M = A.desc.shape[0], K = A.desc.shape[1], Kb = B.desc.shape[0], N = B.desc.shape[1];
  if (K != Kb) return Status::ShapeMismatch;
  if (gY.desc.shape[0] != M || gY.desc.shape[1] != N) return Status::ShapeMismatch;
  if (Z.desc.shape[0] != M || Z.desc.shape[1] != N) return Status::ShapeMismatch;
  if (gA && (gA->desc.shape[0] != M || gA->desc.shape[1] != K)) return Status::ShapeMismatch;
  if (gB && (gB->desc.shape[0] != K || gB->desc.shape[1] != N)) return Status::ShapeMismatch;
  if (gC) {
    if (!C) return Status::MissingInput;
    if (gC->desc.shape[0] != M || gC->desc.shape[1] != N) return Status::ShapeMismatch;
  }

  const std::int64_t lda = infer_ld(A), ldb = infer_ld(B), ldgY = infer_ld(gY), ldZ = infer_ld(Z);
  if (lda < K || ldb < N || ldgY < N || ldZ < N) return Status::StrideMismatch;
  std::int64_t ldgA = 0, ldgB = 0, ldgC = 0;
  if (gA) { ldgA = infer_ld(*gA); if (ldgA < K) return Status::StrideMismatch; }
  if (gB) { ldgB = infer_ld(*gB); if (ldgB < N) return Status::StrideMismatch; }
  if (gC) { ldgC = infer_ld(*gC); if (ldgC < N) return Status::StrideMismatch; }
  if (!fits_i32(M) || !fits_i32(N) || !fits_i32(K) || !fits_i32(lda) || !fits_i32(ldb) || !fits_i32(ldgY) ||
      !fits_i32(ldZ) || !fits_i32(ldgA) || !fits_i32(ldgB) || !fits_i32(ldgC))
    return Status::Invalid;

  int bias_kind = kBiasNone;
  if (gBias && gBias->data) {
    bias_kind = decide_bias_kind(gBias, M, N);
    if (!bias_buffer_ok(gBias, bias_kind)) return Status::Invalid;
  }
  if (!ws_lt_ok(ws)) return Status::Invalid;
  if (ws && ws->scratch && ws->scratch_bytes > 0 &&
      ws->scratch_bytes < static_cast<std::size_t>(M) * static_cast<std::size_t>(N) * sizeof(float))
    return Status::Invalid;
  if (M <= 0 || N <= 0 || K <= 0) return Status::Invalid;

  ge2b::DenseBackward b;
  b.M = static_cast<int>(M); b.N = static_cast<int>(N); b.K = static_cast<int>(K);
  b.dtype = static_cast<int>(dt); b.z_dtype = static_cast<int>(zdt);
  b.math = (dt == DType::F32) ? ge2b::default_fp32_math() : 1;
  b.A = A.data; b.lda = lda;
  b.B = B.data; b.ldb = ldb;
  b.C = C ? C->data : nullptr; b.ldc = C ? infer_ld(*C) : 0;
  b.gY = gY.data; b.ldgY = ldgY;
  b.Z = Z.data; b.ldZ = ldZ;
  b.gA = gA ? gA->data : nullptr; b.ldgA = ldgA;
  b.gB = gB ? gB->data : nullptr; b.ldgB = ldgB;
  b.gC = gC ? gC->data : nullptr; b.ldgC = ldgC;
  b.gBias = (gBias && gBias->data) ? static_cast<float*>(gBias->data) : nullptr;
  b.bias_kind = bias_kind;
  b.act = static_cast<int>(attrs.act);
  b.leaky = attrs.leaky_slope;
  b.alpha = 1.f;
  b.beta = (C && gC) ? 1.f : 0.f;
  b.scratch = ws ? ws->scratch : nullptr;
  b.scratch_bytes = ws ? ws->scratch_bytes : 0;
  ge2b::ScopedLease lease(ws ? ws->lt_workspace : nullptr, ws ? ws->lt_workspace_bytes : 0, false);
  return from_rc(ge2b::dense_backward(b, reinterpret_cast<cudaStream_t>(stream)));
}

namespace {
ge2b::DenseForward forward_from_params(const GemmBiasActParamsEx& p) {
  ge2b::DenseForward f;
  f.M = p.M; f.N = p.N; f.K = p.K;
  f.dtype = ge2b::kF32; f.z_dtype = ge2b::kF32; f.math = 0;
  f.A = p.A; f.lda = p.lda; f.B = p.B; f.ldb = p.ldb;
  f.C = p.C; f.ldc = p.ldc;
  f.D = p.D; f.ldd = p.ldd;
  f.Z = (p.save_preact && p.Z) ? p.Z : nullptr; f.ldz = p.ldZ == 0 ? p.ldd : p.ldZ;
  f.bias = static_cast<const float*>(p.bias);
  f.bias_kind = p.bias ? static_cast<int>(p.bias_kind) : kBiasNone;
  f.act = static_cast<int>(p.act); f.leaky = p.leaky_slope;
  f.alpha = p.alpha; f.beta = p.C ? p.beta : 0.f;
  return f;
}
}  // namespace

void gemm_bias_act_f32_ex(const GemmBiasActParamsEx& p, CUstream_st* stream) {
  (void)ge2b::dense_forward(forward_from_params(p), reinterpret_cast<cudaStream_t>(stream));
}

void launch_gemm_bias_act_f32_smoke_ex(const GemmBiasActParamsEx& p, CUstream_st* stream) {
  gemm_bias_act_f32_ex(p, stream);     // the router picks the one-thread-per-output kernel by the same size rule
}

void gemm_bias_act_f32(const GemmBiasActParams& p, CUstream_st* stream) {
  GemmBiasActParamsEx e{};
  e.M = p.M; e.N = p.N; e.K = p.K;
  e.A = p.A; e.lda = p.lda; e.B = p.B; e.ldb = p.ldb; e.C = p.C; e.ldc = p.ldc; e.D = p.D; e.ldd = p.ldd;
  e.alpha = p.alpha; e.beta = p.beta; e.bias = p.bias; e.bias_kind = p.bias_kind; e.act = p.act;
  e.leaky_slope = p.leaky_slope; e.Z = nullptr; e.ldZ = 0; e.save_preact = 0;
  gemm_bias_act_f32_ex(e, stream);
}

void gemm_bias_act_bwd_f32(const GemmBiasActBwdParams& p, CUstream_st* stream) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) throw std::invalid_argument("invalid dims");
  if (!p.gY || !p.Z) throw std::invalid_argument("gY/Z is null");
  if (p.ldgY < p.N || p.ldZ < p.N) throw std::invalid_argument("ldgY/ldZ < N");
  if (p.gZ_scratch && p.ldgZ != 0 && p.ldgZ != p.N) throw std::invalid_argument("gZ_scratch provided but ldgZ != N");
  ge2b::DenseBackward b;
  b.M = p.M; b.N = p.N; b.K = p.K;
  b.dtype = ge2b::kF32; b.z_dtype = ge2b::kF32; b.math = 0;
  b.A = p.A; b.lda = p.lda; b.B = p.B; b.ldb = p.ldb; b.C = p.C; b.ldc = p.ldc;
  b.gY = p.gY; b.ldgY = p.ldgY; b.Z = p.Z; b.ldZ = p.ldZ;
  b.gA = p.gA; b.ldgA = p.ldgA; b.gB = p.gB; b.ldgB = p.ldgB; b.gC = p.gC; b.ldgC = p.ldgC;
  b.gBias = static_cast<float*>(p.gBias);
  b.bias_kind = p.gBias ? static_cast<int>(p.bias_kind) : kBiasNone;
  b.act = static_cast<int>(p.act); b.leaky = p.leaky_slope;
  b.alpha = p.alpha; b.beta = p.beta;
  b.scratch = p.gZ_scratch; b.scratch_bytes = 0;
  if (ge2b::dense_backward(b, reinterpret_cast<cudaStream_t>(stream)) == ge2b::kBadArgs)
    throw std::invalid_argument("gemm_bias_act_bwd_f32: inconsistent arguments");
}

}  // namespace ai::cuda::shim

namespace ge2b {
namespace {
ai::cuda::shim::Status fwd_entry(const ai::cuda::shim::Tensor& A, const ai::cuda::shim::Tensor& B,
                                 const ai::cuda::shim::Tensor* Bias, ai::cuda::shim::Tensor& Y,
                                 const ai::cuda::shim::GemmAttrs& attrs, ai::cuda::shim::StreamHandle s,
                                 ai::cuda::shim::Tensor* Z) {
  return ai::cuda::shim::GemmCudaLaunch(A, B, Bias, Y, attrs, s, Z, nullptr);
}
ai::cuda::shim::Status bwd_entry(const ai::cuda::shim::Tensor& A, const ai::cuda::shim::Tensor& B,
                                 const ai::cuda::shim::Tensor* C, const ai::cuda::shim::Tensor& gY,
                                 const ai::cuda::shim::Tensor& Z, ai::cuda::shim::Tensor* gA,
                                 ai::cuda::shim::Tensor* gB, ai::cuda::shim::Tensor* gC,
                                 ai::cuda::shim::Tensor* gBias, const ai::cuda::shim::GemmAttrs& attrs,
                                 ai::cuda::shim::StreamHandle s) {
  return ai::cuda::shim::GemmCudaBackward(A, B, C, gY, Z, gA, gB, gC, gBias, attrs, s, nullptr);
}
}  // namespace
KernelFn gemm_forward_kernel_fn() { return &fwd_entry; }
GemmBwdFn gemm_backward_kernel_fn() { return &bwd_entry; }
}  // namespace ge2b
