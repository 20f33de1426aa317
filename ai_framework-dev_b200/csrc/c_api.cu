// extern "C" launch layer.  Parses the reference's bufs[] + trailing-host-params convention
// (dev/backend/graph_executor_v2/src/my_kernels.cu:36-254, src/launch_table.cpp:31-96) and the typed
// additions, and hands a DenseForward / DenseBackward to the kernel router.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"

using namespace ge2b;

namespace {

int map_bias(int k) {   // C-ABI numbering -> internal numbering
  switch (k) {
    case GE2_BIAS_PER_M: return kBiasPerM;
    case GE2_BIAS_PER_N: return kBiasPerN;
    case GE2_BIAS_SCALAR:
    default:             return kBiasScalar;
  }
}
int map_act(int a) { return (a >= 0 && a <= 5) ? a : kActNone; }
bool dtype_ok(int dt) { return dt == GE2_DT_F32 || dt == GE2_DT_F16 || dt == GE2_DT_BF16; }

// Shared parser of the forward bufs layout [A, B, (C), D, (bias), (Z), &params].
int forward_from_bufs(const ge2_uintptr* bufs, int n, const ge2_gemm_bias_act_params_ex_t& px, DenseForward& f) {
  int need = 4 + (px.use_C ? 1 : 0) + (px.has_bias ? 1 : 0) + (px.save_preact ? 1 : 0);
  if (n < need) return kBadArgs;
  int i = 0;
  f.A = reinterpret_cast<const void*>(bufs[i++]);
  f.B = reinterpret_cast<const void*>(bufs[i++]);
  if (px.use_C) f.C = reinterpret_cast<const void*>(bufs[i++]);
  f.D = reinterpret_cast<void*>(bufs[i++]);
  if (px.has_bias) f.bias = reinterpret_cast<const float*>(bufs[i++]);
  if (px.save_preact) f.Z = reinterpret_cast<void*>(bufs[i++]);
  f.M = px.M; f.N = px.N; f.K = px.K;
  f.lda = px.lda > 0 ? px.lda : (long long)(f.trans_a ? px.M : px.K);
  f.ldb = px.ldb > 0 ? px.ldb : (long long)(f.trans_b ? px.K : px.N);
  f.ldc = px.ldc > 0 ? px.ldc : (long long)px.N;
  f.ldd = px.ldd > 0 ? px.ldd : (long long)px.N;
  f.ldz = px.ldZ > 0 ? px.ldZ : f.ldd;
  f.alpha = (px.alpha == 0.f) ? 1.f : px.alpha;
  f.beta = px.beta;
  f.bias_kind = f.bias ? map_bias(px.bias_kind) : kBiasNone;
  f.act = map_act(px.act_kind);
  f.leaky = px.leaky_slope;
  if (px.save_preact && !f.Z) return kBadArgs;
  return kOk;
}

}  // namespace

extern "C" {

int ge2_launch_gemm_bias_act_f32(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 4) return kBadArgs;
  const auto* po = reinterpret_cast<const ge2_gemm_bias_act_params_t*>(bufs[n - 1]);
  if (!po) return kBadArgs;
  if (po->has_bias && n < 5) return kBadArgs;
  DenseForward f;
  f.A = reinterpret_cast<const void*>(bufs[0]);
  f.B = reinterpret_cast<const void*>(bufs[1]);
  f.bias = po->has_bias ? reinterpret_cast<const float*>(bufs[2]) : nullptr;
  f.D = reinterpret_cast<void*>(bufs[po->has_bias ? 3 : 2]);
  f.M = po->M; f.N = po->N; f.K = po->K;
  f.lda = po->K; f.ldb = po->N; f.ldd = po->N;
  f.bias_kind = f.bias ? kBiasPerN : kBiasNone;
  f.act = (po->act == 1) ? kActReLU : kActNone;
  f.dtype = kF32; f.z_dtype = kF32; f.math = 0;
  return dense_forward(f, reinterpret_cast<cudaStream_t>(stream));
}

int ge2_launch_gemm_bias_act_tc_f16(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 4) return kBadArgs;
  const auto* po = reinterpret_cast<const ge2_gemm_bias_act_params_t*>(bufs[n - 1]);
  if (!po) return kBadArgs;
  if (po->has_bias && n < 5) return kBadArgs;
  DenseForward f;
  f.A = reinterpret_cast<const void*>(bufs[0]);
  f.B = reinterpret_cast<const void*>(bufs[1]);
  f.bias = po->has_bias ? reinterpret_cast<const float*>(bufs[2]) : nullptr;
  f.D = reinterpret_cast<void*>(bufs[po->has_bias ? 3 : 2]);
  f.M = po->M; f.N = po->N; f.K = po->K;
  f.lda = po->K; f.ldb = po->N; f.ldd = po->N;
  f.bias_kind = f.bias ? kBiasPerN : kBiasNone;
  f.act = (po->act == 1) ? kActReLU : kActNone;
  f.dtype = kF16; f.z_dtype = kF16; f.math = 1;
  return dense_forward(f, reinterpret_cast<cudaStream_t>(stream));
}

int ge2_launch_gemm_bias_act_f32_ex(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 4) return kBadArgs;
  const auto* px = reinterpret_cast<const ge2_gemm_bias_act_params_ex_t*>(bufs[n - 1]);
  if (!px) return kBadArgs;
  DenseForward f;
  f.dtype = kF32; f.z_dtype = kF32; f.math = 0;
  const int rc = forward_from_bufs(bufs, n, *px, f);
  if (rc != kOk) return rc;
  return dense_forward(f, reinterpret_cast<cudaStream_t>(stream));
}

int ge2_launch_gemm_bias_act_typed(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 4) return kBadArgs;
  const auto* pt = reinterpret_cast<const ge2_gemm_typed_params_t*>(bufs[n - 1]);
  if (!pt) return kBadArgs;
  if (!dtype_ok(pt->dtype) || !dtype_ok(pt->z_dtype)) return kBadArgs;
  DenseForward f;
  f.dtype = pt->dtype; f.z_dtype = pt->z_dtype;
  f.math = (pt->dtype == GE2_DT_F32) ? (pt->math == GE2_MATH_TENSOR ? 1 : (pt->math == GE2_MATH_FP32X3 ? 2 : 0)) : 1;
  f.trans_b = pt->trans_b != 0;
  f.trans_a = pt->trans_a != 0;
  const int rc = forward_from_bufs(bufs, n, pt->base, f);
  if (rc != kOk) return rc;
  f.batch = pt->batch > 1 ? pt->batch : 1;
  f.strideA = pt->strideA; f.strideB = pt->strideB; f.strideC = pt->strideC;
  f.strideD = pt->strideD; f.strideZ = pt->strideZ;
  if (f.batch > 1 && (f.strideA < 0 || f.strideB < 0 || f.strideC < 0 || f.strideD <= 0 || f.strideZ < 0)) return kBadArgs;
  return dense_forward(f, reinterpret_cast<cudaStream_t>(stream));
}

static int backward_common(const ge2_uintptr* bufs, const ge2_gemm_bias_act_bwd_params_t& pb, int dtype, int z_dtype,
                           int math, void* scratch, size_t scratch_bytes, bool reuse_gz, void* stream) {
  DenseBackward b;
  b.M = pb.M; b.N = pb.N; b.K = pb.K;
  b.dtype = dtype; b.z_dtype = z_dtype; b.math = math;
  b.A = reinterpret_cast<const void*>(bufs[0]);
  b.B = reinterpret_cast<const void*>(bufs[1]);
  b.C = reinterpret_cast<const void*>(bufs[2]);
  b.gY = reinterpret_cast<const void*>(bufs[3]);
  b.Z = reinterpret_cast<const void*>(bufs[4]);
  b.gA = reinterpret_cast<void*>(bufs[5]);
  b.gB = reinterpret_cast<void*>(bufs[6]);
  b.gC = reinterpret_cast<void*>(bufs[7]);
  b.gBias = reinterpret_cast<float*>(bufs[8]);
  b.lda = pb.lda > 0 ? pb.lda : pb.K;   b.ldb = pb.ldb > 0 ? pb.ldb : pb.N;   b.ldc = pb.ldc > 0 ? pb.ldc : pb.N;
  b.ldgY = pb.ldgY > 0 ? pb.ldgY : pb.N; b.ldZ = pb.ldZ > 0 ? pb.ldZ : pb.N;
  b.ldgA = pb.ldgA > 0 ? pb.ldgA : pb.K; b.ldgB = pb.ldgB > 0 ? pb.ldgB : pb.N; b.ldgC = pb.ldgC > 0 ? pb.ldgC : pb.N;
  b.alpha = pb.alpha; b.beta = pb.beta;
  b.bias_kind = b.gBias ? map_bias(pb.bias_kind) : kBiasNone;
  b.act = map_act(pb.act_kind);
  b.leaky = pb.leaky_slope;
  b.scratch = scratch; b.scratch_bytes = scratch_bytes; b.reuse_gz = reuse_gz;
  return dense_backward(b, reinterpret_cast<cudaStream_t>(stream));
}

int ge2_launch_gemm_bias_act_bwd_f32_ex(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 10) return kBadArgs;
  const auto* pb = reinterpret_cast<const ge2_gemm_bias_act_bwd_params_t*>(bufs[n - 1]);
  if (!pb) return kBadArgs;
  return backward_common(bufs, *pb, kF32, kF32, 0, nullptr, 0, false, stream);
}

int ge2_launch_gemm_bias_act_bwd_typed(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 11) return kBadArgs;
  const auto* pt = reinterpret_cast<const ge2_gemm_bwd_typed_params_t*>(bufs[n - 1]);
  if (!pt) return kBadArgs;
  if (!dtype_ok(pt->dtype) || !dtype_ok(pt->z_dtype)) return kBadArgs;
  const int math = (pt->dtype == GE2_DT_F32) ? (pt->math == GE2_MATH_TENSOR ? 1 : (pt->math == GE2_MATH_FP32X3 ? 2 : 0)) : 1;
  return backward_common(bufs, pt->base, pt->dtype, pt->z_dtype, math, reinterpret_cast<void*>(bufs[9]),
                         pt->scratch_bytes, pt->reuse_gz != 0, stream);
}

int ge2_launch(const char* name, const ge2_uintptr* bufs, int n, void* stream) {
  if (!name) return kBadArgs;
  auto too_few = [&](int want) {
    if (n < want) { std::fprintf(stderr, "[GE2] '%s' needs >= %d bufs (got %d)\n", name, want, n); return true; }
    return false;
  };
  if (!std::strcmp(name, "gemm_bias_act_f32"))
    return too_few(4) ? kBadArgs : ge2_launch_gemm_bias_act_f32(bufs, n, stream);
  if (!std::strcmp(name, "gemm_bias_act_tc_f16"))
    return too_few(4) ? kBadArgs : ge2_launch_gemm_bias_act_tc_f16(bufs, n, stream);
  if (!std::strcmp(name, "gemm_bias_act_f32_ex") || !std::strcmp(name, "gemm_bias_act_ex"))
    return too_few(4) ? kBadArgs : ge2_launch_gemm_bias_act_f32_ex(bufs, n, stream);
  if (!std::strcmp(name, "gemm_bias_act_bwd_f32_ex") || !std::strcmp(name, "gemm_bias_act_bwd"))
    return too_few(10) ? kBadArgs : ge2_launch_gemm_bias_act_bwd_f32_ex(bufs, n, stream);
  if (!std::strcmp(name, "gemm_bias_act_typed") || !std::strcmp(name, "gemm_strided_batched"))
    return too_few(4) ? kBadArgs : ge2_launch_gemm_bias_act_typed(bufs, n, stream);
  if (!std::strcmp(name, "gemm_bias_act_bwd_typed"))
    return too_few(11) ? kBadArgs : ge2_launch_gemm_bias_act_bwd_typed(bufs, n, stream);
  std::fprintf(stderr, "[GE2] unknown kernel: %s\n", name);
  return kBadArgs;
}

size_t ge2b_backward_scratch_bytes(long long M, long long N) {
  return (M <= 0 || N <= 0) ? 0 : static_cast<size_t>(M) * static_cast<size_t>(N) * sizeof(float);
}
int ge2b_device_status(int clear) { return device_status_word(clear != 0); }
int ge2b_sm_count(void) { return sm_count(); }
void ge2b_set_sm_limit(int n) { set_sm_limit(n); }
const char* ge2b_version(void) { return "ge2_b200 0.1 (sm_100a)"; }

// Not part of the public header: introspection used by the test-suite and the benchmark.
int ge2b_last_route(void) { return last_route(); }
long long ge2b_launches_total(void) { return launches_total(); }
long long ge2b_split_unavailable_total(void) { return split_unavailable_total(); }
void ge2b_release_scratch(void) { release_library_scratch(); }

}  // extern "C"
