// Backward of the dense layer for callers that must not allocate device memory.
//
// The ordinary backward entry points need a scratch buffer for gZ = gY * act'(Z): either the caller passes
// one, or the library takes it from the stream-ordered allocator.  Some callers can do neither: a plugin that
// runs inside a framework whose memory pool has reserved the whole GPU (any further cudaMalloc fails), or a
// serving / control loop in which allocator calls are forbidden because they may block or fail at an
// arbitrary moment, and which only hands over the operator's inputs and outputs.  For them this file keeps the
// scratch in a fixed array inside the library's device image.
//
// Cost and limits, stated plainly:
//   * the array is GE2B_NOALLOC_SCRATCH_BYTES (16 MiB) and every GPU that loads the library holds it until the
//     process exits, used or not;
//   * a call is refused (-1) when M * N * sizeof(element) exceeds that size;
//   * all calls share the one array per GPU and it keeps whatever the previous call left there.  Nothing in it
//     has to start at zero except the split-K arrival counters, which every launch that uses them clears on the
//     stream first; the prologue kernel overwrites the M x N region before the GEMMs read it; gBias / gC are zeroed
//     by cudaMemsetAsync as in the ordinary path.  Two calls whose kernels overlap on the GPU (different streams
//     without ordering) race on the array: order them;
//   * what the array has left after gZ is lent to the GEMM launches for their split-K partial sums (problems smaller
//     than one wave of the machine); when that is too little for a split the launch runs unsplit.  While the call
//     is running the launch layer is forbidden to create scratch of its own (ScopedLease with no_alloc);
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress) and, inside the
//     GEMM launcher, sets a function attribute; make that first call before starting any stream capture.  With
//     lazy module loading that first call is also the moment the driver reserves the 16 MiB for the array: under a
//     pool that has already taken every byte of the GPU it fails with -2; load the library before the pool grows.
// The entry point calls no cudaMalloc / cudaFree / cudaMallocAsync and no allocating library routine.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"

using namespace ge2b;

namespace {

static __device__ __align__(256) unsigned char g_noalloc_scratch[GE2B_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDev = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDev] = {};

// In host code the name `g_noalloc_scratch` is only a handle for the symbol, not a device address: the address
// a kernel can use has to be asked for, once per device, with that device current.
void* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess) return nullptr;
    g_scratch_addr[dev] = p;
  }
  return g_scratch_addr[dev];
}

int map_bias(int k) {
  switch (k) {
    case GE2_BIAS_PER_M: return kBiasPerM;
    case GE2_BIAS_PER_N: return kBiasPerN;
    default:             return kBiasScalar;
  }
}

}  // namespace

extern "C" int ge2_launch_gemm_bias_act_bwd_noalloc(const ge2_uintptr* bufs, int n, void* stream) {
  if (!bufs || n < 10) return kBadArgs;
  const auto* pt = reinterpret_cast<const ge2_gemm_bwd_typed_params_t*>(bufs[n - 1]);
  if (!pt) return kBadArgs;
  const int dt = pt->dtype, zdt = pt->z_dtype;
  auto dtype_ok = [](int d) { return d == GE2_DT_F32 || d == GE2_DT_F16 || d == GE2_DT_BF16; };
  if (!dtype_ok(dt) || !dtype_ok(zdt)) return kBadArgs;
  const ge2_gemm_bias_act_bwd_params_t& pb = pt->base;
  if (pb.M <= 0 || pb.N <= 0 || pb.K <= 0) return kBadArgs;
  const size_t need = static_cast<size_t>(pb.M) * static_cast<size_t>(pb.N) * static_cast<size_t>(dtype_bytes(dt));
  if (need > static_cast<size_t>(GE2B_NOALLOC_SCRATCH_BYTES)) return kBadArgs;   // larger than the fixed scratch

  void* scratch = scratch_for_current_device();
  if (!scratch) return kCudaError;

  DenseBackward b;
  b.M = pb.M; b.N = pb.N; b.K = pb.K;
  b.dtype = dt; b.z_dtype = zdt;
  b.math = (dt == GE2_DT_F32) ? (pt->math == GE2_MATH_TENSOR ? 1 : (pt->math == GE2_MATH_FP32X3 ? 2 : 0)) : 1;
  b.A = reinterpret_cast<const void*>(bufs[0]);
  b.B = reinterpret_cast<const void*>(bufs[1]);
  b.C = reinterpret_cast<const void*>(bufs[2]);
  b.gY = reinterpret_cast<const void*>(bufs[3]);
  b.Z = reinterpret_cast<const void*>(bufs[4]);
  b.gA = reinterpret_cast<void*>(bufs[5]);
  b.gB = reinterpret_cast<void*>(bufs[6]);
  b.gC = reinterpret_cast<void*>(bufs[7]);
  b.gBias = reinterpret_cast<float*>(bufs[8]);
  b.lda = pb.lda > 0 ? pb.lda : pb.K;    b.ldb = pb.ldb > 0 ? pb.ldb : pb.N;    b.ldc = pb.ldc > 0 ? pb.ldc : pb.N;
  b.ldgY = pb.ldgY > 0 ? pb.ldgY : pb.N; b.ldZ = pb.ldZ > 0 ? pb.ldZ : pb.N;
  b.ldgA = pb.ldgA > 0 ? pb.ldgA : pb.K; b.ldgB = pb.ldgB > 0 ? pb.ldgB : pb.N; b.ldgC = pb.ldgC > 0 ? pb.ldgC : pb.N;
  b.alpha = pb.alpha; b.beta = pb.beta;
  b.bias_kind = b.gBias ? map_bias(pb.bias_kind) : kBiasNone;
  const int act_code = static_cast<int>(pb.act_kind);
  b.act = (act_code >= 0 && act_code <= 5) ? act_code : static_cast<int>(kActNone);
  b.leaky = pb.leaky_slope;
  b.scratch = scratch;
  b.scratch_bytes = GE2B_NOALLOC_SCRATCH_BYTES;
  b.reuse_gz = false;
  // the rest of the array serves the GEMM launches' split-K partial sums; nothing may be allocated meanwhile
  const size_t used = (need + 255u) & ~static_cast<size_t>(255u);
  ScopedLease lease(static_cast<unsigned char*>(scratch) + used,
                    used < static_cast<size_t>(GE2B_NOALLOC_SCRATCH_BYTES) ? GE2B_NOALLOC_SCRATCH_BYTES - used : 0, true);
  return dense_backward(b, reinterpret_cast<cudaStream_t>(stream));
}
