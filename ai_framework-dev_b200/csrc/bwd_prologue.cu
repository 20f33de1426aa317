// Backward prologue of the dense layer:  gZ = gY * act'(Z), optional gC = beta * gZ, and the bias
// gradient as a reduction of gZ over rows (per-column bias), over columns (per-row bias) or over
// everything (scalar bias).
//
// Replaces the reference's bwd_epilogue_kernel (backends/cuda/ops/gemm/kernels/regemm_backward.cu:92-130),
// which issues one atomicAdd per element for the bias gradient.  Here each thread owns 8 consecutive
// columns (one or two 16-byte accesses), a CTA covers 256 columns x 64 rows, sums in registers and shared
// memory; the per-column bias gradient is then added over the row blocks in a fixed order (run-to-run identical
// bits) by the GEMM launch that follows or by a small kernel (DbFinish); one fp32 atomic per column per CTA only when
// no scratch is to be had, and for per-row / scalar bias gradients.  The bias gradient is always formed
// from the fp32 value of gZ, before gZ is rounded to its storage type.  The buffer gZ is scratch memory
// that the two backward GEMMs read afterwards.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "epilogue_math.cuh"
#include "ge2_internal.hpp"
#include "sm100_ptx.cuh"

namespace ge2b {
namespace {

constexpr int kColsPerThread = 8;
constexpr int kTX = 32, kTY = 8;
constexpr int kTileCols = kTX * kColsPerThread;   // 256
constexpr int kTileRows = 64;
constexpr int kFastRows = 32;   // rows per CTA of the specialised kernel: more, smaller CTAs fill the last wave better

struct ProParams {
  BwdPrologueArgs a;
  int gy_vec, z_vec, gz_vec, gc_vec;
};

__device__ __forceinline__ void load8(const void* base, long long off, int dt, bool vec, int n, float (&v)[8]) {
  if (vec && n == 8) {
    if (dt == kF32) {
      const float4 x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
      const float4 y = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off + 4);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
    } else {
      const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(base) + off);
      const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (dt == kBF16) {
          v[2 * t]     = __uint_as_float(w[t] << 16);
          v[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u);
        } else {
          const __half2 h = *reinterpret_cast<const __half2*>(&w[t]);
          v[2 * t] = __low2float(h); v[2 * t + 1] = __high2float(h);
        }
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (j < n) ? load_as_f32(base, off + j, dt) : 0.f;
  }
}

__device__ __forceinline__ void store8(void* base, long long off, int dt, bool vec, int n, const float (&v)[8]) {
  if (vec && n == 8) {
    if (dt == kF32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off)     = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      unsigned w[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (dt == kBF16) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
          w[t] = *reinterpret_cast<const unsigned*>(&h);
        } else {
          const __half2 h = __floats2half2_rn(v[2 * t], v[2 * t + 1]);
          w[t] = *reinterpret_cast<const unsigned*>(&h);
        }
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(base) + off) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < n) store_from_f32(base, off + j, dt, v[j]);
  }
}

// Per-column bias gradient of one CTA: `s` is this thread's column (c = ty * 32 + tx) summed over the CTA's rows.
// With a partial buffer the CTA just stores its 256 column sums; the sum over row blocks is taken afterwards in a
// fixed order (run-to-run identical bits) by DbFinish.  Without one: one atomic per column.
__device__ __forceinline__ void finish_db_per_column(const BwdPrologueArgs& a, float s, float (&red)[kTY][kTileCols + 1]) {
  const int c = threadIdx.y * kTX + threadIdx.x;
  const int gc = blockIdx.x * kTileCols + c;
  if (a.db_partial == nullptr) {
    if (gc < a.N) atomicAdd(a.gBias + gc, s);
    return;
  }
  a.db_partial[static_cast<long long>(blockIdx.y) * a.db_pitch + gc] = s;      // the pitch covers the padded columns
}

// out[c] = sum over row blocks, ascending, eight loads in flight per thread
__global__ void __launch_bounds__(256) db_finish_kernel(const DbFinish f) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= f.n) return;
  const float* p = f.partial + c;
  float acc = 0.f;
  int b = 0;
  for (; b + 8 <= f.blocks; b += 8) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __ldcg(p + static_cast<long long>(b + i) * f.pitch);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += v[i];
  }
  for (; b < f.blocks; ++b) acc += __ldcg(p + static_cast<long long>(b) * f.pitch);
  f.out[c] = acc;
}

// kRowSum: the bias gradient needs sums along rows (per-row or scalar bias); the common per-column case does not.
template <int ACT, bool kFast, bool kRowSum>
__global__ void __launch_bounds__(kTX * kTY)
bwd_prologue_kernel(const ProParams pp) {
  ptx::griddep_launch();
  ptx::griddep_wait();          // Z comes from the kernel before this one
  const BwdPrologueArgs& a = pp.a;
  __shared__ float red[kTY][kTileCols + 1];

  const int col0 = blockIdx.x * kTileCols + threadIdx.x * kColsPerThread;
  const int row_base = blockIdx.y * kTileRows;
  const int ncols = min(kColsPerThread, a.N - col0);   // <= 0 when this thread is past the edge
  const bool want_bias = a.gBias != nullptr && a.bias_kind != kBiasNone;

  float colsum[kColsPerThread];
#pragma unroll
  for (int j = 0; j < kColsPerThread; ++j) colsum[j] = 0.f;
  float total = 0.f;

  for (int r = threadIdx.y; r < kTileRows; r += kTY) {
    const int m = row_base + r;
    float rowsum = 0.f;
    if (m < a.M && ncols > 0) {
      float gy[8], z[8], gz[8];
      load8(a.gY, static_cast<long long>(m) * a.ldgY + col0, a.gy_dtype, pp.gy_vec != 0, ncols, gy);
      load8(a.Z, static_cast<long long>(m) * a.ldZ + col0, a.z_dtype, pp.z_vec != 0, ncols, z);
      if (ncols == 8) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          gz[j] = gy[j] * act_bwd<ACT, kFast>(z[j], a.leaky);
          colsum[j] += gz[j];
          if constexpr (kRowSum) rowsum += gz[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          gz[j] = (j < ncols) ? gy[j] * act_bwd<ACT, kFast>(z[j], a.leaky) : 0.f;
          colsum[j] += gz[j];
          if constexpr (kRowSum) rowsum += gz[j];
        }
      }
      store8(a.gZ, static_cast<long long>(m) * a.ldgZ + col0, a.gz_dtype, pp.gz_vec != 0, ncols, gz);
      if (a.gC != nullptr) {
        float gc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) gc[j] = a.beta * gz[j];
        store8(a.gC, static_cast<long long>(m) * a.ldgC + col0, a.gc_dtype, pp.gc_vec != 0, ncols, gc);
      }
    }
    if constexpr (kRowSum) {
      if (want_bias && a.bias_kind == kBiasPerM) {
        // all 32 lanes of a warp share the row: one atomic per (row, CTA)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) rowsum += __shfl_xor_sync(0xffffffffu, rowsum, o);
        if (threadIdx.x == 0 && m < a.M) atomicAdd(a.gBias + m, rowsum);
      }
      total += rowsum;
    }
  }

  if (!want_bias || a.bias_kind == kBiasPerM) return;

  if (a.bias_kind == kBiasPerN) {
#pragma unroll
    for (int j = 0; j < kColsPerThread; ++j) red[threadIdx.y][threadIdx.x * kColsPerThread + j] = colsum[j];
    __syncthreads();
    const int c = threadIdx.y * kTX + threadIdx.x;     // 0..255: one column each
    float s = 0.f;
#pragma unroll
    for (int y = 0; y < kTY; ++y) s += red[y][c];
    finish_db_per_column(a, s, red);
  } else {  // scalar: everything
    // `total` here is the per-lane partial (rowsum before the per-row shuffle is only taken for PerM)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (threadIdx.x == 0) red[threadIdx.y][0] = total;
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0) {
      float s = 0.f;
#pragma unroll
      for (int y = 0; y < kTY; ++y) s += red[y][0];
      atomicAdd(a.gBias, s);
    }
  }
}

// Fast form for the common call: gY, Z and gZ all 16-bit of one type, every row 16-byte aligned, N a multiple of
// 8, no gC, bias gradient per column or none.  Same arithmetic as the general kernel (fp32 derivative, fp32 column
// sums taken before gZ is rounded), but the dtype is a template parameter, a thread's 8 rows x 8 columns are loaded
// four rows at a time before any of them is used (8 independent 16-byte loads in flight per thread), and all index
// arithmetic is hoisted out of the row loop.
template <int ACT, bool kBf16>
__global__ void __launch_bounds__(kTX * kTY)
bwd_prologue_fast_kernel(const ProParams pp) {
  ptx::griddep_launch();
  ptx::griddep_wait();          // Z comes from the kernel before this one
  const BwdPrologueArgs& a = pp.a;
  __shared__ float red[kTY][kTileCols + 1];
  const int col0 = blockIdx.x * kTileCols + threadIdx.x * kColsPerThread;
  const int row0 = blockIdx.y * kFastRows + threadIdx.y;
  const bool col_ok = col0 < a.N;
  const bool want_bias = a.gBias != nullptr;

  float colsum[kColsPerThread];
#pragma unroll
  for (int j = 0; j < kColsPerThread; ++j) colsum[j] = 0.f;

  if (col_ok) {
    const unsigned short* gy_p = static_cast<const unsigned short*>(a.gY) + static_cast<long long>(row0) * a.ldgY + col0;
    const unsigned short* z_p = static_cast<const unsigned short*>(a.Z) + static_cast<long long>(row0) * a.ldZ + col0;
    unsigned short* gz_p = static_cast<unsigned short*>(a.gZ) + static_cast<long long>(row0) * a.ldgZ + col0;
    const long long gy_step = static_cast<long long>(kTY) * a.ldgY, z_step = static_cast<long long>(kTY) * a.ldZ,
                    gz_step = static_cast<long long>(kTY) * a.ldgZ;
    constexpr int kBatch = 4;
#pragma unroll
    for (int r0 = 0; r0 < kFastRows / kTY; r0 += kBatch) {
      uint4 gy[kBatch], z[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const bool ok = row0 + (r0 + i) * kTY < a.M;
        gy[i] = ok ? __ldg(reinterpret_cast<const uint4*>(gy_p + (r0 + i) * gy_step)) : make_uint4(0, 0, 0, 0);
        z[i]  = ok ? __ldg(reinterpret_cast<const uint4*>(z_p + (r0 + i) * z_step)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const unsigned gw[4] = {gy[i].x, gy[i].y, gy[i].z, gy[i].w};
        const unsigned zw[4] = {z[i].x, z[i].y, z[i].z, z[i].w};
        unsigned ow[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float g0, g1, z0, z1;
          if constexpr (kBf16) {
            g0 = __uint_as_float(gw[t] << 16); g1 = __uint_as_float(gw[t] & 0xffff0000u);
            z0 = __uint_as_float(zw[t] << 16); z1 = __uint_as_float(zw[t] & 0xffff0000u);
          } else {
            const __half2 gh = *reinterpret_cast<const __half2*>(&gw[t]);
            const __half2 zh = *reinterpret_cast<const __half2*>(&zw[t]);
            g0 = __low2float(gh); g1 = __high2float(gh); z0 = __low2float(zh); z1 = __high2float(zh);
          }
          const float r0v = g0 * act_bwd<ACT, true>(z0, a.leaky);
          const float r1v = g1 * act_bwd<ACT, true>(z1, a.leaky);
          colsum[2 * t] += r0v;          // rows past M were loaded as zeros: they add nothing
          colsum[2 * t + 1] += r1v;
          if constexpr (kBf16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(r0v, r1v);
            ow[t] = *reinterpret_cast<const unsigned*>(&h);
          } else {
            const __half2 h = __floats2half2_rn(r0v, r1v);
            ow[t] = *reinterpret_cast<const unsigned*>(&h);
          }
        }
        if (row0 + (r0 + i) * kTY < a.M)
          *reinterpret_cast<uint4*>(gz_p + (r0 + i) * gz_step) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
  }
  if (!want_bias) return;
#pragma unroll
  for (int j = 0; j < kColsPerThread; ++j) red[threadIdx.y][threadIdx.x * kColsPerThread + j] = colsum[j];
  __syncthreads();
  const int c = threadIdx.y * kTX + threadIdx.x;     // 0..255: one column each
  float s = 0.f;
#pragma unroll
  for (int y = 0; y < kTY; ++y) s += red[y][c];
  finish_db_per_column(a, s, red);
}

// Launch that may start while the kernel before it in the stream is finishing (the kernel waits at griddep_wait()).
template <typename K>
void launch_early(K kernel, dim3 grid, dim3 block, cudaStream_t s, const ProParams& pp) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early_start_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, pp);
}

bool vec_ok(const void* p, long long ld, int dt) {
  if (!p) return false;
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (ld * dtype_bytes(dt)) % 16 == 0;
}

}  // namespace

cudaError_t launch_db_finish(const DbFinish& f, cudaStream_t s) {
  if (!f.partial || !f.out || f.n < 1 || f.blocks < 1) return cudaSuccess;
  db_finish_kernel<<<(f.n + 255) / 256, 256, 0, s>>>(f);
  return cudaGetLastError();
}

cudaError_t launch_bwd_prologue(const BwdPrologueArgs& a, cudaStream_t s, DbFinish* pending, bool zero_gbias) {
  if (pending) *pending = DbFinish{};
  if (a.M < 1 || a.N < 1 || !a.gY || !a.Z || !a.gZ) return cudaErrorInvalidValue;
  ProParams pp{};
  pp.a = a;
  pp.gy_vec = vec_ok(a.gY, a.ldgY, a.gy_dtype);
  pp.z_vec  = vec_ok(a.Z, a.ldZ, a.z_dtype);
  pp.gz_vec = vec_ok(a.gZ, a.ldgZ, a.gz_dtype);
  pp.gc_vec = vec_ok(a.gC, a.ldgC, a.gc_dtype);
  dim3 block(kTX, kTY), grid((a.N + kTileCols - 1) / kTileCols, (a.M + kTileRows - 1) / kTileRows);
  // Deterministic per-column bias gradient: partial sums per row block in stream scratch, when there is some.
  // The partial sums go at the END of the stream scratch: its start belongs to the split-K partial tiles of the GEMM
  // launch that carries the finish.
  auto want_partials = [&](unsigned row_blocks) {
    pp.a.db_partial = nullptr; pp.a.db_pitch = 0;
    if (pending == nullptr || a.gBias == nullptr || a.bias_kind != kBiasPerN || row_blocks < 2) return cudaSuccess;
    float* ws = nullptr; int* flags = nullptr; size_t ws_bytes = 0, flag_bytes = 0; bool lent = false;
    if (!borrow_stream_scratch(s, &ws, &ws_bytes, &flags, &flag_bytes, &lent)) return cudaSuccess;   // atomics instead
    const long long pitch = static_cast<long long>(grid.x) * kTileCols;
    const size_t need = static_cast<size_t>(row_blocks) * pitch * sizeof(float);
    if (need > ws_bytes / 4) return cudaSuccess;           // leave at least three quarters to the GEMMs
    float* part = ws + (ws_bytes - need) / sizeof(float);
    pp.a.db_partial = part; pp.a.db_pitch = pitch;
    pending->partial = part; pending->pitch = pitch; pending->blocks = static_cast<int>(row_blocks);
    pending->out = a.gBias; pending->n = a.N;
    return cudaSuccess;
  };
  auto zero_if_atomic = [&]() {
    if (!zero_gbias || a.gBias == nullptr || a.bias_kind == kBiasNone || pp.a.db_partial != nullptr) return cudaSuccess;
    const size_t n = a.bias_kind == kBiasScalar ? 1 : (a.bias_kind == kBiasPerM ? a.M : a.N);
    return cudaMemsetAsync(a.gBias, 0, n * sizeof(float), s);
  };
  // gZ stored in 16 bits: the exp-based derivative forms are accurate enough (see epilogue_math.cuh)
  // the common 16-bit call takes the specialised kernel
  const bool same16 = a.gy_dtype != kF32 && a.gy_dtype == a.z_dtype && a.gy_dtype == a.gz_dtype;
  const bool col_bias_or_none = a.gBias == nullptr || a.bias_kind == kBiasPerN || a.bias_kind == kBiasNone;
  if (same16 && pp.gy_vec && pp.z_vec && pp.gz_vec && a.N % 8 == 0 && a.gC == nullptr && col_bias_or_none) {
    if (a.gBias != nullptr && a.bias_kind == kBiasNone) pp.a.gBias = nullptr;
    const bool bf = a.gy_dtype == kBF16;
    const dim3 fgrid((a.N + kTileCols - 1) / kTileCols, (a.M + kFastRows - 1) / kFastRows);
    if (want_partials(fgrid.y) != cudaSuccess || zero_if_atomic() != cudaSuccess) return cudaErrorUnknown;
#define GE2B_LAUNCH_FAST(ACT_)                                                                \
    do {                                                                                      \
      if (bf) launch_early(bwd_prologue_fast_kernel<ACT_, true>, fgrid, block, s, pp);        \
      else    launch_early(bwd_prologue_fast_kernel<ACT_, false>, fgrid, block, s, pp);       \
    } while (0)
    switch (a.act) {
      case kActReLU:    GE2B_LAUNCH_FAST(kActReLU); break;
      case kActLeaky:   GE2B_LAUNCH_FAST(kActLeaky); break;
      case kActGELU:    GE2B_LAUNCH_FAST(kActGELU); break;
      case kActSigmoid: GE2B_LAUNCH_FAST(kActSigmoid); break;
      case kActTanh:    GE2B_LAUNCH_FAST(kActTanh); break;
      default:          GE2B_LAUNCH_FAST(kActNone); break;
    }
#undef GE2B_LAUNCH_FAST
    return cudaGetLastError();
  }
  if (want_partials(grid.y) != cudaSuccess || zero_if_atomic() != cudaSuccess) return cudaErrorUnknown;
  const bool fast = a.gz_dtype != kF32;
  const bool rowsum = a.gBias != nullptr && (a.bias_kind == kBiasPerM || a.bias_kind == kBiasScalar);
#define GE2B_LAUNCH_PRO(ACT_)                                                                   \
  do {                                                                                          \
    if (fast) {                                                                                 \
      if (rowsum) bwd_prologue_kernel<ACT_, true, true><<<grid, block, 0, s>>>(pp);             \
      else        bwd_prologue_kernel<ACT_, true, false><<<grid, block, 0, s>>>(pp);            \
    } else {                                                                                    \
      if (rowsum) bwd_prologue_kernel<ACT_, false, true><<<grid, block, 0, s>>>(pp);            \
      else        bwd_prologue_kernel<ACT_, false, false><<<grid, block, 0, s>>>(pp);           \
    }                                                                                           \
  } while (0)
  switch (a.act) {
    case kActReLU:    GE2B_LAUNCH_PRO(kActReLU); break;
    case kActLeaky:   GE2B_LAUNCH_PRO(kActLeaky); break;
    case kActGELU:    GE2B_LAUNCH_PRO(kActGELU); break;
    case kActSigmoid: GE2B_LAUNCH_PRO(kActSigmoid); break;
    case kActTanh:    GE2B_LAUNCH_PRO(kActTanh); break;
    default:          GE2B_LAUNCH_PRO(kActNone); break;
  }
#undef GE2B_LAUNCH_PRO
  return cudaGetLastError();
}

}  // namespace ge2b
