// 2-D convolution as an IMPLICIT GEMM for sm_100a: the column matrix is never written to memory.
//
// The reference builds Col = im2col(X[n]) in global memory per image and hands it to its GEMM
// (backends/cuda/ops/conv2d/launcher.cu:180-227, kernels.cu:12-45); its backward writes dCol and scatters it back with
// col2im (launcher.cu:330-462, kernels.cu:47-110).  Here one persistent kernel computes, for 128 consecutive output
// positions p = (n, ho, wo) of the whole batch and a tile of output channels,
//     D[p][co] = sum_k  Col[p][k] . Wm[co][k]          k = (c, kh, kw)
// with the Col tile gathered by eight producer warps straight from the NCHW input into the shared-memory operand
// stage (positions contiguous: the "M-contiguous" 128-byte-swizzled layout tcgen05.mma reads), the weight tile loaded
// by TMA, the accumulator in TMEM (positions on the 128 lanes, channels on the columns) and an epilogue that adds the
// per-channel bias, applies the activation and writes Y (and the pre-activation Z) in NCHW: a warp's 32 lanes hold 32
// consecutive positions of one channel plane, so every store instruction writes one contiguous run.
//     warp 0        TMA producer of the weight tiles          warp 1        MMA issuer
//     warps 2..5    epilogue (one TMEM lane quarter each)     warps 6..13   gather of the Col tile
// The same kernel computes the input gradient of a unit-stride convolution: dX is the convolution of gZ (Cout planes)
// with the taps mirrored (offset pad - kh*dil instead of kh*dil - pad) and the weight read as [Cin][Cout*Kh*Kw].
// A gather chunk is 8 consecutive positions of one k (16 bytes).  When the 8 positions lie in one input row at unit
// stride and rows start on 16-byte boundaries, the chunk is cut out of two aligned 16-byte loads with funnel shifts
// (an input row shifted by one pixel is never 16-byte aligned, which is why TMA cannot fetch it); otherwise the chunk
// is put together from eight 2-byte loads.  Padding pixels are zeros in both forms.
// Every mbarrier wait is bounded (sm100_ptx.cuh); on expiry the CTA records kErrWaitTimeout in the device status
// word, frees its TMEM and returns.  No TMA load uses cluster multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "conv2d_implicit.hpp"
#include "epilogue_math.cuh"
#include "gemm_tc_kernel.cuh"
#include "sm100_ptx.cuh"

namespace ge2b {
namespace {

constexpr int kBM = 128;                 // output positions per tile (one TMEM lane each)
constexpr int kBK = 64;                  // reduction indices per stage
constexpr int kConvThreads = 448;
constexpr int kEpiWarpsConv = 4;          // warps 2..5
constexpr int kGatherWarp0 = 6, kGatherWarps = 8;
constexpr int kAStageBytes = kBM * kBK * 2;

struct ConvParams {
  const unsigned short* X;               // input planes [n][c][h][w], 16-bit elements
  long long img_pitch, plane_pitch;      // elements from image to image / plane to plane
  int row_pitch;                         // elements from row to row
  int H, W;                              // extent of one input plane
  int Wo, HWo;                           // extent of one output plane (Wo columns, HWo positions)
  int sh, sw;
  int taps;                              // Kh * Kw
  unsigned tap_magic;                    // ceil(2^32 / taps): k / taps == umulhi(k, tap_magic) for every k the kernel sees
  int K, k_blocks;
  int Cout;                              // output channels (rows of the weight matrix)
  long long P;                           // output positions of the whole batch: images * HWo
  int pos_tiles, n_tiles;
  void* Y; void* Z; const float* bias;
  long long out_img_pitch;               // elements from image to image in Y / Z
  int y_dtype, z_dtype, act;
  float leaky;
  int fast;                              // the aligned 16-byte gather may be used
  uint32_t idesc;
  int* status;
  // weight-gradient kernel only
  int bpi, red_blocks;                   // 64-position blocks per image / in the batch
  int split, per;                        // slices of the reduction per output tile, blocks per slice
  int m_tiles;                           // 128-row tiles of the K rows of dW^T
  float* part;                           // partial sums [slice][Cout][K]
  short2 tap_off[kConvMaxTaps];          // per tap: (row offset, column offset) added to (ho*sh, wo*sw)
};

__device__ __forceinline__ uint4 ldg16(const unsigned short* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Output position -> image, row and column.
struct Pos { int n, ho, wo; };
__device__ __forceinline__ Pos decode_pos(const ConvParams& p, long long pos) {
  Pos r;
  r.n = static_cast<int>(pos / p.HWo);
  const int hw = static_cast<int>(pos - static_cast<long long>(r.n) * p.HWo);
  r.ho = hw / p.Wo;
  r.wo = hw - r.ho * p.Wo;
  return r;
}

// Aligned form of the gather, in two halves so that a thread can have the loads of several chunks in flight before it
// uses the first: the chunk of eight consecutive positions starting at column wo of output row ho, read through the
// tap offset `off`, lies inside two aligned 16-byte pieces of one input row (all eight positions share the image and
// the output row; unit column stride; rows start on 16-byte boundaries).
struct RawChunk { uint4 lo, hi; int e; };
__device__ __forceinline__ RawChunk gather_issue(const ConvParams& p, const unsigned short* plane, short2 off, int ho,
                                                 int wo, bool on) {
  RawChunk r;
  const int hi_row = ho * p.sh + off.x;
  on = on && static_cast<unsigned>(hi_row) < static_cast<unsigned>(p.H);
  const unsigned short* row = plane + static_cast<long long>(hi_row) * p.row_pitch;
  const int wi0 = wo + off.y;
  r.e = wi0 & 7;
  const int a = wi0 - r.e;                               // aligned piece [a, a+8), element offset e inside it
  const bool on_lo = on && static_cast<unsigned>(a) < static_cast<unsigned>(p.W);
  const bool on_hi = on && r.e != 0 && static_cast<unsigned>(a + 8) < static_cast<unsigned>(p.W);
  r.lo = on_lo ? ldg16(row + a) : make_uint4(0u, 0u, 0u, 0u);
  r.hi = on_hi ? ldg16(row + a + 8) : make_uint4(0u, 0u, 0u, 0u);
  return r;
}
// Elements e .. e+7 of the 16 elements (lo, hi): a 256-bit value shifted right by 16 e bits, without branches.
__device__ __forceinline__ uint4 gather_finish(const RawChunk& r) {
  const bool two = (r.e & 4) != 0, one = (r.e & 2) != 0;
  const uint32_t t0 = two ? r.lo.z : r.lo.x, t1 = two ? r.lo.w : r.lo.y, t2 = two ? r.hi.x : r.lo.z,
                 t3 = two ? r.hi.y : r.lo.w, t4 = two ? r.hi.z : r.hi.x, t5 = two ? r.hi.w : r.hi.y;
  const uint32_t u0 = one ? t1 : t0, u1 = one ? t2 : t1, u2 = one ? t3 : t2, u3 = one ? t4 : t3, u4 = one ? t5 : t4;
  const uint32_t sft = (r.e & 1) * 16;
  return make_uint4(__funnelshift_r(u0, u1, sft), __funnelshift_r(u1, u2, sft), __funnelshift_r(u2, u3, sft),
                    __funnelshift_r(u3, u4, sft));
}

// General form of the gather: one 2-byte load per position, walking (column, row, image) as the positions advance;
// positions from `valid` on are zeros.
__device__ __forceinline__ uint4 gather_general(const ConvParams& p, const unsigned short* plane, short2 off, int ho, int wo,
                                                int valid) {
  const int Ho = p.HWo / p.Wo;
  uint32_t v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int hi = ho * p.sh + off.x, wi = wo * p.sw + off.y;
    const bool on = j < valid && static_cast<unsigned>(hi) < static_cast<unsigned>(p.H) &&
                    static_cast<unsigned>(wi) < static_cast<unsigned>(p.W);
    v[j] = on ? __ldg(plane + static_cast<long long>(hi) * p.row_pitch + wi) : static_cast<unsigned short>(0);
    if (++wo == p.Wo) {
      wo = 0;
      if (++ho == Ho) { ho = 0; plane += p.img_pitch; }
    }
  }
  return make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
}

// Reduction index k -> channel and tap.
__device__ __forceinline__ int channel_of(const ConvParams& p, int k) {
  return p.taps == 1 ? k : static_cast<int>(__umulhi(static_cast<unsigned>(k), p.tap_magic));
}

template <int ACT>
__device__ __forceinline__ void epilogue_chunk(const ConvParams& p, const uint32_t (&r)[32], int co0, long long off) {
  // 32 channels co0 .. co0+31 of one output position; `off` is the element offset of (n, co0, hw) in Y / Z
  const int n_co = min(32, p.Cout - co0);
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (j < n_co) {
      float v = __uint_as_float(r[j]);
      if (p.bias != nullptr) v += __ldg(p.bias + co0 + j);
      const long long o = off + static_cast<long long>(j) * p.HWo;
      if (p.Z != nullptr) {
        if (p.z_dtype == kF32)       static_cast<float*>(p.Z)[o] = v;
        else if (p.z_dtype == kBF16) static_cast<__nv_bfloat16*>(p.Z)[o] = __float2bfloat16_rn(v);
        else                         static_cast<__half*>(p.Z)[o] = __float2half_rn(v);
      }
      const float y = act_fwd<ACT, true>(v, p.leaky);
      if (p.y_dtype == kBF16) static_cast<__nv_bfloat16*>(p.Y)[o] = __float2bfloat16_rn(y);
      else                    static_cast<__half*>(p.Y)[o] = __float2half_rn(y);
    }
  }
}

template <int kBN, int kStages>
__global__ void __launch_bounds__(kConvThreads, 1)
conv_implicit_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ ConvParams p) {
  constexpr int kBStageBytes = kBN * 128;
  constexpr int kStageBytes = kAStageBytes + kBStageBytes;
  constexpr int kTmemCols = 2 * kBN;
  // Stage fills are dealt round-robin to kSpan groups of gather warps.  A group's next fill is kSpan fills after its
  // last one; kSpan <= kStages keeps it less than two laps of the ring ahead of the consumer, which is what the
  // one-bit phase of the empty barriers can tell apart.
  constexpr int kSpan = kStages >= kGatherWarps ? kGatherWarps : 4;
  constexpr int kWarpsPerStage = kGatherWarps / kSpan;
  constexpr int kStepsPerWarp = 32 / kWarpsPerStage;     // of the 32 row steps of one stage
  static_assert(kSpan <= kStages && kGatherWarps % kSpan == 0, "gather groups and ring depth do not fit");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t base = raw_addr + pad;
  uint8_t* tail = smem + kStages * kStageBytes;
  const uint32_t bar0 = base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(tail + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * (2 * kStages + 4) + 8);
  short2* tap_s = reinterpret_cast<short2*>(tail + 8 * (2 * kStages + 4) + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tiles = static_cast<long long>(p.pos_tiles) * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1 + kWarpsPerStage); ptx::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), kEpiWarpsConv); }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmW);
  }
  for (int t = threadIdx.x; t < p.taps; t += kConvThreads) tap_s[t] = p.tap_off[t];
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ===================== weight tiles by TMA =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        const int nt = static_cast<int>(t % p.n_tiles);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(full_bar(stage), kBStageBytes);
          ptx::tma_load_3d(base + stage * kStageBytes + kAStageBytes, &tmW, full_bar(stage), kb * kBK, nt * kBN, 0);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = base + stage * kStageBytes;
          // Col tile: each 128-byte row holds one k and 64 positions, 8 rows form a 1024-byte group, the second block
          // of 64 positions starts kBK rows later; one MMA consumes 16 rows.  Weight tile: 128-byte rows of 64 k.
          const uint64_t ad = ptx::make_smem_desc_sw128(a_addr, kBK * 128, 1024u, 2u);
          const uint64_t bd = ptx::make_smem_desc_sw128(a_addr + kAStageBytes, 0u, 1024u);
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks)
            ptx::umma<false>(d_tmem, ad + ks * ((16 * 128) >> 4), bd + ks * 2, p.idesc, (kb | ks) ? 1u : 0u);
          ptx::umma_commit(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(tfull_bar(acc));
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp < kGatherWarp0) {
    // ===================== epilogue =====================
    const int q = warp & 3;                            // hardware rule: a warp reads TMEM lanes 32*(warp%4)..+31
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
      const long long pt = t / p.n_tiles;
      const int nt = static_cast<int>(t - pt * p.n_tiles);
      const long long pos = pt * kBM + q * 32 + lane;
      const bool pos_ok = pos < p.P;
      const int n = static_cast<int>((pos_ok ? pos : 0) / p.HWo);
      const int hw = static_cast<int>((pos_ok ? pos : 0) - static_cast<long long>(n) * p.HWo);
      const long long off0 = n * p.out_img_pitch + hw;
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag));
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * kBN + (static_cast<uint32_t>(q * 32) << 16);
      const int co_tile = nt * kBN;
      const int chunks = min(kBN / 32, (p.Cout - co_tile + 31) / 32);
      for (int c = 0; c < chunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(t_row + c * 32, r);
        ptx::tmem_wait_ld();
        if (c == chunks - 1) {
          // the accumulator is in registers: the MMA warp may start the tile after next
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        }
        if (pos_ok) {
          const int co0 = co_tile + c * 32;
          const long long off = off0 + static_cast<long long>(co0) * p.HWo;
          switch (p.act) {
            case kActReLU:    epilogue_chunk<kActReLU>(p, r, co0, off); break;
            case kActLeaky:   epilogue_chunk<kActLeaky>(p, r, co0, off); break;
            case kActGELU:    epilogue_chunk<kActGELU>(p, r, co0, off); break;
            case kActSigmoid: epilogue_chunk<kActSigmoid>(p, r, co0, off); break;
            case kActTanh:    epilogue_chunk<kActTanh>(p, r, co0, off); break;
            default:          epilogue_chunk<kActNone>(p, r, co0, off); break;
          }
        }
      }
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
    ptx::tc_fence_before_sync();
  } else {
    // ===================== gather of the Col tile =====================
    // Every gather warp produces whole stages (the stage's running index modulo the number of gather warps picks the
    // warp), so that as many stages are being fetched at once as the ring has slots: one stage is one round trip to
    // L2 per batch of loads, and only several in flight hide it.  A stage holds 16 position chunks x 64 k rows; a
    // half-warp covers the 16 chunks of one k row (256 bytes of positions, contiguous in the input at unit stride).
    const int g = warp - kGatherWarp0;
    const int chunk = lane & 15, r_half = lane >> 4;
    const int t_first = (g / kSpan) * kStepsPerWarp;    // this warp's share of the stage's row steps
    const uint32_t chunk_off = static_cast<uint32_t>(chunk >> 3) * (kBK * 128);
    constexpr int kBatch = 8;                           // chunks whose loads a thread issues before it uses the first
    long long idx = 0;                                  // running index of the stage fills of this CTA
    bool ok = true;
    for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
      const long long pt = t / p.n_tiles;
      const long long p0 = pt * kBM + chunk * 8;
      const bool pos_on = p0 < p.P;
      const Pos q = decode_pos(p, pos_on ? p0 : 0);
      const unsigned short* img = p.X + q.n * p.img_pitch;
      const long long left = p.P - p0;
      const int valid = left < 8 ? static_cast<int>(left) : 8;
      for (int kb = 0; kb < p.k_blocks; ++kb, ++idx) {
        if (static_cast<int>(idx % kSpan) != g % kSpan) continue;
        const int stage = static_cast<int>(idx % kStages);
        const uint32_t phase = static_cast<uint32_t>(idx / kStages) & 1u;
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag));
        if (!ok) break;
        uint8_t* a_stage = smem + stage * kStageBytes + chunk_off;
        if (p.fast) {
#pragma unroll 1
          for (int t0 = t_first; t0 < t_first + kStepsPerWarp; t0 += kBatch) {
            RawChunk raw[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              const int k = kb * kBK + 2 * (t0 + u) + r_half;
              const bool on = pos_on && k < p.K;
              const int c = on ? channel_of(p, k) : 0;
              raw[u] = gather_issue(p, img + c * p.plane_pitch, tap_s[on ? k - c * p.taps : 0], q.ho, q.wo, on);
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              const int r = 2 * (t0 + u) + r_half;
              *reinterpret_cast<uint4*>(a_stage + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) = gather_finish(raw[u]);
            }
          }
        } else {
#pragma unroll 2
          for (int t0 = t_first; t0 < t_first + kStepsPerWarp; ++t0) {
            const int r = 2 * t0 + r_half;
            const int k = kb * kBK + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (pos_on && k < p.K) {
              const int c = channel_of(p, k);
              v = gather_general(p, img + c * p.plane_pitch, tap_s[k - c * p.taps], q.ho, q.wo, valid);
            }
            *reinterpret_cast<uint4*>(a_stage + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) = v;
          }
        }
        ptx::fence_proxy_async_smem();                 // the MMA reads the stage through the async proxy
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(full_bar(stage));
      }
    }
  }

  __syncthreads();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0) atomicOr(p.status, kErrWaitTimeout);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }      // copies in flight land before the memory goes away
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int kBN, int kStages>
int launch_cfg(const CUtensorMap& tmW, ConvParams& p, cudaStream_t s) {
  constexpr int kSmem = kStages * (kAStageBytes + kBN * 128) + 8 * (2 * kStages + 4) + 16 + kConvMaxTaps * 4 + 1024;
  static_assert(kSmem <= 232448, "convolution stages exceed the shared memory of one SM");
  auto kernel = conv_implicit_kernel<kBN, kStages>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] { attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem); });
  if (attr_err != cudaSuccess) return kCudaError;
  p.n_tiles = (p.Cout + kBN - 1) / kBN;
  p.idesc = ptx::make_idesc(p.y_dtype == kBF16 ? 1 : 0, true, false, kBM, kBN);
  const long long tiles = static_cast<long long>(p.pos_tiles) * p.n_tiles;
  const long long grid = tiles < sm_budget() ? tiles : sm_budget();
  kernel<<<static_cast<unsigned>(grid), kConvThreads, kSmem, s>>>(tmW, p);
  if (cudaGetLastError() != cudaSuccess) return kCudaError;
  note_tensor_launch(1);
  return kOk;
}

// ---------------------------------------------------------------------------------------------------------------
// Weight gradient  dW[co][k] = sum over images and output positions of gZ[n][co][pos] . Col[n][k][pos],  k = (c, kh, kw)
// as D[k][co] (128 k rows on the TMEM lanes) with the reduction over blocks of 64 positions.  Both operands have the
// reduction index contiguous: the Col tile (128 k rows x 64 positions) is gathered as above, the gZ tile (Cout rows x
// 64 positions) comes by TMA (positions past the end of an image read as zero).  The blocks of the batch are cut
// into `split` slices per output tile so that every SM has work; a slice stores its fp32 partial tile to
// part[slice][co][k] and wgrad_finish_kernel adds the slices in index order (same result on every run).
template <int kBN, int kStages>
__global__ void __launch_bounds__(kConvThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmG, const __grid_constant__ ConvParams p) {
  constexpr int kBStageBytes = kBN * 128;
  constexpr int kStageBytes = kAStageBytes + kBStageBytes;
  constexpr int kTmemCols = 2 * kBN;
  // Stage fills are dealt round-robin to kSpan groups of gather warps.  A group's next fill is kSpan fills after its
  // last one; kSpan <= kStages keeps it less than two laps of the ring ahead of the consumer, which is what the
  // one-bit phase of the empty barriers can tell apart.
  constexpr int kSpan = kStages >= kGatherWarps ? kGatherWarps : 4;
  constexpr int kWarpsPerStage = kGatherWarps / kSpan;
  constexpr int kStepsPerWarp = 32 / kWarpsPerStage;     // of the 32 row steps of one stage
  static_assert(kSpan <= kStages && kGatherWarps % kSpan == 0, "gather groups and ring depth do not fit");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t base = raw_addr + pad;
  uint8_t* tail = smem + kStages * kStageBytes;
  const uint32_t bar0 = base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(tail + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * (2 * kStages + 4) + 8);
  short2* tap_s = reinterpret_cast<short2*>(tail + 8 * (2 * kStages + 4) + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long units = static_cast<long long>(p.m_tiles) * p.n_tiles * p.split;
  // unit -> (k tile, channel tile, slice) and the slice's range of position blocks
  struct Unit { int mt, nt, sl, b0, b1; };
  auto decode_unit = [&](long long u) {
    Unit w;
    w.sl = static_cast<int>(u % p.split);
    const long long t = u / p.split;
    w.nt = static_cast<int>(t % p.n_tiles);
    w.mt = static_cast<int>(t / p.n_tiles);
    w.b0 = w.sl * p.per;
    w.b1 = min(w.b0 + p.per, p.red_blocks);
    return w;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1 + kWarpsPerStage); ptx::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), kEpiWarpsConv); }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmG);
  }
  for (int t = threadIdx.x; t < p.taps; t += kConvThreads) tap_s[t] = p.tap_off[t];
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ===================== gZ tiles by TMA =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (long long u = blockIdx.x; ok && u < units; u += gridDim.x) {
        const Unit w = decode_unit(u);
        for (int b = w.b0; b < w.b1; ++b) {
          const int n = b / p.bpi, j = b - n * p.bpi;
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(full_bar(stage), kBStageBytes);
          ptx::tma_load_3d(base + stage * kStageBytes + kAStageBytes, &tmG, full_bar(stage), j * 64, w.nt * kBN, n);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (long long u = blockIdx.x; ok && u < units; u += gridDim.x) {
        const Unit w = decode_unit(u);
        if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int b = w.b0; b < w.b1; ++b) {
          if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = base + stage * kStageBytes;
          // both tiles: 128-byte rows of 64 positions, 8-row groups 1024 bytes apart, 32 bytes per MMA step
          const uint64_t ad = ptx::make_smem_desc_sw128(a_addr, 0u, 1024u);
          const uint64_t bd = ptx::make_smem_desc_sw128(a_addr + kAStageBytes, 0u, 1024u);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ptx::umma<false>(d_tmem, ad + ks * 2, bd + ks * 2, p.idesc, (b > w.b0 || ks) ? 1u : 0u);
          ptx::umma_commit(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(tfull_bar(acc));
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp < kGatherWarp0) {
    // ===================== epilogue: partial tile -> part[slice][co][k] =====================
    const int q = warp & 3;
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    for (long long u = blockIdx.x; ok && u < units; u += gridDim.x) {
      const Unit w = decode_unit(u);
      const int k = w.mt * kBM + q * 32 + lane;
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag));
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * kBN + (static_cast<uint32_t>(q * 32) << 16);
      const int co_tile = w.nt * kBN;
      const int chunks = min(kBN / 32, (p.Cout - co_tile + 31) / 32);
      float* dst = p.part + (static_cast<long long>(w.sl) * p.Cout + co_tile) * p.K + k;
      for (int c = 0; c < chunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(t_row + c * 32, r);
        ptx::tmem_wait_ld();
        if (c == chunks - 1) {
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        }
        if (k < p.K) {
          const int n_co = min(32, p.Cout - (co_tile + c * 32));
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < n_co) dst[static_cast<long long>(c * 32 + j) * p.K] = __uint_as_float(r[j]);
        }
      }
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
    ptx::tc_fence_before_sync();
  } else {
    // ===================== gather of the Col tile (128 k rows x 8 position chunks per stage) =====================
    // As in the forward kernel every gather warp produces whole stages.  Eight lanes cover the 8 chunks of one k row
    // (128 bytes of positions), a warp four rows per step.
    const int g = warp - kGatherWarp0;
    const int chunk = lane & 7, r_quarter = lane >> 3;
    const int t_first = (g / kSpan) * kStepsPerWarp;
    constexpr int kBatch = 8;
    long long idx = 0;
    bool ok = true;
    for (long long u = blockIdx.x; ok && u < units; u += gridDim.x) {
      const Unit w = decode_unit(u);
      for (int b = w.b0; b < w.b1; ++b, ++idx) {
        if (static_cast<int>(idx % kSpan) != g % kSpan) continue;
        const int stage = static_cast<int>(idx % kStages);
        const uint32_t phase = static_cast<uint32_t>(idx / kStages) & 1u;
        const int n = b / p.bpi, j = b - n * p.bpi;
        const int hw0 = j * 64 + chunk * 8;
        const int valid = min(8, p.HWo - hw0);          // <= 0: the chunk lies past the end of the image
        const int ho = hw0 / p.Wo, wo = hw0 - ho * p.Wo;
        const unsigned short* img = p.X + n * p.img_pitch;
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag));
        if (!ok) break;
        uint8_t* a_stage = smem + stage * kStageBytes;
        if (p.fast) {
#pragma unroll 1
          for (int t0 = t_first; t0 < t_first + kStepsPerWarp; t0 += kBatch) {
            RawChunk raw[kBatch];
#pragma unroll
            for (int v = 0; v < kBatch; ++v) {
              const int k = w.mt * kBM + 4 * (t0 + v) + r_quarter;
              const bool on = valid > 0 && k < p.K;
              const int c = on ? channel_of(p, k) : 0;
              raw[v] = gather_issue(p, img + c * p.plane_pitch, tap_s[on ? k - c * p.taps : 0], ho, wo, on);
            }
#pragma unroll
            for (int v = 0; v < kBatch; ++v) {
              const int r = 4 * (t0 + v) + r_quarter;
              *reinterpret_cast<uint4*>(a_stage + r * 128 + ((chunk ^ (r & 7)) << 4)) = gather_finish(raw[v]);
            }
          }
        } else {
#pragma unroll 2
          for (int t0 = t_first; t0 < t_first + kStepsPerWarp; ++t0) {
            const int r = 4 * t0 + r_quarter;
            const int k = w.mt * kBM + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (valid > 0 && k < p.K) {
              const int c = channel_of(p, k);
              v = gather_general(p, img + c * p.plane_pitch, tap_s[k - c * p.taps], ho, wo, valid);
            }
            *reinterpret_cast<uint4*>(a_stage + r * 128 + ((chunk ^ (r & 7)) << 4)) = v;
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(full_bar(stage));
      }
    }
  }

  __syncthreads();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0) atomicOr(p.status, kErrWaitTimeout);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// dW[i] = sum over slices, in slice order, of part[slice][i]   (i over Cout * K)
__global__ void wgrad_finish_kernel(const float* __restrict__ part, void* __restrict__ dW, long long elems, int split,
                                    int dt) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < elems; i += gridDim.x * 256ll) {
    float acc = 0.f;
    for (int s = 0; s < split; ++s) acc += part[static_cast<long long>(s) * elems + i];
    store_from_f32(dW, i, dt, acc);
  }
}

template <int kBN, int kStages>
int launch_wgrad_cfg(const CUtensorMap& tmG, ConvParams& p, cudaStream_t s) {
  constexpr int kSmem = kStages * (kAStageBytes + kBN * 128) + 8 * (2 * kStages + 4) + 16 + kConvMaxTaps * 4 + 1024;
  auto kernel = conv_wgrad_kernel<kBN, kStages>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] { attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem); });
  if (attr_err != cudaSuccess) return kCudaError;
  const long long units = static_cast<long long>(p.m_tiles) * p.n_tiles * p.split;
  const long long grid = units < sm_budget() ? units : sm_budget();
  kernel<<<static_cast<unsigned>(grid), kConvThreads, kSmem, s>>>(tmG, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

__global__ void transpose_weight_kernel(const unsigned short* __restrict__ W, unsigned short* __restrict__ Wt, int Cout,
                                        int Cin, int taps, long long ldt) {
  // Wt[ci][co * taps + t] = W[(co * Cin + ci) * taps + t]
  const long long total = static_cast<long long>(Cout) * Cin * taps;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const int t = static_cast<int>(i % taps);
    const long long r = i / taps;
    const int co = static_cast<int>(r % Cout), ci = static_cast<int>(r / Cout);
    Wt[ci * ldt + static_cast<long long>(co) * taps + t] = W[(static_cast<long long>(co) * Cin + ci) * taps + t];
  }
}

}  // namespace

namespace {

// Fields of ConvParams that describe the gathered input; shared by the two launchers.
int fill_gather_params(const ImplicitConv& d, ConvParams& p) {
  p.X = static_cast<const unsigned short*>(d.X);
  p.img_pitch = d.img_pitch; p.plane_pitch = d.plane_pitch; p.row_pitch = d.row_pitch;
  p.H = d.H; p.W = d.W; p.Wo = d.Wo; p.HWo = d.Ho * d.Wo;
  p.sh = d.sh; p.sw = d.sw;
  p.taps = d.taps;
  p.K = d.K; p.k_blocks = (d.K + kBK - 1) / kBK;
  p.tap_magic = d.taps > 1 ? static_cast<unsigned>(((1ull << 32) + d.taps - 1) / d.taps) : 0u;
  // the multiply-high division must be exact for every k a gather thread forms (k < K rounded up to a tile)
  const long long k_end = (static_cast<long long>(d.K) + kBM - 1) / kBM * kBM;
  for (long long k = 0; k < k_end && d.taps > 1; ++k)
    if (static_cast<long long>((static_cast<unsigned long long>(k) * p.tap_magic) >> 32) != k / d.taps) return kUnimplemented;
  p.Cout = d.Cout;
  // aligned 16-byte gather: unit column stride, chunks of 8 positions inside one output row, rows on 16-byte boundaries
  p.fast = (d.sw == 1 && d.Wo % 8 == 0 && d.W % 8 == 0 && d.row_pitch % 8 == 0 && d.plane_pitch % 8 == 0 &&
            d.img_pitch % 8 == 0 && (reinterpret_cast<uintptr_t>(d.X) & 15u) == 0) ? 1 : 0;
  if (d.force_general) p.fast = 0;
  p.status = device_status_ptr();
  if (!p.status) return kCudaError;
  for (int t = 0; t < d.taps; ++t) p.tap_off[t] = make_short2(static_cast<short>(d.tap_row[t]), static_cast<short>(d.tap_col[t]));
  return kOk;
}

bool gather_shape_ok(const ImplicitConv& d) {
  if (!(d.dtype == kBF16 || d.dtype == kF16)) return false;
  if (d.taps < 1 || d.taps > kConvMaxTaps || d.K < 1 || d.K > (1 << 24)) return false;
  for (int t = 0; t < d.taps; ++t)
    if (d.tap_row[t] < -32768 || d.tap_row[t] > 32767 || d.tap_col[t] < -32768 || d.tap_col[t] > 32767) return false;
  return tc::driver_has_tensor_maps();
}

int wgrad_tile_n(int Cout) { return Cout <= 64 ? 64 : (Cout <= 128 ? 128 : 256); }

}  // namespace

bool conv_implicit_supported(const ImplicitConv& d) {
  if (!gather_shape_ok(d)) return false;
  if (d.P < 1 || d.P > (1ll << 40) || (d.P + kBM - 1) / kBM > 0x7fffffffll) return false;
  if ((d.ldw * 2) % 16 != 0 || (reinterpret_cast<uintptr_t>(d.Wm) & 15u) != 0) return false;
  return true;
}

int conv_implicit_launch(const ImplicitConv& d, cudaStream_t s) {
  if (!conv_implicit_supported(d)) return kUnimplemented;
  ConvParams p{};
  const int rc = fill_gather_params(d, p);
  if (rc != kOk) return rc;
  p.P = d.P;
  p.pos_tiles = static_cast<int>((d.P + kBM - 1) / kBM);
  p.Y = d.Y; p.Z = d.Z; p.bias = d.bias;
  p.out_img_pitch = d.out_img_pitch;
  p.y_dtype = d.dtype; p.z_dtype = d.Z ? d.z_dtype : d.dtype; p.act = d.act; p.leaky = d.leaky;
  const int bn = d.Cout <= 64 ? 64 : (d.Cout <= 128 ? 128 : 256);
  CUtensorMap tmW;
  if (!tc::make_operand_map(&tmW, d.dtype, d.Wm, d.K, d.Cout, d.ldw, 1, 0, kBK, bn, false)) return kCudaError;
  switch (bn) {
    case 64:  return launch_cfg<64, 9>(tmW, p, s);
    case 128: return launch_cfg<128, 7>(tmW, p, s);
    default:  return launch_cfg<256, 4>(tmW, p, s);
  }
}

bool conv_wgrad_plan(const ImplicitWgrad& w, int* split, size_t* part_bytes) {
  const ImplicitConv& d = w.in;
  if (!gather_shape_ok(d) || w.imgs < 1 || d.Ho < 1 || d.Wo < 1) return false;
  if ((reinterpret_cast<uintptr_t>(w.G) & 15u) != 0 || (w.g_plane_pitch * 2) % 16 != 0 || (w.g_img_pitch * 2) % 16 != 0)
    return false;
  const long long hwo = static_cast<long long>(d.Ho) * d.Wo;
  const long long bpi = (hwo + 63) / 64, red = bpi * w.imgs;
  if (red > 0x7fffffffll) return false;
  const int bn = wgrad_tile_n(d.Cout);
  const long long tiles = static_cast<long long>((d.K + kBM - 1) / kBM) * ((d.Cout + bn - 1) / bn);
  long long sp = sm_budget() / tiles;
  if (sp > red / 8) sp = red / 8;                        // a slice sums at least 8 blocks before it stores a tile
  if (sp < 1) sp = 1;
  const long long per = (red + sp - 1) / sp;
  sp = (red + per - 1) / per;
  *split = static_cast<int>(sp);
  *part_bytes = static_cast<size_t>(sp) * d.Cout * d.K * sizeof(float);
  return true;
}

int conv_wgrad_launch(const ImplicitWgrad& w, cudaStream_t s) {
  const ImplicitConv& d = w.in;
  int split = 0; size_t need = 0;
  if (!conv_wgrad_plan(w, &split, &need)) return kUnimplemented;
  if (!w.part || w.part_bytes < need || !w.dW) return kBadArgs;
  ConvParams p{};
  const int rc = fill_gather_params(d, p);
  if (rc != kOk) return rc;
  const int bn = wgrad_tile_n(d.Cout);
  p.bpi = (p.HWo + 63) / 64;
  p.red_blocks = p.bpi * w.imgs;
  p.split = split;
  p.per = (p.red_blocks + split - 1) / split;
  p.m_tiles = (d.K + kBM - 1) / kBM;
  p.n_tiles = (d.Cout + bn - 1) / bn;
  p.part = w.part;
  p.idesc = ptx::make_idesc(d.dtype == kBF16 ? 1 : 0, false, false, kBM, bn);
  CUtensorMap tmG;
  if (!tc::make_operand_map(&tmG, d.dtype, w.G, p.HWo, d.Cout, w.g_plane_pitch, w.imgs, w.g_img_pitch, 64, bn, false))
    return kCudaError;
  int lrc;
  switch (bn) {
    case 64:  lrc = launch_wgrad_cfg<64, 9>(tmG, p, s); break;
    case 128: lrc = launch_wgrad_cfg<128, 7>(tmG, p, s); break;
    default:  lrc = launch_wgrad_cfg<256, 4>(tmG, p, s); break;
  }
  if (lrc != kOk) return lrc;
  const long long elems = static_cast<long long>(d.Cout) * d.K;
  long long blocks = (elems + 255) / 256;
  if (blocks > 4096) blocks = 4096;
  wgrad_finish_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(w.part, w.dW, elems, split, d.dtype);
  if (cudaGetLastError() != cudaSuccess) return kCudaError;
  note_tensor_launch(2);
  return kOk;
}

cudaError_t launch_transpose_weight(const void* W, void* Wt, int Cout, int Cin, int taps, long long ldt, cudaStream_t s) {
  const long long total = static_cast<long long>(Cout) * Cin * taps;
  long long blocks = (total + 255) / 256;
  if (blocks > 2048) blocks = 2048;
  transpose_weight_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      static_cast<const unsigned short*>(W), static_cast<unsigned short*>(Wt), Cout, Cin, taps, ldt);
  return cudaGetLastError();
}

}  // namespace ge2b
