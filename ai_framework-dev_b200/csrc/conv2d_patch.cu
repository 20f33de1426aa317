// Unit-stride 2-D convolution as an implicit GEMM whose operand tiles are WINDOWS of one input patch in shared memory.
//
// The reference materialises Col = im2col(X[n]) in global memory and multiplies it with the packed weight
// (backends/cuda/ops/conv2d/launcher.cu:180-227, kernels.cu:12-45).  Here nothing of Col exists anywhere: in the
// zero-padded coordinates of one image (rows of Wp = W + 2*pad_w pixels) the input pixel that output position u needs
// for tap (kh, kw) is pixel u + kh*dil_h*Wp + kw*dil_w, a pure shift.  So a CTA that owns 128 consecutive padded
// output positions of one image
//   * copies the input pixels [u0, u0 + 128 + largest shift) of 64 channels into shared memory ONCE, position-major
//     (a pixel's channels side by side, 16 bytes = 8 channels per cell, cells of one channel group 16 bytes apart), and
//   * issues, per tap, tcgen05.mma with an A descriptor that simply starts `shift` rows further down the patch:
//     every element of the patch feeds Kh*Kw MMAs and no per-tap data movement happens at all.
// The patch layout is the canonical un-swizzled reduction-contiguous operand layout (8 x 16-byte core matrices, 128
// bytes from one 8-row group to the next, one channel group every R*16 bytes), which is what lets a window start at
// any row: only the 16-byte start address changes.  The weight is re-laid as Wr[Cout][tap][channel] by a small kernel
// and comes in by TMA (128-byte swizzle); accumulators live in TMEM (positions on the lanes, channels on the
// columns); the epilogue adds the per-channel bias, applies the activation and writes Y / Z in NCHW, skipping the
// lanes that fall into the padding columns.  The input gradient of the same convolution is this kernel run on gZ with
// the weight flipped and transposed.
//     warp 0      TMA producer of the weight tiles         warp 1      MMA issuer
//     warps 2..5  epilogue (one TMEM lane quarter each)    warps 6..13 patch fill (NCHW -> position-major)
// Every mbarrier wait is bounded (sm100_ptx.cuh); on expiry the CTA records kErrWaitTimeout in the device status
// word, frees its TMEM and returns.  No TMA load uses cluster multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

#include "conv2d_implicit.hpp"
#include "epilogue_math.cuh"
#include "gemm_tc_kernel.cuh"
#include "sm100_ptx.cuh"

namespace ge2b {
namespace {

constexpr int kPM = 128;                  // padded output positions per tile (one TMEM lane each)
constexpr int kPThreads = 448;
constexpr int kPEpiWarps = 4;             // warps 2..5
constexpr int kFillWarp0 = 6, kFillWarps = 8;
constexpr int kFillThreads = kFillWarps * 32;

struct PatchParams {
  const unsigned short* X;                // input planes [image][channel][row][column], 16-bit elements
  long long img_pitch, plane_pitch; int row_pitch;
  int Cin, H, W, ph, pw;                  // channels, plane extent, zero border above / left of the plane
  int Wp, Hp;                             // padded extent: W + 2 pw, H + 2 ph
  int Ho, Wo;                             // output extent
  int tiles_per_img, n_tiles, cblocks;    // 128-position tiles per image, channel tiles of the output, 64-channel blocks
  long long tiles;                        // images * tiles_per_img * n_tiles
  int taps, Cp;                           // Kh * Kw; channels rounded up to 64 (row length of one tap in Wr)
  int R, R_alloc;                         // patch rows used (128 + largest shift) / allocated (== 1 mod 8)
  int V;                                  // elements per fill load: 8, 4, 2 or 1
  int Cout;
  void* Y; void* Z; const float* bias;
  long long out_img_pitch;                // elements from image to image in Y / Z
  int out_plane, out_row_pitch;           // elements from channel plane to plane / row to row of the output
  int osh, osw, out_off;                  // output pixel of position (ho, wq): row ho*osh, column wq*osw, plus out_off
  int y_dtype, z_dtype, act;
  float leaky;
  uint32_t idesc;
  int* status;
  int shift[kConvMaxTaps];                // per tap: rows down the patch = kh*dil_h*Wp + kw*dil_w
};

template <bool kBf16>
__device__ __forceinline__ uint32_t to_bits16(float v) {
  if constexpr (kBf16) return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
  else                 return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(v)));
}

// 32 channels co0 .. co0+31 of one output position; `off` is the element offset of (image, co0, position) in Y / Z.
// kZ: 0 no pre-activation output, 1 in the tensors' 16-bit type, 2 fp32.  `bias_s`: the channel tile's biases in
// shared memory (zeros when the layer has none).
template <int ACT, bool kBf16, int kZ>
__device__ __forceinline__ void patch_epilogue_chunk(const PatchParams& p, const uint32_t (&r)[32], const float* bias_s,
                                                     int n_co, long long off, int plane, bool pos_ok) {
  if (!pos_ok) return;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (j < n_co) {
      const float v = __uint_as_float(r[j]) + bias_s[j];
      const long long o = off + static_cast<long long>(j) * plane;
      if constexpr (kZ == 2) static_cast<float*>(p.Z)[o] = v;
      if constexpr (kZ == 1) static_cast<unsigned short*>(p.Z)[o] = static_cast<unsigned short>(to_bits16<kBf16>(v));
      static_cast<unsigned short*>(p.Y)[o] = static_cast<unsigned short>(to_bits16<kBf16>(act_fwd<ACT, true>(v, p.leaky)));
    }
  }
}

// The same with two positions per store: an even lane and its odd neighbour hold two adjacent positions of one output
// row; for every pair of channels they swap one value each, so that the even lane writes both positions of the even
// channel and the odd lane both positions of the odd channel as one 32-bit store (Y and a 16-bit Z travel through the
// swap packed in one word).  Needs even Wo and Wp (then a pair never straddles a row end and starts on a 4-byte
// boundary) and kZ < 2; the warp calls it converged, lanes without a valid position only swap.
template <int ACT, bool kBf16, int kZ>
__device__ __forceinline__ void patch_epilogue_chunk_pairs(const PatchParams& p, const uint32_t (&r)[32],
                                                           const float* bias_s, int n_co, long long off, int plane,
                                                           bool pos_ok, int lane) {
  const bool odd = (lane & 1) != 0;
  // element offset of the pair's first position in this lane's channel of the first channel pair
  const long long off_pair = (odd ? off - 1 + plane : off);
  uint32_t* y32 = static_cast<uint32_t*>(p.Y);
  uint32_t* z32 = static_cast<uint32_t*>(p.Z);
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    const float v0 = __uint_as_float(r[j]) + bias_s[j], v1 = __uint_as_float(r[j + 1]) + bias_s[j + 1];
    uint32_t w0 = to_bits16<kBf16>(act_fwd<ACT, true>(v0, p.leaky)), w1 = to_bits16<kBf16>(act_fwd<ACT, true>(v1, p.leaky));
    if constexpr (kZ == 1) { w0 |= to_bits16<kBf16>(v0) << 16; w1 |= to_bits16<kBf16>(v1) << 16; }
    const uint32_t got = __shfl_xor_sync(0xffffffffu, odd ? w0 : w1, 1);
    const uint32_t mine = odd ? w1 : w0;
    const uint32_t lo = odd ? got : mine, hi = odd ? mine : got;     // first / second position of the pair
    if (pos_ok && j + (odd ? 1 : 0) < n_co) {
      const long long o = (off_pair + static_cast<long long>(j) * plane) >> 1;
      y32[o] = __byte_perm(lo, hi, 0x5410);
      if constexpr (kZ == 1) z32[o] = __byte_perm(lo, hi, 0x7632);
    }
  }
}

// One fill item: V consecutive pixels of one channel (one load), scattered to V patch rows.
template <int V> struct Piece;
template <> struct Piece<8> { uint4 d; };
template <> struct Piece<4> { uint2 d; };
template <> struct Piece<2> { uint32_t d; };
template <> struct Piece<1> { unsigned short d; };
template <int V>
__device__ __forceinline__ Piece<V> piece_load(const unsigned short* src, bool on) {
  Piece<V> r;
  if constexpr (V == 8)      r.d = on ? __ldg(reinterpret_cast<const uint4*>(src)) : make_uint4(0u, 0u, 0u, 0u);
  else if constexpr (V == 4) r.d = on ? __ldg(reinterpret_cast<const uint2*>(src)) : make_uint2(0u, 0u);
  else if constexpr (V == 2) r.d = on ? __ldg(reinterpret_cast<const uint32_t*>(src)) : 0u;
  else                       r.d = on ? __ldg(src) : static_cast<unsigned short>(0);
  return r;
}
template <int V>
__device__ __forceinline__ unsigned short piece_elem(const Piece<V>& r, int j) {
  if constexpr (V == 8) {
    const uint32_t w = j < 2 ? r.d.x : (j < 4 ? r.d.y : (j < 6 ? r.d.z : r.d.w));
    return static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xffffu));
  } else if constexpr (V == 4) {
    const uint32_t w = j < 2 ? r.d.x : r.d.y;
    return static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xffffu));
  } else if constexpr (V == 2) {
    return static_cast<unsigned short>(j ? (r.d >> 16) : (r.d & 0xffffu));
  } else {
    return r.d;
  }
}

// Fills one patch: pixels [u0, u0 + R) (padded coordinates of image n) of channels [c0, c0 + 64), zero where the pixel
// lies in the border or the channel does not exist.  Called by all fill warps; `ft` is the thread's index among them.
// The fill warps meet between the zeroing and the scatter at an mbarrier (`zero_bar`, one arrival per warp) so that
// the wait is bounded like every other wait of the kernel; false: the wait was given up.
template <int V>
__device__ __forceinline__ bool fill_patch(const PatchParams& p, uint8_t* patch, int n, int c0, int u0, int ft,
                                           uint32_t zero_bar, uint32_t zero_parity, volatile int* abort_flag) {
  // zero everything first (border pixels, missing channels, rows past the image), then scatter the real pixels
  for (int i = ft; i < p.R_alloc * 8; i += kFillThreads)
    *reinterpret_cast<uint4*>(patch + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  const int lane = ft & 31, fw = ft >> 5;
  __syncwarp();
  if (lane == 0) ptx::mbar_arrive(zero_bar);
  if (!__all_sync(0xffffffffu, ptx::mbar_wait(zero_bar, zero_parity, abort_flag))) return false;
  const int hp_lo = u0 / p.Wp, hp_hi = min((u0 + p.R - 1) / p.Wp, p.Hp - 1);
  const int hi_lo = max(hp_lo - p.ph, 0), hi_hi = min(hp_hi - p.ph, p.H - 1);
  const int ppr = p.W / V;                                      // loads per input row
  const int items = max(hi_hi - hi_lo + 1, 0) * ppr * 2;        // x 2 halves of 32 channels (one per lane)
  const unsigned short* img = p.X + n * p.img_pitch;
  constexpr int kB = 6;                                         // loads in flight per thread
#pragma unroll 1
  for (int it0 = fw; it0 < items; it0 += kFillWarps * kB) {
    Piece<V> pc[kB]; int v0[kB]; int cl[kB];
#pragma unroll
    for (int b = 0; b < kB; ++b) {
      const int it = it0 + b * kFillWarps;
      const bool on_it = it < items;
      const int rp = it >> 1;
      const int row = rp / ppr, piece = rp - row * ppr;
      const int hi = hi_lo + row;
      cl[b] = (it & 1) * 32 + lane;
      const int c = c0 + cl[b];
      const bool on = on_it && c < p.Cin;
      pc[b] = piece_load<V>(img + c * p.plane_pitch + static_cast<long long>(hi) * p.row_pitch + piece * V, on);
      v0[b] = on ? (hi + p.ph) * p.Wp + p.pw + piece * V - u0 : -(1 << 20);
    }
#pragma unroll
    for (int b = 0; b < kB; ++b) {
      uint8_t* dst = patch + (cl[b] >> 3) * (p.R_alloc * 16) + (cl[b] & 7) * 2;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const int v = v0[b] + j;
        if (static_cast<unsigned>(v) < static_cast<unsigned>(p.R))
          *reinterpret_cast<unsigned short*>(dst + v * 16) = piece_elem<V>(pc[b], j);
      }
    }
  }
  return true;
}

template <int kBN, int kStages>
__global__ void __launch_bounds__(kPThreads, 2)
conv_patch_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ PatchParams p) {
  constexpr int kBStageBytes = kBN * 128;
  constexpr int kTmemCols = 2 * kBN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t base = raw_addr + pad;
  // [weight ring][barriers, 256 bytes][patch 0][patch 1][one copy of the channel tile's biases per epilogue warp]
  uint8_t* tail = smem + kStages * kBStageBytes;
  const uint32_t bar0 = base + kStages * kBStageBytes;
  auto bfull_bar = [&](int s) { return bar0 + 8u * s; };
  auto bempty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto pfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto pempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 4 + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 6 + a); };
  auto pzero_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 8 + b); };
  static_assert(8 * (2 * kStages + 10) + 16 <= 256, "barrier block too small");
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(tail + 8 * (2 * kStages + 10));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * (2 * kStages + 10) + 8);
  const uint32_t patch_bytes = static_cast<uint32_t>(p.R_alloc) * 128u;
  uint8_t* patch_ptr = tail + 256;
  const uint32_t patch_addr = bar0 + 256u;
  float* bias_all = reinterpret_cast<float*>(patch_ptr + 2 * ((patch_bytes + 15u) & ~15u));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // tile -> (image, tile in the image, channel tile)
  struct Tile { int n, j, nt; };
  auto decode_tile = [&](long long t) {
    Tile w;
    w.nt = static_cast<int>(t % p.n_tiles);
    const long long r = t / p.n_tiles;
    w.j = static_cast<int>(r % p.tiles_per_img);
    w.n = static_cast<int>(r / p.tiles_per_img);
    return w;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(bfull_bar(s), 1); ptx::mbar_init(bempty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(pfull_bar(b), kFillWarps); ptx::mbar_init(pempty_bar(b), 1);
      ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), kPEpiWarps);
      ptx::mbar_init(pzero_bar(b), kFillWarps);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmW);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ===================== weight tiles by TMA: per (channel block, tap) one tile of kBN x 64 =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (long long t = blockIdx.x; ok && t < p.tiles; t += gridDim.x) {
        const Tile w = decode_tile(t);
        for (int cb = 0; ok && cb < p.cblocks; ++cb)
          for (int tap = 0; tap < p.taps; ++tap) {
            if (!ptx::mbar_wait(bempty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
            ptx::mbar_arrive_expect_tx(bfull_bar(stage), kBStageBytes);
            ptx::tma_load_3d(base + stage * kBStageBytes, &tmW, bfull_bar(stage), tap * p.Cp + cb * 64, w.nt * kBN, 0);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      long long fills = 0;                                      // patches consumed so far: buffer = fills & 1
      const uint32_t lbo = static_cast<uint32_t>(p.R_alloc) * 16u;
      for (long long t = blockIdx.x; ok && t < p.tiles; t += gridDim.x) {
        if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int cb = 0; ok && cb < p.cblocks; ++cb, ++fills) {
          const int buf = static_cast<int>(fills & 1);
          if (!ptx::mbar_wait(pfull_bar(buf), static_cast<uint32_t>(fills >> 1) & 1u, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t pa = patch_addr + buf * patch_bytes;
          for (int tap = 0; tap < p.taps; ++tap) {
            if (!ptx::mbar_wait(bfull_bar(stage), phase, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after_sync();
            // A: window of the patch that starts `shift` rows down; un-swizzled, 8-row groups 128 bytes apart, channel
            // groups R_alloc*16 bytes apart; one MMA consumes 16 channels = two channel groups.
            const uint64_t ad = ptx::make_smem_desc_sw128(pa + static_cast<uint32_t>(p.shift[tap]) * 16u, lbo, 128u, 0u);
            const uint64_t bd = ptx::make_smem_desc_sw128(base + stage * kBStageBytes, 0u, 1024u);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              ptx::umma<false>(d_tmem, ad + static_cast<uint64_t>((2u * lbo * ks) >> 4), bd + ks * 2, p.idesc,
                               (cb | tap | ks) ? 1u : 0u);
            ptx::umma_commit(bempty_bar(stage));
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          ptx::umma_commit(pempty_bar(buf));                    // the patch may be overwritten once these MMAs are done
        }
        if (!ok) break;
        ptx::umma_commit(tfull_bar(acc));
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp < kFillWarp0) {
    // ===================== epilogue =====================
    const int q = warp & 3;                            // hardware rule: a warp reads TMEM lanes 32*(warp%4)..+31
    const int plane = p.out_plane;
    const int zkind = p.Z == nullptr ? 0 : (p.z_dtype == kF32 ? 2 : 1);
    // two positions per store where pairs of lanes map to pairs of pixels of one row on 4-byte boundaries
    const bool pairs = p.osw == 1 && !(p.Wo & 1) && !(p.Wp & 1) && !(p.out_img_pitch & 1) && !(p.out_plane & 1) &&
                       !(p.out_row_pitch & 1) && !(p.out_off & 1) && (p.Z == nullptr || p.z_dtype != kF32) &&
                       !((reinterpret_cast<uintptr_t>(p.Y) | reinterpret_cast<uintptr_t>(p.Z)) & 3);
    float* bias_s = bias_all + (warp - 2) * kBN;
    int bias_nt = -1;
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    for (long long t = blockIdx.x; ok && t < p.tiles; t += gridDim.x) {
      const Tile w = decode_tile(t);
      if (w.nt != bias_nt) {                         // this warp's copy of the channel tile's biases
        __syncwarp();
        for (int i = lane; i < kBN; i += 32) {
          const int co = w.nt * kBN + i;
          bias_s[i] = (p.bias != nullptr && co < p.Cout) ? __ldg(p.bias + co) : 0.f;
        }
        __syncwarp();
        bias_nt = w.nt;
      }
      const int u = w.j * kPM + q * 32 + lane;         // padded position of this lane
      const int ho = u / p.Wp, wq = u - ho * p.Wp;
      const bool pos_ok = ho < p.Ho && wq < p.Wo;
      const long long off0 = w.n * p.out_img_pitch + (pos_ok ? ho * p.osh * p.out_row_pitch + wq * p.osw + p.out_off : 0);
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag));
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * kBN + (static_cast<uint32_t>(q * 32) << 16);
      const int co_tile = w.nt * kBN;
      const int chunks = min(kBN / 32, (p.Cout - co_tile + 31) / 32);
      for (int c = 0; c < chunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(t_row + c * 32, r);
        ptx::tmem_wait_ld();
        if (c == chunks - 1) {
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        }
        {
          const int co0 = co_tile + c * 32;
          const long long off = off0 + static_cast<long long>(co0) * plane;
          const int n_co = min(32, p.Cout - co0);
          const float* bs = bias_s + c * 32;
#define GE2B_PATCH_EPI3(ACT_, BF_, Z_)                                                                        \
          do {                                                                                                \
            if (pairs) patch_epilogue_chunk_pairs<ACT_, BF_, (Z_ == 2 ? 0 : Z_)>(p, r, bs, n_co, off, plane, pos_ok, lane); \
            else       patch_epilogue_chunk<ACT_, BF_, Z_>(p, r, bs, n_co, off, plane, pos_ok);               \
          } while (0)
#define GE2B_PATCH_EPI2(ACT_, BF_)                                                                            \
          do {                                                                                                \
            if (zkind == 0)      GE2B_PATCH_EPI3(ACT_, BF_, 0);                                               \
            else if (zkind == 1) GE2B_PATCH_EPI3(ACT_, BF_, 1);                                               \
            else                 GE2B_PATCH_EPI3(ACT_, BF_, 2);                                               \
          } while (0)
#define GE2B_PATCH_EPI(ACT_)                                                                                  \
          do {                                                                                                \
            if (p.y_dtype == kBF16) GE2B_PATCH_EPI2(ACT_, true);                                              \
            else                    GE2B_PATCH_EPI2(ACT_, false);                                             \
          } while (0)
          switch (p.act) {
            case kActReLU:    GE2B_PATCH_EPI(kActReLU); break;
            case kActLeaky:   GE2B_PATCH_EPI(kActLeaky); break;
            case kActGELU:    GE2B_PATCH_EPI(kActGELU); break;
            case kActSigmoid: GE2B_PATCH_EPI(kActSigmoid); break;
            case kActTanh:    GE2B_PATCH_EPI(kActTanh); break;
            default:          GE2B_PATCH_EPI(kActNone); break;
          }
#undef GE2B_PATCH_EPI
#undef GE2B_PATCH_EPI2
#undef GE2B_PATCH_EPI3
        }
      }
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
    ptx::tc_fence_before_sync();
  } else {
    // ===================== patch fill =====================
    const int ft = threadIdx.x - kFillWarp0 * 32;
    long long fills = 0;
    bool ok = true;
    for (long long t = blockIdx.x; ok && t < p.tiles; t += gridDim.x) {
      const Tile w = decode_tile(t);
      for (int cb = 0; cb < p.cblocks; ++cb, ++fills) {
        const int buf = static_cast<int>(fills & 1);
        ok = __all_sync(0xffffffffu,
                        ptx::mbar_wait(pempty_bar(buf), (static_cast<uint32_t>(fills >> 1) & 1u) ^ 1u, abort_flag));
        if (!ok) break;
        uint8_t* patch = patch_ptr + buf * patch_bytes;
        const uint32_t zb = pzero_bar(buf), zp = static_cast<uint32_t>(fills >> 1) & 1u;
        switch (p.V) {
          case 8:  ok = fill_patch<8>(p, patch, w.n, cb * 64, w.j * kPM, ft, zb, zp, abort_flag); break;
          case 4:  ok = fill_patch<4>(p, patch, w.n, cb * 64, w.j * kPM, ft, zb, zp, abort_flag); break;
          case 2:  ok = fill_patch<2>(p, patch, w.n, cb * 64, w.j * kPM, ft, zb, zp, abort_flag); break;
          default: ok = fill_patch<1>(p, patch, w.n, cb * 64, w.j * kPM, ft, zb, zp, abort_flag); break;
        }
        if (!ok) break;
        ptx::fence_proxy_async_smem();                 // the MMA reads the patch through the async proxy
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(pfull_bar(buf));
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

// Wr[o][t * Cp + c] = W[o * so + c * sc + map.src[t]] for the taps t the convolution uses, zero for c >= C.
struct TapMap { int src[kConvMaxTaps]; };
__global__ void relayout_weight_kernel(const unsigned short* __restrict__ W, unsigned short* __restrict__ Wr, int rows,
                                       int C, int Cp, int taps, long long so, long long sc, const TapMap map) {
  const long long total = static_cast<long long>(rows) * taps * Cp;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const int c = static_cast<int>(i % Cp);
    const long long r = i / Cp;
    const int t = static_cast<int>(r % taps);
    const long long o = r / taps;
    Wr[i] = c < C ? W[o * so + c * sc + map.src[t]] : static_cast<unsigned short>(0);
  }
}

template <int kBN, int kStages>
int launch_patch_cfg(const CUtensorMap& tmW, PatchParams& p, cudaStream_t s, bool dry) {
  const size_t smem = static_cast<size_t>(kStages) * kBN * 128 + 256 + 2ull * p.R_alloc * 128 + 16 * kBN + 1024;
  if (smem > 232448) return kUnimplemented;
  if (dry) return kOk;
  auto kernel = conv_patch_kernel<kBN, kStages>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] { attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448); });
  if (attr_err != cudaSuccess) return kCudaError;
  p.idesc = ptx::make_idesc(p.y_dtype == kBF16 ? 1 : 0, false, false, kPM, kBN);
  // two CTAs share an SM when their shared memory and TMEM columns allow: each one's fill, MMA and epilogue hide the
  // other's waits
  const bool two = 2 * (smem + 1024) <= 232448 && 2 * (2 * kBN) <= 512;
  const long long slots = static_cast<long long>(sm_budget()) * (two ? 2 : 1);
  const long long grid = p.tiles < slots ? p.tiles : slots;
  kernel<<<static_cast<unsigned>(grid), kPThreads, smem, s>>>(tmW, p);
  if (cudaGetLastError() != cudaSuccess) return kCudaError;
  note_tensor_launch(1);
  return kOk;
}

// The taps of a call: the full Kh x Kw grid (mirrored for the input-gradient form) or the caller's list.
struct TapList { int n; int r[kConvMaxTaps], c[kConvMaxTaps], src[kConvMaxTaps]; };
bool make_taps(const PatchConv& d, TapList& t) {
  if (d.n_taps > 0) {
    if (d.n_taps > kConvMaxTaps) return false;
    t.n = d.n_taps;
    for (int i = 0; i < t.n; ++i) {
      if (d.tap_r[i] < 0 || d.tap_c[i] < 0 || d.tap_src[i] < 0) return false;
      t.r[i] = d.tap_r[i]; t.c[i] = d.tap_c[i]; t.src[i] = d.tap_src[i];
    }
    return true;
  }
  if (d.Kh < 1 || d.Kw < 1 || d.Kh * d.Kw > kConvMaxTaps || d.dh < 1 || d.dw < 1) return false;
  t.n = d.Kh * d.Kw;
  for (int kh = 0; kh < d.Kh; ++kh)
    for (int kw = 0; kw < d.Kw; ++kw) {
      const int i = kh * d.Kw + kw;
      t.r[i] = kh * d.dh; t.c[i] = kw * d.dw;
      t.src[i] = d.flip_taps ? t.n - 1 - i : i;
    }
  return true;
}

// Fills the geometry part of the parameters; false when the shape is outside what the kernel takes.
bool patch_geometry(const PatchConv& d, PatchParams& p, TapList& taps) {
  if (!(d.dtype == kBF16 || d.dtype == kF16)) return false;
  if (d.ph < 0 || d.pw < 0 || !make_taps(d, taps)) return false;
  if (d.imgs < 1 || d.Cin < 1 || d.Cout < 1 || d.H < 1 || d.W < 1) return false;
  int max_tr = 0, max_tc = 0;
  for (int i = 0; i < taps.n; ++i) { max_tr = std::max(max_tr, taps.r[i]); max_tc = std::max(max_tc, taps.c[i]); }
  p.Cin = d.Cin; p.H = d.H; p.W = d.W; p.ph = d.ph; p.pw = d.pw;
  p.Wp = d.Wp > 0 ? d.Wp : d.W + 2 * d.pw;
  p.Hp = d.H + d.ph;                       // rows from here on hold no pixels (they read as zero)
  p.Ho = d.out_H > 0 ? d.out_H : d.H + 2 * d.ph - max_tr;
  p.Wo = d.out_W > 0 ? d.out_W : p.Wp - max_tc;
  if (p.Ho < 1 || p.Wo < 1) return false;
  // a row of the padded plane must hold the pixels and everything a valid output reads
  if (p.Wp < d.W + d.pw || p.Wp < p.Wo + max_tc) return false;
  const long long upos = static_cast<long long>(p.Ho) * p.Wp;           // padded output positions per image
  const long long max_shift = static_cast<long long>(max_tr) * p.Wp + max_tc;
  if (upos > (1 << 28) || max_shift > 1400) return false;
  p.R = kPM + static_cast<int>(max_shift);
  p.R_alloc = (p.R + 7) / 8 * 8 + 1;          // == 1 (mod 8): the four channel groups a warp stores to hit different banks
  p.tiles_per_img = static_cast<int>((upos + kPM - 1) / kPM);
  p.cblocks = (d.Cin + 63) / 64;
  p.Cp = p.cblocks * 64;
  p.taps = taps.n;
  for (int i = 0; i < taps.n; ++i) p.shift[i] = taps.r[i] * p.Wp + taps.c[i];
  // output addressing: dense planes unless the caller spreads the positions out
  p.out_row_pitch = d.out_row_pitch > 0 ? d.out_row_pitch : p.Wo;
  p.out_plane = d.out_plane > 0 ? static_cast<int>(d.out_plane) : p.Ho * p.Wo;
  p.osh = d.osh > 0 ? d.osh : 1; p.osw = d.osw > 0 ? d.osw : 1; p.out_off = d.out_off;
  if (d.out_plane > 0x7fffffffll) return false;
  // channel offsets stay inside 32-bit arithmetic in the fill
  if (d.img_pitch > 0x7fffffffll || d.plane_pitch * d.Cin > 0x7fffffffll) return false;
  p.X = static_cast<const unsigned short*>(d.X);
  p.img_pitch = d.img_pitch; p.plane_pitch = d.plane_pitch; p.row_pitch = d.row_pitch;
  int v = 8;
  const uintptr_t xa = reinterpret_cast<uintptr_t>(d.X);
  while (v > 1 && (d.W % v || d.row_pitch % v || d.plane_pitch % v || d.img_pitch % v || xa % (2 * v))) v >>= 1;
  p.V = v;
  return tc::driver_has_tensor_maps();
}

// Output channels per tile: the widest tile that still gives every SM a tile (a wide tile copies each patch for more
// channels at once, but a 14 x 14 or 7 x 7 layer has too few position tiles to fill the GPU with wide ones).
int patch_tile_n(int Cout, long long position_tiles) {
  int bn = Cout <= 64 ? 64 : (Cout <= 128 ? 128 : 256);
  while (bn > 64 && position_tiles * ((Cout + bn - 1) / bn) < sm_budget()) bn >>= 1;
  return bn;
}

template <typename F>
int for_patch_cfg(int bn, const PatchParams& p, F&& f) {
  // deepest weight ring that fits beside the two patches
  const size_t patches = 2ull * p.R_alloc * 128 + 256 + 1024 + 16ull * bn;
  auto fits = [&](int stages) { return patches + static_cast<size_t>(stages) * bn * 128 <= 232448; };
  // a shallower ring that lets two CTAs share the SM comes first
  auto fits_twice = [&](int stages) { return 2 * (patches + static_cast<size_t>(stages) * bn * 128 + 1024) <= 232448; };
  if (bn == 64)  { if (fits_twice(6)) return f(std::integral_constant<int, 64>{}, std::integral_constant<int, 6>{});
                   if (fits_twice(4)) return f(std::integral_constant<int, 64>{}, std::integral_constant<int, 4>{});
                   if (fits(8)) return f(std::integral_constant<int, 64>{}, std::integral_constant<int, 8>{});
                   if (fits(4)) return f(std::integral_constant<int, 64>{}, std::integral_constant<int, 4>{}); }
  if (bn == 128) { if (fits_twice(3)) return f(std::integral_constant<int, 128>{}, std::integral_constant<int, 3>{});
                   if (fits(6)) return f(std::integral_constant<int, 128>{}, std::integral_constant<int, 6>{});
                   if (fits(3)) return f(std::integral_constant<int, 128>{}, std::integral_constant<int, 3>{}); }
  if (bn == 256) { if (fits(4)) return f(std::integral_constant<int, 256>{}, std::integral_constant<int, 4>{});
                   if (fits(2)) return f(std::integral_constant<int, 256>{}, std::integral_constant<int, 2>{}); }
  return static_cast<int>(kUnimplemented);
}

}  // namespace

size_t conv_patch_weight_bytes(const PatchConv& d) {
  const int taps = d.n_taps > 0 ? d.n_taps : d.Kh * d.Kw;
  return static_cast<size_t>(d.Cout) * taps * ((d.Cin + 63) / 64 * 64) * 2;
}

bool conv_patch_supported(const PatchConv& d) {
  PatchParams p{};
  TapList taps{};
  if (!patch_geometry(d, p, taps)) return false;
  const int bn = patch_tile_n(d.Cout, static_cast<long long>(d.imgs) * p.tiles_per_img);
  CUtensorMap dummy{};
  return for_patch_cfg(bn, p, [&](auto bn_c, auto st_c) {
           return launch_patch_cfg<decltype(bn_c)::value, decltype(st_c)::value>(dummy, p, nullptr, true);
         }) == kOk;
}

int conv_patch_launch(const PatchConv& d, cudaStream_t s) {
  PatchParams p{};
  TapList taps{};
  if (!patch_geometry(d, p, taps)) return kUnimplemented;
  if (!d.Wr || !d.W_ || !d.Y) return kBadArgs;
  const int bn = patch_tile_n(d.Cout, static_cast<long long>(d.imgs) * p.tiles_per_img);
  p.n_tiles = (d.Cout + bn - 1) / bn;
  p.tiles = static_cast<long long>(d.imgs) * p.tiles_per_img * p.n_tiles;
  p.Cout = d.Cout;
  p.Y = d.Y; p.Z = d.Z; p.bias = d.bias;
  p.out_img_pitch = d.out_img_pitch;
  p.y_dtype = d.dtype; p.z_dtype = d.Z ? d.z_dtype : d.dtype; p.act = d.act; p.leaky = d.leaky;
  p.status = device_status_ptr();
  if (!p.status) return kCudaError;
  // weight -> Wr[Cout][tap][Cp]
  TapMap map{};
  for (int i = 0; i < taps.n; ++i) map.src[i] = taps.src[i];
  const long long ldr = static_cast<long long>(p.taps) * p.Cp;
  {
    const long long total = static_cast<long long>(d.Cout) * ldr;
    long long blocks = (total + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    relayout_weight_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const unsigned short*>(d.W_), static_cast<unsigned short*>(d.Wr), d.Cout, d.Cin, p.Cp, p.taps, d.w_row_stride,
        d.w_chan_stride, map);
    if (cudaGetLastError() != cudaSuccess) return kCudaError;
    note_tensor_launch(1);
  }
  CUtensorMap tmW;
  if (!tc::make_operand_map(&tmW, d.dtype, d.Wr, ldr, d.Cout, ldr, 1, 0, 64, bn, false)) return kCudaError;
  return for_patch_cfg(bn, p, [&](auto bn_c, auto st_c) {
    return launch_patch_cfg<decltype(bn_c)::value, decltype(st_c)::value>(tmW, p, s, false);
  });
}

}  // namespace ge2b
