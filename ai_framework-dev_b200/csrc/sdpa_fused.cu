// Fused scaled-dot-product attention forward for sm_100a:  O = softmax(scale * Q.K^T + mask) . V  per (batch, head),
// with the scores never leaving the SM.
//
// The reference computes this per (b, h) slice as transpose(K) -> GEMM -> scale kernel -> mask kernel -> softmax ->
// GEMM, with S and P materialised as fp32 [B,H,M,N] tensors (backends/cuda/ops/sdpa/launcher.cu:129-270; scale default
// 1/sqrt(D): :162; causal: n > m masked, :38-48; additive fp32 mask or 0/1 integer mask [B,1,M,N]: :56-95).  Here one CTA
// owns 256 query rows of one slice as TWO tiles of 128 rows and walks the keys in blocks of 128:
//   warp 0       TMA producer: both Q tiles once, then K_j (two-deep ring) and V_j (128-byte-swizzled tiles)
//   warp 1       MMA issuer:   per tile t: S_t = Q_t.K_j^T into TMEM (kind::f16, 128 x 128 x 16), O_t += P_t.V_j
//   warps 2..5   softmax of tile 0, warps 6..9 softmax of tile 1: one query row per thread, two passes over the row of
//                S_t in TMEM in chunks of 32 columns (tcgen05.ld): running max, then P_t = exp2(...) written as bf16
//                into shared memory in the swizzled operand layout; O_t rescaled in TMEM by exp2(m_old - m_new)
//                (tcgen05.ld / tcgen05.st) when the maximum moved; at the end O_t / sum -> global memory
// The two tiles take turns on the tensor pipe: while the softmax warps of one tile work, the MMAs of the other run,
// and eight softmax warps give every scheduler two warps to switch between.  The row loops are kept as loops over
// 32-column chunks: fully unrolled over 128 columns the code outgrows the instruction cache, which with so few warps
// per scheduler costs more than anything else in the kernel (measured: 2.9 ms against 0.4 ms at B.H = 128, L = 2048).
// Every mbarrier wait is bounded (sm100_ptx.cuh); on expiry the CTA records kErrWaitTimeout in the device status
// word, frees its TMEM and returns.  No TMA load uses cluster multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <mutex>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"
#include "gemm_tc_kernel.cuh"
#include "sm100_ptx.cuh"

using namespace ge2b;

namespace {

constexpr int kBlockQ = 128;       // query rows per tile (one TMEM lane each)
constexpr int kTiles = 2;          // tiles per CTA
constexpr int kBlockKV = 128;      // keys per step
constexpr int kSdpaThreads = 320;  // warp 0 TMA, warp 1 MMA, warps 2..5 / 6..9 softmax of tile 0 / 1
constexpr int kSoftmaxWarps = 4;   // per tile

struct SdpaParams {
  int B, H, M, N;                  // batch, heads, queries, keys
  int causal;
  float scale_log2;                // scale * log2(e): p = exp2(s * scale_log2 - m)
  const void* mask; int mask_kind; // 0 none, 1 fp32 additive, 2 int8 (non-zero = masked), 3 int32; [B,1,M,N]
  void* O; int o_dtype;            // [B,H,M,D]
  float* lse;                      // optional [B,H,M]: log-sum-exp of the scaled, masked scores (natural log)
  int* status;
};

template <int kD>
struct SdpaCfg {
  static constexpr int kKB = kD / 64;                    // 64-element (128-byte) blocks along the head dimension
  static constexpr int kQBytes = kBlockQ * kD * 2;       // per tile: kKB tiles of [128 rows x 128 B]
  static constexpr int kKBytes = kBlockKV * kD * 2;      // kKB tiles of [128 keys x 128 B]   (d contiguous)
  static constexpr int kVBytes = kBlockKV * kD * 2;      // 2 key halves x kKB boxes of [64 keys x 128 B] (d contiguous)
  static constexpr int kPBytes = kBlockQ * kBlockKV * 2; // per tile: 2 tiles of [128 rows x 128 B]  (keys contiguous)
  static constexpr int kSmem = kTiles * kQBytes + 2 * kKBytes + kVBytes + kTiles * kPBytes + 256 + 1024;
  static constexpr int kTmemCols = 512;                  // S_t: columns [128 t, 128 t + 128), O_t: [256 + 128 t, ... + kD)
  static_assert(kSmem <= 232448, "attention tiles exceed the shared memory of one SM");
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// One 32-column chunk of a row of scores, scaled (log2 units) and masked: v[i] for keys key0 .. key0 + 31.
__device__ __forceinline__ void masked_scores(const SdpaParams& p, const uint32_t (&r)[32], float (&v)[32], int key0, int row,
                                              bool row_ok, long long mask_row) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int key = key0 + i;
    float x = __uint_as_float(r[i]) * p.scale_log2;
    bool dead = key >= p.N || (p.causal && key > row);
    if (p.mask_kind != 0 && !dead && row_ok) {
      if (p.mask_kind == 1)      x += static_cast<const float*>(p.mask)[mask_row + key] * 1.4426950408889634f;
      else if (p.mask_kind == 2) dead = static_cast<const signed char*>(p.mask)[mask_row + key] != 0;
      else                       dead = static_cast<const int*>(p.mask)[mask_row + key] != 0;
    }
    v[i] = dead ? -CUDART_INF_F : x;
  }
}

template <int kD>
__global__ void __launch_bounds__(kSdpaThreads, 1)
sdpa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ SdpaParams p) {
  using Cfg = SdpaCfg<kD>;
  constexpr int kKB = Cfg::kKB;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t base = raw_addr + pad;
  const uint32_t q_smem = base;                                   // 2 tiles
  const uint32_t k_smem = q_smem + kTiles * Cfg::kQBytes;         // 2 stages
  const uint32_t v_smem = k_smem + 2 * Cfg::kKBytes;              // 1 stage
  const uint32_t p_smem = v_smem + Cfg::kVBytes;                  // 2 tiles
  constexpr int kPOff = kTiles * Cfg::kQBytes + 2 * Cfg::kKBytes + Cfg::kVBytes;
  uint8_t* p_ptr = smem + kPOff;
  const uint32_t bar0 = p_smem + kTiles * Cfg::kPBytes;
  uint8_t* bar_ptr = p_ptr + kTiles * Cfg::kPBytes;
  // barriers (8 bytes each)
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  const uint32_t v_full = bar0 + 8u * 5, v_empty = bar0 + 8u * 6;
  auto s_full = [&](int t) { return bar0 + 8u * (7 + t); };
  auto p_full = [&](int t) { return bar0 + 8u * (9 + t); };
  auto o_done = [&](int t) { return bar0 + 8u * (11 + t); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * 13 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blocks = (p.M + kTiles * kBlockQ - 1) / (kTiles * kBlockQ);
  const int slice = blockIdx.x / q_blocks;                        // b * H + h
  const int qb = blockIdx.x - slice * q_blocks;
  const int q0 = qb * kTiles * kBlockQ;
  // key blocks per tile: under a causal mask a tile needs no keys beyond its own last row, so tile 0 stops one block
  // before tile 1; n_kv is the CTA's count (tile 1 uses every block that is loaded)
  const int n_all = (p.N + kBlockKV - 1) / kBlockKV;
  auto tile_blocks = [&](int t) {
    return p.causal ? min(n_all, (min(q0 + (t + 1) * kBlockQ, max(p.M, q0 + 1)) + kBlockKV - 1) / kBlockKV) : n_all;
  };
  const int n_kv0 = tile_blocks(0);
  const int n_kv = max(n_kv0, tile_blocks(1));

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { ptx::mbar_init(k_full(s), 1); ptx::mbar_init(k_empty(s), 1); }
    ptx::mbar_init(v_full, 1); ptx::mbar_init(v_empty, 1);
    for (int t = 0; t < kTiles; ++t) {
      ptx::mbar_init(s_full(t), 1); ptx::mbar_init(p_full(t), kSoftmaxWarps); ptx::mbar_init(o_done(t), 1);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmQ); ptx::prefetch_tensormap(&tmK); ptx::prefetch_tensormap(&tmV);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(q_full, kTiles * Cfg::kQBytes);
#pragma unroll
      for (int t = 0; t < kTiles; ++t)
#pragma unroll
        for (int kb = 0; kb < kKB; ++kb)
          ptx::tma_load_3d(q_smem + t * Cfg::kQBytes + kb * (kBlockQ * 128), &tmQ, q_full, kb * 64, q0 + t * kBlockQ, slice);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!ptx::mbar_wait(k_empty(s), ((j >> 1) & 1) ^ 1u, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(k_full(s), Cfg::kKBytes);
#pragma unroll
        for (int kb = 0; kb < kKB; ++kb)
          ptx::tma_load_3d(k_smem + s * Cfg::kKBytes + kb * (kBlockKV * 128), &tmK, k_full(s), kb * 64, j * kBlockKV, slice);
        if (!ptx::mbar_wait(v_empty, (j & 1) ^ 1u, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(v_full, Cfg::kVBytes);
        // V block: two halves of 64 keys (the reduction blocks of P.V), each kKB boxes of {64 d, 64 keys}
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int kb = 0; kb < kKB; ++kb)
            ptx::tma_load_3d(v_smem + h * (64 * kD * 2) + kb * (64 * 128), &tmV, v_full, kb * 64, j * kBlockKV + h * 64, slice);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const uint32_t idesc_s = ptx::make_idesc(1, false, false, kBlockQ, kBlockKV);   // bf16, Q and K reduction-contiguous
      const uint32_t idesc_o = ptx::make_idesc(1, false, true, kBlockQ, kD);          // P reduction-contiguous, V d-contiguous
      bool ok = ptx::mbar_wait(q_full, 0u, abort_flag);
      auto issue_s = [&](int t, int j) {                        // S_t = Q_t . K_j^T
        const int s = j & 1;
        if (!ptx::mbar_wait(k_full(s), (j >> 1) & 1, abort_flag)) { ok = false; return; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + t * 128;
#pragma unroll
        for (int kb = 0; kb < kKB; ++kb) {
          const uint64_t a0 = ptx::make_smem_desc_sw128(q_smem + t * Cfg::kQBytes + kb * (kBlockQ * 128), 0u, 1024u);
          const uint64_t b0 = ptx::make_smem_desc_sw128(k_smem + s * Cfg::kKBytes + kb * (kBlockKV * 128), 0u, 1024u);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ptx::umma<false>(d_tmem, a0 + ks * 2, b0 + ks * 2, idesc_s, (kb | ks) ? 1u : 0u);
        }
        if (t == kTiles - 1) ptx::umma_commit(k_empty(s));      // both tiles have read this K block
        ptx::umma_commit(s_full(t));
      };
      auto issue_pv = [&](int t, int j) {                       // O_t += P_t . V_j
        if (!ptx::mbar_wait(p_full(t), j & 1, abort_flag)) { ok = false; return; }   // P_t written, O_t rescaled, S_t read
        if (!ptx::mbar_wait(v_full, j & 1, abort_flag)) { ok = false; return; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + 256 + t * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint64_t a0 = ptx::make_smem_desc_sw128(p_smem + t * Cfg::kPBytes + h * (kBlockQ * 128), 0u, 1024u);
          const uint64_t b0 = ptx::make_smem_desc_sw128(v_smem + h * (64 * kD * 2), 64u * 128u, 1024u);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ptx::umma<false>(d_tmem, a0 + ks * 2, b0 + ks * ((16 * 128) >> 4), idesc_o, (j > 0 || (h | ks)) ? 1u : 0u);
        }
        if (t == kTiles - 1) ptx::umma_commit(v_empty);         // both tiles have read this V block
        ptx::umma_commit(o_done(t));
      };
      if (ok && n_kv > 0) { issue_s(0, 0); if (ok) issue_s(1, 0); }
      for (int j = 0; ok && j < n_kv; ++j) {
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
          const int mine = t == 0 ? n_kv0 : n_kv;               // tile 1 walks every block: it frees the K / V slots
          if (!ok || j >= mine) continue;
          issue_pv(t, j);
          if (ok && j + 1 < mine) issue_s(t, j + 1);            // the tile's next scores while its softmax warps wait
        }
      }
    }
    __syncwarp();
  } else {
    // ===================== softmax: one query row per thread =====================
    const int t = (warp - 2) >> 2;                            // tile of this warp
    const int q = warp & 3;                                   // TMEM lane quarter this warp may access
    const int r_in = q * 32 + lane;
    const int row = q0 + t * kBlockQ + r_in;
    const bool row_ok = row < p.M;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_tmem = tmem_base + t * 128 + lane_sel, o_tmem = tmem_base + 256 + t * 128 + lane_sel;
    uint8_t* my_p = p_ptr + t * Cfg::kPBytes + r_in * 128;
    const int swz = r_in & 7;
    float m_run = -CUDART_INF_F, l_run = 0.f;
    const long long mask_row = p.mask ? (static_cast<long long>(slice / p.H) * p.M + row) * p.N : 0;
    bool ok = true;
    const int my_kv = t == 0 ? n_kv0 : n_kv;
#pragma unroll 1
    for (int j = 0; ok && j < my_kv; ++j) {
      // the TMEM accesses below are warp-collective: the warp stays or leaves together
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(s_full(t), j & 1, abort_flag))) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const int key0 = j * kBlockKV;
      // Three forms of the per-element work, chosen per key block and warp (warp-uniform):
      //   0  nothing is masked: the row maximum is the maximum of the raw scores times the (positive) scale;
      //   1  a column limit: keys beyond N in the last block and / or the diagonal of a causal mask, i.e. column i
      //      of the block is dead iff i > limit (per row);
      //   2  explicit masks or a non-positive scale: every element goes through masked_scores().
      const int warp_row0 = row - lane;
      const int form = (p.mask_kind != 0 || !(p.scale_log2 > 0.f)) ? 2
                       : (key0 + kBlockKV > p.N || (p.causal && key0 + kBlockKV - 1 > warp_row0)) ? 1 : 0;
      const int limit = min(p.N - 1 - key0, p.causal ? row - key0 : kBlockKV);      // last live column of this row
      float mx[4], ls[4], neg_m = 0.f;
      // raw (unscaled) maxima of one chunk, live columns only
      auto max_chunk = [&](int c, const uint32_t (&r)[32]) {
        if (form == 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            mx[i & 3] = fmaxf(mx[i & 3], (c * 32 + i <= limit) ? __uint_as_float(r[i]) : -CUDART_INF_F);
        }
      };
      // pass 1: row maximum of the scaled, masked scores of this block
      auto block_max = [&]() -> float {
        if (form != 2) {
          mx[0] = mx[1] = mx[2] = mx[3] = -CUDART_INF_F;
          uint32_t ra[32], rb[32];                                      // two 32-column TMEM loads in flight at a time
          ptx::tmem_ld_32x32(s_tmem, ra);
          ptx::tmem_ld_32x32(s_tmem + 32, rb);
          ptx::tmem_wait_ld();
          max_chunk(0, ra); max_chunk(1, rb);
          ptx::tmem_ld_32x32(s_tmem + 64, ra);
          ptx::tmem_ld_32x32(s_tmem + 96, rb);
          ptx::tmem_wait_ld();
          max_chunk(2, ra); max_chunk(3, rb);
          return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;     // (-inf stays -inf)
        }
        float m = -CUDART_INF_F;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          float v[32];
          ptx::tmem_ld_32x32(s_tmem + c * 32, r);
          ptx::tmem_wait_ld();
          masked_scores(p, r, v, key0 + c * 32, row, row_ok, mask_row);
#pragma unroll
          for (int i = 0; i < 32; ++i) m = fmaxf(m, v[i]);
        }
        return m;
      };
      // rows of O times alpha (warp-collective TMEM traffic: every lane takes part, with its own alpha)
      auto rescale_o = [&](float alpha) {
#pragma unroll 1
        for (int c = 0; c < kD / 32; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(o_tmem + c * 32, r);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(o_tmem + c * 32, r);
        }
        tmem_wait_st();
      };
      // one chunk: P = exp2(v - m) as bf16 into the operand layout (2 tiles of 64 keys, [128 rows x 128 B], 16-byte
      // chunk index XOR (row & 7)) and the row sum (fp32 values, four independent partial sums)
      auto exp_chunk = [&](int c, const uint32_t (&r)[32]) {
        uint32_t pk[16];
        if (form == 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float e0 = ex2(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, neg_m));
            const float e1 = ex2(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, neg_m));
            ls[(2 * i) & 3] += e0; ls[(2 * i + 1) & 3] += e1;
            const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
            pk[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
        } else if (form == 1) {
          const int lim_c = limit - c * 32;                             // last live column within this chunk
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float e0 = ex2(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, neg_m));
            float e1 = ex2(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, neg_m));
            e0 = (2 * i <= lim_c) ? e0 : 0.f;
            e1 = (2 * i + 1 <= lim_c) ? e1 : 0.f;
            ls[(2 * i) & 3] += e0; ls[(2 * i + 1) & 3] += e1;
            const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
            pk[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
        } else {
          float v[32];
          masked_scores(p, r, v, key0 + c * 32, row, row_ok, mask_row);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float e0 = ex2(v[2 * i] + neg_m), e1 = ex2(v[2 * i + 1] + neg_m);
            ls[(2 * i) & 3] += e0; ls[(2 * i + 1) & 3] += e1;
            const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
            pk[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        uint8_t* dst = my_p + (c >> 1) * (kBlockQ * 128);               // chunk c: keys 32 c .. 32 c + 31 of the block
#pragma unroll
        for (int k = 0; k < 4; ++k)
          *reinterpret_cast<uint4*>(dst + ((((c & 1) * 4 + k) ^ swz) * 16)) =
              make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
      };
      // pass 2: the whole block with reference -neg_m; the TMEM load of chunk c + 1 is in flight while chunk c is
      // turned into probabilities.  kTrack: also collect the block's raw maxima on the way (forms 0 and 1).
      auto exp_block = [&](bool track) {
        ls[0] = ls[1] = ls[2] = ls[3] = 0.f;
        if (track) mx[0] = mx[1] = mx[2] = mx[3] = -CUDART_INF_F;
        uint32_t ra[32], rb[32];
        ptx::tmem_ld_32x32(s_tmem, ra);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32(s_tmem + 32, rb);
        if (track) max_chunk(0, ra);
        exp_chunk(0, ra);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32(s_tmem + 64, ra);
        if (track) max_chunk(1, rb);
        exp_chunk(1, rb);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32(s_tmem + 96, rb);
        if (track) max_chunk(2, ra);
        exp_chunk(2, ra);
        ptx::tmem_wait_ld();
        if (track) max_chunk(3, rb);
        exp_chunk(3, rb);
      };

      // The reference point m of the exponentials only has to stay within range, not be the exact maximum: while the
      // row maximum has grown by less than 8 (a factor 256, harmless for fp32 sums and bf16 P) the old reference is
      // kept and O needs no rescaling; the final O / l is exact either way.
      float alpha = 1.f;
      const bool two_pass = form == 2 || __any_sync(0xffffffffu, m_run == -CUDART_INF_F);
      if (two_pass) {
        // first live block of a row, or explicit masks: maximum first, then the probabilities
        const float m_blk = block_max();
        const float m_cand = fmaxf(m_run, m_blk);
        const float m_new = (m_run != -CUDART_INF_F && m_cand - m_run <= 8.f) ? m_run : m_cand;
        const float m_use = (m_new == -CUDART_INF_F) ? 0.f : m_new;     // a fully masked row so far: keep everything 0
        alpha = (m_new == m_run) ? 1.f : ex2(m_run - m_use);            // exp2(-inf) = 0 on the first live block
        m_run = m_new;
        if (j > 0) {      // the tile's previous P.V must have finished: it read P's buffer and wrote O
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(o_done(t), (j - 1) & 1, abort_flag))) { ok = false; break; }
          ptx::tc_fence_after_sync();
          if (__any_sync(0xffffffffu, alpha != 1.f)) rescale_o(alpha);
        }
        neg_m = -m_use;
        exp_block(false);
      } else {
        // the usual block: ONE pass with the reference as it stands, collecting the block's maximum on the way; only
        // if that maximum turns out to exceed the reference by more than 8 (rare after the first blocks) is the
        // reference moved, O rescaled and the block redone
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(o_done(t), (j - 1) & 1, abort_flag))) { ok = false; break; }
        ptx::tc_fence_after_sync();
        neg_m = -m_run;
        exp_block(true);
        const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
        const bool grew = m_blk - m_run > 8.f;
        if (__any_sync(0xffffffffu, grew)) {
          const float m_new = grew ? m_blk : m_run;
          alpha = grew ? ex2(m_run - m_new) : 1.f;
          m_run = m_new;
          rescale_o(alpha);
          neg_m = -m_new;
          exp_block(false);
        }
      }
      const float l_blk = (ls[0] + ls[1]) + (ls[2] + ls[3]);
      l_run = l_run * alpha + l_blk;
      ptx::fence_proxy_async_smem();                                    // the MMA reads P through the async proxy
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(p_full(t));
    }
    // ---- O / l -> global memory ----
    if (ok && my_kv > 0) ok = __all_sync(0xffffffffu, ptx::mbar_wait(o_done(t), (my_kv - 1) & 1, abort_flag));
    if (ok) {
      ptx::tc_fence_after_sync();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const long long o_off = (static_cast<long long>(slice) * p.M + row) * kD;
#pragma unroll 1
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t r[32];
        if (my_kv > 0) { ptx::tmem_ld_32x32(o_tmem + c * 32, r); ptx::tmem_wait_ld(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_ok) {
          if (p.o_dtype == kF32) {
            float* dst = static_cast<float*>(p.O) + o_off + c * 32;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(r[4 * i]) * inv, __uint_as_float(r[4 * i + 1]) * inv,
                                                               __uint_as_float(r[4 * i + 2]) * inv, __uint_as_float(r[4 * i + 3]) * inv);
          } else {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float a = __uint_as_float(r[2 * i]) * inv, b = __uint_as_float(r[2 * i + 1]) * inv;
              if (p.o_dtype == kBF16) { const __nv_bfloat162 h = __floats2bfloat162_rn(a, b); w[i] = *reinterpret_cast<const uint32_t*>(&h); }
              else                    { const __half2 h = __floats2half2_rn(a, b);           w[i] = *reinterpret_cast<const uint32_t*>(&h); }
            }
            uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned short*>(p.O) + o_off + c * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          }
        }
      }
      if (p.lse != nullptr && row_ok)
        p.lse[static_cast<long long>(slice) * p.M + row] =
            l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -CUDART_INF_F;
    }
    ptx::tc_fence_before_sync();
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
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int kD>
int launch_sdpa(const ge2b_sdpa_params_t& a, const void* Q, const void* K, const void* V, const void* mask, void* O,
                float* lse, cudaStream_t s) {
  using Cfg = SdpaCfg<kD>;
  auto kernel = sdpa_fwd_kernel<kD>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] { attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem); });
  if (attr_err != cudaSuccess) return kCudaError;
  const long long slices = static_cast<long long>(a.B) * a.H;
  CUtensorMap tmQ, tmK, tmV;
  // 3-D maps {d, rows of the slice, slice}: a box never crosses into the next slice, rows beyond M / N read as zero
  if (!tc::make_operand_map(&tmQ, a.dtype, Q, kD, a.M, kD, slices, static_cast<long long>(a.M) * kD, 64, kBlockQ, false) ||
      !tc::make_operand_map(&tmK, a.dtype, K, kD, a.N, kD, slices, static_cast<long long>(a.N) * kD, 64, kBlockKV, false) ||
      !tc::make_operand_map(&tmV, a.dtype, V, kD, a.N, kD, slices, static_cast<long long>(a.N) * kD, 64, 64, false))
    return kCudaError;
  SdpaParams p{};
  p.B = a.B; p.H = a.H; p.M = a.M; p.N = a.N;
  p.causal = a.causal ? 1 : 0;
  const float scale = a.scale != 0.f ? a.scale : 1.f / sqrtf(static_cast<float>(kD));
  p.scale_log2 = scale * 1.4426950408889634f;
  p.mask = mask; p.mask_kind = mask ? a.mask_kind : 0;
  p.O = O; p.o_dtype = a.dtype; p.lse = lse;
  p.status = device_status_ptr();
  if (!p.status) return kCudaError;
  const int q_blocks = (a.M + kTiles * kBlockQ - 1) / (kTiles * kBlockQ);
  const long long grid = slices * q_blocks;
  if (grid > 0x7fffffffll) return kBadArgs;
  kernel<<<static_cast<unsigned>(grid), kSdpaThreads, Cfg::kSmem, s>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace

extern "C" int ge2b_sdpa_forward(const ge2b_sdpa_params_t* a, const void* Q, const void* K, const void* V, const void* mask,
                                 void* O, float* lse, void* stream) {
  if (!a || !Q || !K || !V || !O || a->B < 1 || a->H < 1 || a->M < 1 || a->N < 1) return kBadArgs;
  if (a->dtype != GE2_DT_BF16) return kUnimplemented;          // the tile layouts below are the 16-bit ones; f16 would need its own MMA format flag
  if (a->D != 64 && a->D != 128) return kUnimplemented;
  if (a->dropout_p != 0.f) return kUnimplemented;               // inference / deterministic training only
  if (mask && (a->mask_kind < 1 || a->mask_kind > 3)) return kBadArgs;
  auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (!aligned(Q) || !aligned(K) || !aligned(V) || !aligned(O)) return kBadArgs;
  if (!tc::driver_has_tensor_maps()) return kCudaError;
  NvtxRange range("sdpa.fwd");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return a->D == 128 ? launch_sdpa<128>(*a, Q, K, V, mask, O, lse, s) : launch_sdpa<64>(*a, Q, K, V, mask, O, lse, s);
}
