// Kernel template and per-configuration launchers of the tensor-core GEMM; included by gemm_tc.cu (dispatch and
// host helpers) and by the gemm_tc_inst_*.cu files, each of which instantiates one operand-order / dtype family so
// that the families compile in parallel.
#pragma once
// Tensor-core GEMM with fused epilogue for sm_100a:  D[b] = act(alpha * A[b].B[b] + beta * C[b] + bias).
//
// This is the B200 replacement for the reference's fp32 SIMT forward kernel
// (backends/cuda/ops/gemm/kernels/regemm_gemm_bias_act.cu:254-395) and for the two cublasSgemm
// calls of its backward (regemm_backward.cu:265-291).  One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer: 128-byte-swizzled operand tiles into a shared-memory ring
//   warp 1      MMA issuer:   tcgen05.mma (kind::f16 for bf16/f16, kind::tf32 for fp32) into TMEM;
//               also owns TMEM allocation
//   warps 2..9  epilogue:     tcgen05.ld of the finished accumulator, alpha/beta.C/bias/activation,
//               optional pre-activation stash, one store of D; two warps per TMEM lane quarter, each
//               taking one half of the tile's columns
// The accumulator is double-buffered in TMEM (2 x BLOCK_N columns) so the epilogue of tile i overlaps
// the main loop of tile i+1.  Operands may be stored with either the reduction index or the M/N index
// contiguous, which lets forward (X.W), dX (gZ.W^T) and dW (X^T.gZ) all read the caller's row-major
// tensors directly, and a third tensor-map dimension carries the batch of the strided-batched form.
// No TMA load uses cluster multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "epilogue_math.cuh"
#include "ge2_internal.hpp"
#include "sm100_ptx.cuh"

namespace ge2b {
namespace tc {


constexpr int kBlockM        = 128;   // UMMA M (one TMEM lane per output row)
constexpr int kNumThreads    = 320;   // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int kEpiWarps      = 8;     // two per TMEM lane quarter: each takes one half of the tile columns
constexpr int kGroupM        = 8;     // tile rasterisation: groups of (by default) 8 row-blocks sweep the columns
constexpr int kStoreStageWarp = 4096; // 32 rows x 32 columns x 4 bytes: one epilogue warp's transpose buffer

struct TcParams {
  int M, N, K, batch;
  int m_blocks, n_blocks, k_blocks;
  int group_m;              // row-blocks per rasterisation group
  int a_bcast, b_bcast;     // operand has batch stride 0: always read slice 0
  int kb_per_slice;         // > 0: the reduction runs over every batch slice in turn (k_blocks = slices * this);
                            // one output matrix, `batch` is 1 for the tile schedule
  int x3_kb;                // > 0: error-compensated fp32 (k_blocks = 3 * this): the reduction is walked three times,
                            // over (A big, B small), (A small, B big), (A big, B big); the small parts' tensor maps
                            // travel in the kernel's second-problem slot
  uint32_t idesc;
  EpilogueArgs epi;
  int d_vec, z_vec, c_vec, bias_vec;   // base, pitch and batch stride 16-byte aligned: D / Z leave through TMA stores,
                                       // C and bias are read with 16-byte loads
  int plain;                           // no C, no bias, no Z, no activation: the epilogue only scales and stores
  int store_dbl;                       // every stored tensor is 16-bit: the staging buffer is used as two halves
  int store_wide;                      // D is the only output and 16-bit: two 32-column fragments leave as one
                                       // 64-column (128-byte rows) bulk store; tmD then has a 64 x 32 box
  // Split-K (problems smaller than one wave): every tile is cut into `split` slices of the reduction so that the
  // launch occupies all SMs.  Items [0, main_tiles) are whole tiles (none today: main_tiles is 0 whenever split > 1);
  // item main_tiles + s * tail_tiles + r is slice s of tail tile r.  Every slice leaves its fp32 partial tile in
  // `ws`.  With few slices (fin_in_kernel) each epilogue warp then counts itself into flags[tile][warp slot], and the
  // warp that arrives last adds the slices' partials of its part of the tile, in slice order, and runs the epilogue;
  // with many slices splitk_finalize_kernel, launched right after, does that with the whole machine.  Either way the
  // result does not depend on arrival order and no CTA waits for another one.
  //
  // Narrow tail (common variant, CTA pairs with 256-column tiles): the tiles of a partly filled last wave are cut
  // into two 128-column halves instead, so that twice as many pairs finish the launch together and nothing is
  // exchanged.  Item main_tiles + i is half (i & 1) of tail tile i / 2; `split` is 2 and `idesc_half` describes the
  // 256 x 128 MMA.
  DbFinish db;              // bias-gradient finish carried by this launch (partial == null: none)
  int main_tiles, tail_tiles, split;
  uint32_t idesc_half;
  float* ws;
  int* flags;
  int fin_in_kernel;
  int* status;
};

// Second problem of a dual launch: one persistent grid walks the tiles of two independent GEMMs (the dense layer's
// dX = gZ.W^T and dW = X^T.gZ) as one list, so that only the last wave of the combined list is partly filled.
// The second problem may store its operands in other orders than the first; it has a plain epilogue.
struct DualParams {
  CUtensorMap tmA, tmB, tmD;
  TcParams p;
};

template <bool kValue> struct BoolC { static constexpr bool value = kValue; };

template <int kElemBytes, int kBlockN, int kStages, int kCG>
struct TcCfg {
  static constexpr int kBlockK     = 128 / kElemBytes;    // one 128-byte swizzle row of the reduction index
  static constexpr int kUmmaK      = 32 / kElemBytes;     // reduction depth of one tcgen05.mma
  static constexpr int kAStage     = kBlockM * 128;             // this CTA's 128 rows of A
  static constexpr int kBStage     = (kBlockN / kCG) * 128;     // this CTA's share of B
  static constexpr int kStageBytes = kAStage + kBStage;
  static constexpr int kTmemCols   = (kCG == 2) ? 512 : 2 * kBlockN;   // pairs take all columns so both CTAs get base 0
  static constexpr int kBarBytes   = 256;
  static constexpr int kStoreStage = kEpiWarps * kStoreStageWarp;       // per-warp transpose buffers of the epilogue
  static constexpr int kSmemBytes  = kStages * kStageBytes + kBarBytes + kStoreStage + 1024;   // +1024: alignment
  static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "TMEM allocation must be a power of two");
  static_assert(kSmemBytes <= 232448, "operand ring exceeds the shared memory of one SM");
  static_assert(8 * (2 * kStages + 4) + 16 <= kBarBytes, "barrier block too small");
};

// ---- row-fragment load: one thread owns `n` (<= 32) consecutive columns of one row of C ----
__device__ __forceinline__ void load_row_frag(const void* base, long long off, int dt, float (&v)[32], int n,
                                              bool vec) {
  if (dt == kF32) {
    const float* p = reinterpret_cast<const float*>(base) + off;
    if (vec && n == 32) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 f = reinterpret_cast<const float4*>(p)[j];
        v[4 * j] = f.x; v[4 * j + 1] = f.y; v[4 * j + 2] = f.z; v[4 * j + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (j < n) ? p[j] : 0.f;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < n) ? load_as_f32(base, off + j, dt) : 0.f;
  }
}

// Per-warp state of the epilogue's stores: the warp's 4 KB staging buffer and which half is next.
struct EpiStage {
  uint8_t* buf;
  int slot;
};

// Store of a 32-row x 32-column fragment held one row per lane: the rows are written to the warp's staging buffer
// in the TMA swizzle pattern (16-byte chunk index XOR (row >> 1) & 3 for 64-byte rows, XOR row & 7 for 128-byte rows,
// which is also what keeps these shared-memory stores free of bank conflicts) and one lane issues a tiled bulk store
// of the 32 x 32 box.  Rows >= M and columns >= N of the box are clipped by the tensor map.  With 16-bit tensors the
// buffer holds two fragments and a store only has to wait for the one issued before the previous one.
__device__ __forceinline__ void store_frag_tma(EpiStage& st, bool dbl, const CUtensorMap* tm, int dt, const float (&v)[32],
                                               int row0, int col0, int b, int lane) {
  const bool wide = (dt == kF32);
  uint8_t* buf = st.buf + ((dbl && st.slot) ? 2048 : 0);
  if (lane == 0) {
    if (dbl) ptx::bulk_wait_group_read<1>();
    else     ptx::bulk_wait_group_read<0>();
  }
  __syncwarp();
  if (wide) {
    const int swz = lane & 7;
    uint8_t* my_row = buf + lane * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<float4*>(my_row + ((c ^ swz) * 16)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  } else {
    const int swz = (lane >> 1) & 3;
    uint8_t* my_row = buf + lane * 64;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float lo = v[8 * c + 2 * t], hi = v[8 * c + 2 * t + 1];
        if (dt == kBF16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
          w[t] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(lo, hi);
          w[t] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      *reinterpret_cast<uint4*>(my_row + ((c ^ swz) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  ptx::fence_proxy_async_smem();        // the bulk store reads shared memory through the async proxy
  __syncwarp();
  if (lane == 0) {
    ptx::tma_store_3d(tm, ptx::smem_u32(buf), col0, row0, b);
    ptx::bulk_commit_group();
  }
  if (dbl) st.slot ^= 1;
}

// Store for outputs whose base or pitch is not 16-byte aligned (no TMA store possible): the fragment goes through the
// warp's staging buffer as fp32, element (r, j) at word r * 32 + (j ^ r) (conflict-free both ways), and leaves one row per instruction
// with consecutive lanes on consecutive columns, so that each store covers one contiguous run of a row instead of
// 32 different rows.  Waits for any bulk store that may still be reading the buffer first.
__device__ __forceinline__ void store_frag_rows(EpiStage& st, void* base, long long off0, long long ld, int dt,
                                                const float (&v)[32], int row0, int col0, int M, int N, int lane) {
  if (lane == 0) ptx::bulk_wait_group_read<0>();
  __syncwarp();
  float* buf = reinterpret_cast<float*>(st.buf);
#pragma unroll
  for (int j = 0; j < 32; ++j) buf[lane * 32 + (j ^ lane)] = v[j];
  __syncwarp();
  const bool col_ok = col0 + lane < N;
  const int rows = min(32, M - row0);
  for (int r = 0; r < rows; ++r) {
    const float x = buf[r * 32 + (lane ^ r)];
    if (col_ok) store_from_f32(base, off0 + static_cast<long long>(row0 + r) * ld + col0 + lane, dt, x);
  }
  __syncwarp();
}

// 16-bit, single output: fragments of two neighbouring 32-column chunks share one buffer of 128-byte rows
// (chunk index XOR row & 7) and leave together, halving the number of bulk stores, proxy fences and waits.
// `second` is the odd chunk of the pair, `flush` says that no further chunk follows (a ragged last pair: the
// columns the missing half would cover lie beyond N and are clipped by the tensor map).
__device__ __forceinline__ void store_frag_tma_wide(EpiStage& st, const CUtensorMap* tm, int dt, const float (&v)[32],
                                                    int row0, int col0, int b, int lane, bool second, bool flush) {
  if (!second) {
    if (lane == 0) ptx::bulk_wait_group_read<0>();
    __syncwarp();
  }
  const int swz = lane & 7;
  uint8_t* my_row = st.buf + lane * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float lo = v[8 * c + 2 * t], hi = v[8 * c + 2 * t + 1];
      if (dt == kBF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        w[t] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(lo, hi);
        w[t] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(my_row + (((second ? 4 + c : c) ^ swz) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  if (second || flush) {
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      ptx::tma_store_3d(tm, ptx::smem_u32(st.buf), second ? col0 - 32 : col0, row0, b);
      ptx::bulk_commit_group();
    }
  }
}

template <int ACT>
__device__ __forceinline__ void apply_act32(float (&v)[32], float leaky, bool fast) {
  if (fast) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = act_fwd<ACT, true>(v[j], leaky);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = act_fwd<ACT, false>(v[j], leaky);
  }
}

// Epilogue math for one 32-column fragment of one row (order of operations follows the reference's
// Epilogue::apply, backends/cuda/ops/_common/shim/traits.hpp:30-73): alpha, + beta*C, + bias, stash Z, act.
__device__ __forceinline__ void epilogue_frag(const TcParams& p, const CUtensorMap* tmD, const CUtensorMap* tmZ,
                                              float (&v)[32], int b, int row, int col0, int ncols, bool row_ok,
                                              EpiStage& stage, int lane, bool second, bool last) {
  const EpilogueArgs& e = p.epi;
  if (e.alpha != 1.f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= e.alpha;
  }
  if (p.plain) {
    // nothing but the scaled product to store (dX, dW, the attention GEMMs): skip the rest of the epilogue's tests
    if (p.store_wide)
      store_frag_tma_wide(stage, tmD, e.d_dtype, v, row - lane, col0, b, lane, second, last);
    else if (p.d_vec)
      store_frag_tma(stage, p.store_dbl != 0, tmD, e.d_dtype, v, row - lane, col0, b, lane);
    else
      store_frag_rows(stage, e.D, static_cast<long long>(b) * e.strideD, e.ldd, e.d_dtype, v, row - lane, col0, p.M, p.N,
                      lane);
    return;
  }
  if (e.C != nullptr && e.beta != 0.f && row_ok) {
    float c[32];
    load_row_frag(e.C, static_cast<long long>(b) * e.strideC + static_cast<long long>(row) * e.ldc + col0, e.d_dtype,
                  c, ncols, p.c_vec != 0);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaf(e.beta, c[j], v[j]);
  }
  if (e.bias != nullptr) {
    if (e.bias_kind == kBiasPerN) {
      if (p.bias_vec && ncols == 32) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(e.bias + col0) + j);
          v[4 * j] += f.x; v[4 * j + 1] += f.y; v[4 * j + 2] += f.z; v[4 * j + 3] += f.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) v[j] += __ldg(e.bias + col0 + j);
      }
    } else if (e.bias_kind == kBiasPerM) {
      const float bm = row_ok ? __ldg(e.bias + row) : 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += bm;
    } else if (e.bias_kind == kBiasScalar) {
      const float bs = __ldg(e.bias);
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += bs;
    }
  }
  if (e.Z != nullptr) {
    if (p.z_vec)
      store_frag_tma(stage, p.store_dbl != 0, tmZ, e.z_dtype, v, row - lane, col0, b, lane);
    else
      store_frag_rows(stage, e.Z, static_cast<long long>(b) * e.strideZ, e.ldz, e.z_dtype, v, row - lane, col0, p.M, p.N,
                      lane);
  }
  const bool fast = e.d_dtype != kF32;       // the result is rounded to 16 bits: exp-based tanh / sigmoid suffice
  switch (e.act) {
    case kActReLU:    apply_act32<kActReLU>(v, e.leaky, false); break;
    case kActLeaky:   apply_act32<kActLeaky>(v, e.leaky, false); break;
    case kActGELU:    apply_act32<kActGELU>(v, e.leaky, fast); break;
    case kActSigmoid: apply_act32<kActSigmoid>(v, e.leaky, fast); break;
    case kActTanh:    apply_act32<kActTanh>(v, e.leaky, fast); break;
    default: break;
  }
  if (p.store_wide)
    store_frag_tma_wide(stage, tmD, e.d_dtype, v, row - lane, col0, b, lane, second, last);
  else if (p.d_vec)
    store_frag_tma(stage, p.store_dbl != 0, tmD, e.d_dtype, v, row - lane, col0, b, lane);
  else
    store_frag_rows(stage, e.D, static_cast<long long>(b) * e.strideD, e.ldd, e.d_dtype, v, row - lane, col0, p.M, p.N,
                    lane);
}

// Persistent tile order: within a batch slice, groups of kGroupM row-blocks sweep all column-blocks,
// so CTAs that run together share operand tiles through L2.
__device__ __forceinline__ void decode_tile(const TcParams& p, long long tile, int& b, int& mb, int& nb) {
  const int per_batch = p.m_blocks * p.n_blocks;
  b = static_cast<int>(tile / per_batch);
  const int t = static_cast<int>(tile - static_cast<long long>(b) * per_batch);
  const int group_sz = p.group_m * p.n_blocks;
  const int g = t / group_sz;
  const int first_m = g * p.group_m;
  const int rows_in_group = min(p.group_m, p.m_blocks - first_m);
  const int r = t - g * group_sz;
  mb = first_m + r % rows_in_group;
  nb = r / rows_in_group;
}

// One unit of work of the persistent loop: a tile and the range of k-blocks to reduce over.
struct WorkItem {
  int b, mb, nb;
  int kb0, kb1;       // k-block range
  int slice, tail;    // slice of a split tile (0 when the tile is whole), index of the tail tile
  bool split;
  bool narrow;        // a 128-column half of a tail tile (narrow-tail form)
  int n_off;          // first column of the item inside its tile: 0, or 128 for the second half
};

__device__ __forceinline__ WorkItem decode_work(const TcParams& p, long long item) {
  WorkItem w;
  long long tile = item;
  w.slice = 0; w.tail = 0; w.split = false; w.narrow = false; w.n_off = 0;
  w.kb0 = 0; w.kb1 = p.k_blocks;
  if (item >= p.main_tiles) {
    const int t = static_cast<int>(item - p.main_tiles);
    w.slice = t / p.tail_tiles;
    w.tail = t - w.slice * p.tail_tiles;
    w.split = true;
    tile = p.main_tiles + w.tail;
    w.kb0 = static_cast<int>(static_cast<long long>(w.slice) * p.k_blocks / p.split);
    w.kb1 = static_cast<int>(static_cast<long long>(w.slice + 1) * p.k_blocks / p.split);
  }
  decode_tile(p, tile, w.b, w.mb, w.nb);
  return w;
}

template <bool kSplit, bool kNarrow>
__device__ __forceinline__ WorkItem get_work(const TcParams& p, long long item) {
  if constexpr (kSplit) {
    return decode_work(p, item);
  } else {
    WorkItem w;
    w.slice = 0; w.tail = 0; w.split = false; w.kb0 = 0; w.kb1 = p.k_blocks; w.narrow = false; w.n_off = 0;
    long long tile = item;
    if constexpr (kNarrow) {
      if (item >= p.main_tiles) {
        const long long i = item - p.main_tiles;
        tile = p.main_tiles + (i >> 1);
        w.narrow = true;
        w.n_off = static_cast<int>(i & 1) * 128;
      }
    }
    decode_tile(p, tile, w.b, w.mb, w.nb);
    return w;
  }
}

// kSplit = true compiles the variant for problems smaller than one wave, whose tiles are also cut along the
// reduction (see TcParams); the common variant carries none of that code.
// kCG = 1: one CTA per tile (128 x kBlockN).  kCG = 2: a pair of CTAs on neighbouring SMs shares one
// 256 x kBlockN tile: each CTA stages its own 128 rows of A and its own half of B, the MMAs are issued by the
// pair's first CTA and write 128 accumulator rows into each CTA's TMEM, and each CTA runs the epilogue of its
// own rows.  Halving B's shared-memory footprint per CTA buys a deeper operand ring.
// kDual: a second problem (d2, operand orders kAMN2 / kBMN2) follows the first in the item list; see DualParams.
template <int kElemBytes, bool kAMN, bool kBMN, int kBlockN, int kStages, int kCG, bool kSplit, bool kDual = false,
          bool kAMN2 = false, bool kBMN2 = false>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmD,
               const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ TcParams p,
               const __grid_constant__ DualParams d2) {
  static_assert(!(kDual && kSplit), "a dual launch has no split-K form");
  // tmBh: B with a box of half as many rows, for the narrow tail's reduction-contiguous B (otherwise a copy of tmB).
  // tmD / tmZ: the outputs as {columns, rows, batch} with a 32 x 32 box (valid when p.d_vec / p.z_vec).
  using Cfg = TcCfg<kElemBytes, kBlockN, kStages, kCG>;
  constexpr bool kTf32 = (kElemBytes == 4);
  constexpr bool kNarrow = (!kSplit && kCG == 2 && kBlockN == 256);   // see TcParams
  constexpr int kTileM = kBlockM * kCG;          // rows of one scheduled tile
  constexpr int kLocalN = kBlockN / kCG;         // B rows/columns staged by one CTA

  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle needs 1024-byte aligned tile bases.
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  // After the operand ring: the epilogue's staging buffers (1024-byte aligned, as the swizzled TMA stores need),
  // then the barrier block.
  uint8_t* store_stage = smem + kStages * Cfg::kStageBytes;
  uint8_t* bar_blk = store_stage + Cfg::kStoreStage;
  const uint32_t bar_base = smem_base + kStages * Cfg::kStageBytes + Cfg::kStoreStage;
  auto full_bar   = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar  = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar  = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bar_blk + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_blk + 8 * (2 * kStages + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCG == 2) ? ptx::cluster_ctarank() : 0u;
  const bool leader = (cta_rank == 0);
  const int unit = (kCG == 2) ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);   // tile walker id
  const int n_units = (kCG == 2) ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), kEpiWarps * kCG); }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    if constexpr (kCG == 2) {
      ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), Cfg::kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), Cfg::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (kCG == 2) ptx::cluster_sync_all();   // the peer's barriers exist before anything signals them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  // Everything above touched only this CTA's shared memory and TMEM; from here on global memory is read and written,
  // so a launch that was allowed to start early waits here for the kernel before it (see sm100_ptx.cuh).
  ptx::griddep_launch();
  ptx::griddep_wait();

  const long long items1 = static_cast<long long>(p.main_tiles) + static_cast<long long>(p.tail_tiles) * p.split;
  const long long total_items = items1 + (kDual ? static_cast<long long>(d2.p.main_tiles) : 0ll);

  if (warp == 0) {
    // ===================== TMA producer (every CTA stages its own share) =====================
    if (lane == 0) {
      const uint32_t full_leader0 = (kCG == 2) ? ptx::map_to_cta(full_bar(0), 0u) : full_bar(0);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      // One item (tile or slice of a tile) of problem `pp`, whose operands are stored in the orders AMN / BMN.
      auto produce = [&](auto amn_c, auto bmn_c, const TcParams& pp, const CUtensorMap* mA, const CUtensorMap* mB,
                         const CUtensorMap* mBh, const WorkItem& w) {   // mA / mB by value: the x3 form re-points them
        constexpr bool AMN = decltype(amn_c)::value, BMN = decltype(bmn_c)::value;
        const int b = w.b;
        const int m0 = w.mb * kTileM + static_cast<int>(cta_rank) * kBlockM;
        const bool narrow = kNarrow && w.narrow;
        const int local_n = narrow ? kLocalN / 2 : kLocalN;          // B rows / columns this CTA stages
        const int n0 = w.nb * kBlockN + w.n_off + static_cast<int>(cta_rank) * local_n;
        const uint32_t stage_tx = (Cfg::kAStage + (narrow ? Cfg::kBStage / 2 : Cfg::kBStage)) * kCG;
        int ba = pp.a_bcast ? 0 : b, bb = pp.b_bcast ? 0 : b;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          // The pair's first CTA owns the "full" barrier and announces the bytes of both CTAs.
          if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), stage_tx);
          const uint32_t fb = full_leader0 + 8u * stage;
          const uint32_t a_dst = smem_base + stage * Cfg::kStageBytes;
          const uint32_t b_dst = a_dst + Cfg::kAStage;
          int k0 = kb * Cfg::kBlockK;
          if (pp.kb_per_slice > 0) {                   // reduction over the batch: slice first, then k inside it
            const int sl = kb / pp.kb_per_slice;
            k0 = (kb - sl * pp.kb_per_slice) * Cfg::kBlockK;
            ba = pp.a_bcast ? 0 : sl; bb = pp.b_bcast ? 0 : sl;
          }
          if constexpr (!kDual) {
            if (pp.x3_kb > 0) {                        // three passes over the reduction with the split operands
              // Order: the two small cross products first, big.big last.  The tensor core adds into its fp32
              // accumulator with truncation, an error of up to one unit in the last place of the ACCUMULATOR per
              // MMA; while only cross terms have been added the accumulator is 2^-11 of its final size and those
              // errors vanish, so only the K/8 additions of the last pass count (measured: big.big first gave
              // 1.5e-5 relative at K = 512, three times what this order gives).
              const int pass = kb / pp.x3_kb;
              k0 = (kb - pass * pp.x3_kb) * Cfg::kBlockK;
              mA = pass == 1 ? &d2.tmA : &tmA;
              mB = pass == 0 ? &d2.tmB : &tmB;
            }
          }
          auto load = [&](uint32_t dst, const void* tm, int c0, int c1, int c2) {
            if constexpr (kCG == 2) ptx::tma_load_3d_pair(dst, tm, fb, c0, c1, c2);
            else                    ptx::tma_load_3d(dst, tm, fb, c0, c1, c2);
          };
          if constexpr (!AMN) {
            load(a_dst, mA, k0, m0, ba);                                        // box {kBlockK, 128}
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / Cfg::kBlockK; ++j)                    // boxes {kBlockK(m), kBlockK(k)}
              load(a_dst + j * (Cfg::kBlockK * 128), mA, m0 + j * Cfg::kBlockK, k0, ba);
          }
          if constexpr (!BMN) {
            if (narrow) load(b_dst, mBh, k0, n0, bb);                           // box {kBlockK, kLocalN / 2}
            else        load(b_dst, mB, k0, n0, bb);                            // box {kBlockK, kLocalN}
          } else {
#pragma unroll
            for (int j = 0; j < kLocalN / Cfg::kBlockK; ++j)
              if (j * Cfg::kBlockK < local_n)
                load(b_dst + j * (Cfg::kBlockK * 128), mB, n0 + j * Cfg::kBlockK, k0, bb);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      };
      for (long long item = unit; ok && item < total_items; item += n_units) {
        if constexpr (kDual) {
          if (item >= items1) {
            produce(BoolC<kAMN2>{}, BoolC<kBMN2>{}, d2.p, &d2.tmA, &d2.tmB, &d2.tmB,
                    get_work<false, false>(d2.p, item - items1));
            continue;
          }
        }
        produce(BoolC<kAMN>{}, BoolC<kBMN>{}, p, &tmA, &tmB, &tmBh, get_work<kSplit, kNarrow>(p, item));
      }
    } else if (p.db.partial != nullptr) {
      // The other 31 lanes of the producer warp have nothing to do: they finish the bias gradient the prologue kernel
      // left as per-row-block column sums (out[c] = sum over row blocks in ascending order: the same bits every run),
      // while lane 0 feeds the ring and the tensor pipe works.
      const int stride = static_cast<int>(gridDim.x) * 31;
      for (int c = static_cast<int>(blockIdx.x) * 31 + lane - 1; c < p.db.n; c += stride) {
        const float* src = p.db.partial + c;
        float acc = 0.f;
        int b = 0;
        for (; b + 8 <= p.db.blocks; b += 8) {
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __ldcg(src + static_cast<long long>(b + i) * p.db.pitch);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc += v[i];
        }
        for (; b < p.db.blocks; ++b) acc += __ldcg(src + static_cast<long long>(b) * p.db.pitch);
        p.db.out[c] = acc;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer (first CTA of the pair only) =====================
    if (lane == 0 && leader) {
      // Descriptor geometry.  Reduction-contiguous tiles: rows of 128 bytes, 8-row groups 1024 bytes apart,
      // a k-step of one MMA is 32 bytes inside the swizzled row.  M/N-contiguous tiles: each 128-byte row holds
      // one reduction index, 8 reduction rows form a 1024-byte group, and the next block of 128 bytes along M/N
      // starts kBlockK rows later; a k-step is kUmmaK rows.
      // 32-bit operands with M/N contiguous use the 32-byte-unit swizzle, whose pattern repeats every 4 rows.
      constexpr uint32_t kLboMN = Cfg::kBlockK * 128, kSbo = 1024;
      constexpr uint32_t kSboMN = kTf32 ? 512 : 1024;
      constexpr uint32_t kTypeMN = kTf32 ? 1u : 2u;
      constexpr uint64_t kStageEnc = Cfg::kStageBytes >> 4;       // descriptor address field counts 16-byte units
      const uint32_t empty0 = empty_bar(0), tfull0 = tfull_bar(0);
      const uint32_t empty_peer0 = (kCG == 2) ? ptx::map_to_cta(empty0, 1u) : 0u;
      const uint32_t tfull_peer0 = (kCG == 2) ? ptx::map_to_cta(tfull0, 1u) : 0u;
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      // The k-loop of one item whose operands are stored in the orders AMN / BMN.  Everything that does not change
      // from one k-block to the next is computed before the loop: the issuing thread shares its scheduler with an
      // epilogue warp, so the per-k-block instruction stream has to stay short.
      auto issue = [&](auto amn_c, auto bmn_c, uint32_t idesc, int k_blocks) {
        constexpr bool AMN = decltype(amn_c)::value, BMN = decltype(bmn_c)::value;
        constexpr uint64_t kAStepEnc = (AMN ? Cfg::kUmmaK * 128 : 32) >> 4, kBStepEnc = (BMN ? Cfg::kUmmaK * 128 : 32) >> 4;
        const uint64_t a_desc0 = AMN ? ptx::make_smem_desc_sw128(smem_base, kLboMN, kSboMN, kTypeMN)
                                     : ptx::make_smem_desc_sw128(smem_base, 0u, kSbo);
        const uint64_t b_desc0 = BMN ? ptx::make_smem_desc_sw128(smem_base + Cfg::kAStage, kLboMN, kSboMN, kTypeMN)
                                     : ptx::make_smem_desc_sw128(smem_base + Cfg::kAStage, 0u, kSbo);
        if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { ok = false; return; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint64_t ad = a_desc0 + stage * kStageEnc;
          const uint64_t bd = b_desc0 + stage * kStageEnc;
#pragma unroll
          for (int ks = 0; ks < Cfg::kBlockK / Cfg::kUmmaK; ++ks) {
            const uint32_t accum = (kb > 0 || ks > 0) ? 1u : 0u;
            if constexpr (kCG == 2) ptx::umma_pair<kTf32>(d_tmem, ad + ks * kAStepEnc, bd + ks * kBStepEnc, idesc, accum);
            else                    ptx::umma<kTf32>(d_tmem, ad + ks * kAStepEnc, bd + ks * kBStepEnc, idesc, accum);
          }
          // frees this ring slot (in both CTAs of a pair) once the MMAs have read it
          if constexpr (kCG == 2) {
            ptx::umma_commit_pair(empty0 + 8u * stage);
            ptx::umma_commit_pair(empty_peer0 + 8u * stage);
          } else {
            ptx::umma_commit(empty0 + 8u * stage);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) return;
        // accumulator complete: the epilogue warps (of both CTAs) may start
        if constexpr (kCG == 2) {
          ptx::umma_commit_pair(tfull0 + 8u * acc);
          ptx::umma_commit_pair(tfull_peer0 + 8u * acc);
        } else {
          ptx::umma_commit(tfull0 + 8u * acc);
        }
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      };
      for (long long item = unit; ok && item < total_items; item += n_units) {
        if constexpr (kDual) {
          if (item >= items1) { issue(BoolC<kAMN2>{}, BoolC<kBMN2>{}, d2.p.idesc, d2.p.k_blocks); continue; }
        }
        int k_blocks = p.k_blocks;
        const uint32_t idesc = (kNarrow && item >= p.main_tiles) ? p.idesc_half : p.idesc;
        if constexpr (kSplit) {
          if (item >= p.main_tiles) { const WorkItem w = decode_work(p, item); k_blocks = w.kb1 - w.kb0; }
        }
        issue(BoolC<kAMN>{}, BoolC<kBMN>{}, idesc, k_blocks);
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue (4 warps, one TMEM lane quarter each) =====================
    const int q = warp & 3;                            // hardware rule: a warp reads lanes 32*(warp%4)..+31
    const int half = (warp - 2) >> 2;                  // which half of the tile's columns this warp owns
    EpiStage my_stage{store_stage + (warp - 2) * kStoreStageWarp, 0};
    const uint32_t tempty_leader = (kCG == 2) ? ptx::map_to_cta(tempty_bar(0), 0u) : tempty_bar(0);
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    for (long long item = unit; ok && item < total_items; item += n_units) {
      const bool second = kDual && item >= items1;              // item of the second problem of a dual launch
      const TcParams& pp = second ? d2.p : p;
      const CUtensorMap* mD = second ? &d2.tmD : &tmD;
      const WorkItem w = second ? get_work<false, false>(d2.p, item - items1) : get_work<kSplit, kNarrow>(p, item);
      const int b = w.b;
      const int row_in_tile = static_cast<int>(cta_rank) * kBlockM + q * 32 + lane;
      const int row = w.mb * kTileM + row_in_tile;
      const bool row_ok = row < pp.M;
      const int n0 = w.nb * kBlockN + w.n_off;
      const int half_cols = (kNarrow && w.narrow) ? kBlockN / 4 : kBlockN / 2;   // columns of this warp's half
      if (!ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * kBlockN + half * half_cols + (static_cast<uint32_t>(q * 32) << 16);
      const int nh0 = n0 + half * half_cols;           // first column of this warp's half
      const int n_chunks = max(0, min(half_cols / 32, (pp.N - nh0 + 31) / 32));
      auto release_acc = [&]() {
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCG == 2) ptx::mbar_arrive_cluster(tempty_leader + 8u * acc);
          else                    ptx::mbar_arrive(tempty_bar(acc));
        }
      };
      if constexpr (!kSplit) {
        // Software pipeline over 32-column chunks: the TMEM load of chunk c+1 is in flight while chunk c is being
        // processed, and the accumulator is handed back to the MMA warp as soon as its last chunk is in registers.
        auto chunk_step = [&](int c, uint32_t (&cur)[32], uint32_t (&nxt)[32]) {
          ptx::tmem_wait_ld();                         // `cur` has landed
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(cur[j]);
          if (c + 1 < n_chunks) ptx::tmem_ld_32x32(t_row + (c + 1) * 32, nxt);
          else                  release_acc();
          const int col0 = nh0 + c * 32;
          epilogue_frag(pp, mD, &tmZ, v, b, row, col0, min(32, pp.N - col0), row_ok, my_stage, lane, (c & 1) != 0,
                        c + 1 == n_chunks);
        };
        uint32_t r0[32], r1[32];
        if (n_chunks == 0) release_acc();
        else ptx::tmem_ld_32x32(t_row, r0);
#pragma unroll 1
        for (int c = 0; c < n_chunks; c += 2) {
          chunk_step(c, r0, r1);
          if (c + 1 < n_chunks) chunk_step(c + 1, r1, r0);
        }
      } else {
        // fp32 partial sums of split tiles: [slice][tail tile][row in tile][column in tile]
        const size_t tile_elems = static_cast<size_t>(kTileM) * kBlockN;
        float* ws_row = nullptr;
        if (w.split)
          ws_row = pp.ws + (static_cast<size_t>(w.slice) * pp.tail_tiles + w.tail) * tile_elems +
                   static_cast<size_t>(row_in_tile) * kBlockN + half * (kBlockN / 2);
        if (n_chunks == 0) release_acc();
#pragma unroll 1
        for (int c = 0; c < n_chunks; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_row + c * 32, r);
          ptx::tmem_wait_ld();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (c + 1 == n_chunks) release_acc();
          const int col0 = nh0 + c * 32;
          if (w.split) {                               // leave this slice's partial sums
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                __stcg(reinterpret_cast<float4*>(ws_row + c * 32) + j,
                       make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
            }
            continue;
          }
          epilogue_frag(pp, mD, &tmZ, v, b, row, col0, min(32, pp.N - col0), row_ok, my_stage, lane, (c & 1) != 0,
                        c + 1 == n_chunks);
        }
        if (w.split && pp.fin_in_kernel) {
          // count this warp's part of the tile as written; the last of the `split` warps that own this part adds up
          // all slices (slice order, so the sum is the same whoever comes last) and finishes the tile
          __threadfence();
          __syncwarp();
          int arrived = 0;
          if (lane == 0)
            arrived = atomicAdd(pp.flags + w.tail * (kEpiWarps * kCG) + static_cast<int>(cta_rank) * kEpiWarps + (warp - 2), 1);
          arrived = __shfl_sync(0xffffffffu, arrived, 0);
          if (arrived == pp.split - 1) {
            __threadfence();
            // last of the slices: put the counter back to zero for the next launch that uses these counters (launches
            // on one stream are ordered, and every warp slot of every tile has exactly one last arriver)
            if (lane == 0)
              pp.flags[w.tail * (kEpiWarps * kCG) + static_cast<int>(cta_rank) * kEpiWarps + (warp - 2)] = 0;
            const float* sum_row = pp.ws + static_cast<size_t>(w.tail) * tile_elems +
                                   static_cast<size_t>(row_in_tile) * kBlockN + half * (kBlockN / 2);
            const size_t slice_stride = static_cast<size_t>(pp.tail_tiles) * tile_elems;
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = 0.f;
              // The partial sums come from L2, about a microsecond away: the loads of two slices are issued together
              // and only then added (in slice order), so a tile cut into `split` slices pays ceil(split / 2) round
              // trips per chunk instead of `split` (three or four at a time would spill registers).
              for (int sl0 = 0; row_ok && sl0 < pp.split; sl0 += 2) {
                const bool two = sl0 + 1 < pp.split;
                const float4* s0 = reinterpret_cast<const float4*>(sum_row + sl0 * slice_stride + c * 32);
                const float4* s1 = reinterpret_cast<const float4*>(sum_row + (two ? sl0 + 1 : sl0) * slice_stride + c * 32);
                float4 f0[8], f1[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f0[j] = __ldcg(s0 + j);
#pragma unroll
                for (int j = 0; j < 8; ++j) f1[j] = __ldcg(s1 + j);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  v[4 * j] += f0[j].x; v[4 * j + 1] += f0[j].y; v[4 * j + 2] += f0[j].z; v[4 * j + 3] += f0[j].w;
                }
                if (two) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    v[4 * j] += f1[j].x; v[4 * j + 1] += f1[j].y; v[4 * j + 2] += f1[j].z; v[4 * j + 3] += f1[j].w;
                  }
                }
              }
              const int col0 = nh0 + c * 32;
              epilogue_frag(pp, mD, &tmZ, v, b, row, col0, min(32, pp.N - col0), row_ok, my_stage, lane, (c & 1) != 0,
                        c + 1 == n_chunks);
            }
          }
        }
      }
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
    // this warp's bulk stores must have left shared memory (and reached global memory) before the CTA goes away
    if (lane == 0) ptx::bulk_wait_group_all();
    __syncwarp();
  }

  __syncthreads();
  if (*abort_flag != 0) {
    // A wait ran out: give copies still in flight time to land before shared memory is released.
    if (threadIdx.x == 0) atomicOr(p.status, kErrWaitTimeout);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
    __syncthreads();
  }
  if constexpr (kCG == 2) {
    // Neither CTA may leave (or free TMEM) while its partner can still signal it or read its shared memory.
    ptx::tc_fence_before_sync();
    ptx::cluster_sync_all();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if constexpr (kCG == 2) ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else                    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


// Second step of a split-K launch: adds the slices' partial tiles in slice order (so the result does not depend on
// which CTA finished first) and applies the epilogue.  grid.x = tail tile, grid.y = row group of the tile; a thread
// owns four consecutive columns, so the partial sums are read with coalesced 16-byte loads.
template <int ACT>
__device__ __forceinline__ float finalize_act(float v, float leaky, bool fast) {
  return fast ? act_fwd<ACT, true>(v, leaky) : act_fwd<ACT, false>(v, leaky);
}

static __global__ void __launch_bounds__(256)
splitk_finalize_kernel(const TcParams p, const int tile_m, const int tile_n) {
  const int r = blockIdx.x;
  int b, mb, nb;
  decode_tile(p, static_cast<long long>(p.main_tiles) + r, b, mb, nb);
  const int quads = tile_n / 4;
  const int quad = threadIdx.x % quads;
  const int rows_per_pass = 256 / quads;
  const size_t tile_elems = static_cast<size_t>(tile_m) * tile_n;
  const EpilogueArgs& e = p.epi;
  const bool fast = e.d_dtype != kF32;
  const int col0 = nb * tile_n + quad * 4;
  if (col0 >= p.N) return;
  for (int rt = blockIdx.y * rows_per_pass + threadIdx.x / quads; rt < tile_m; rt += gridDim.y * rows_per_pass) {
    const int row = mb * tile_m + rt;
    if (row >= p.M) break;
    const float* src = p.ws + static_cast<size_t>(r) * tile_elems + static_cast<size_t>(rt) * tile_n + quad * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sl = 0; sl < p.split; ++sl) {
      const float4 f = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(sl) * p.tail_tiles * tile_elems));
      acc.x += f.x; acc.y += f.y; acc.z += f.z; acc.w += f.w;
    }
    float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = col0 + j;
      if (col >= p.N) break;
      float x = v[j] * e.alpha;
      if (e.C != nullptr && e.beta != 0.f)
        x = fmaf(e.beta, load_as_f32(e.C, static_cast<long long>(b) * e.strideC + static_cast<long long>(row) * e.ldc + col, e.d_dtype), x);
      if (e.bias != nullptr) {
        if (e.bias_kind == kBiasPerN)      x += __ldg(e.bias + col);
        else if (e.bias_kind == kBiasPerM) x += __ldg(e.bias + row);
        else if (e.bias_kind == kBiasScalar) x += __ldg(e.bias);
      }
      if (e.Z != nullptr)
        store_from_f32(e.Z, static_cast<long long>(b) * e.strideZ + static_cast<long long>(row) * e.ldz + col, e.z_dtype, x);
      switch (e.act) {
        case kActReLU:    x = finalize_act<kActReLU>(x, e.leaky, false); break;
        case kActLeaky:   x = finalize_act<kActLeaky>(x, e.leaky, false); break;
        case kActGELU:    x = finalize_act<kActGELU>(x, e.leaky, fast); break;
        case kActSigmoid: x = finalize_act<kActSigmoid>(x, e.leaky, fast); break;
        case kActTanh:    x = finalize_act<kActTanh>(x, e.leaky, fast); break;
        default: break;
      }
      store_from_f32(e.D, static_cast<long long>(b) * e.strideD + static_cast<long long>(row) * e.ldd + col, e.d_dtype, x);
    }
  }
}

// ---- host helpers defined in gemm_tc.cu ----
bool make_operand_map(CUtensorMap* map, int dtype, const void* base, long long inner, long long rows, long long ld,
                      long long batch, long long batch_stride, int box_inner, int box_rows, bool swizzle_32b_units);
bool make_output_map(CUtensorMap* map, int dtype, const void* base, long long cols, long long rows, long long ld,
                     long long batch, long long batch_stride, bool wide);
bool driver_has_tensor_maps();
struct SplitScratch { float* ws = nullptr; int* flags = nullptr; size_t ws_bytes = 0; bool lent = false; };
constexpr size_t kSplitWsBytes = 64u << 20;
constexpr int kSplitMaxTail = 256;
constexpr int kSplitInKernelMax = 8;   // more slices than this: the second kernel adds them up
constexpr size_t kSplitFlagBytes = static_cast<size_t>(kSplitMaxTail) * kEpiWarps * 2 * sizeof(int);
// Split-K scratch for a launch on stream `s`: the memory the caller lent for this call (scratch_lease()) when there is
// one, else the library's own per-(device, stream) buffer, created on first use unless the lease forbids it or the
// stream is being captured.  Returns false when there is none; the launch then runs unsplit.
bool split_scratch(cudaStream_t s, SplitScratch* out);

// Everything one launch of gemm_tc_kernel needs, ready to be handed to the driver: built once per distinct problem
// (tensor maps are the expensive part) and replayed from a per-thread cache on later calls with the same arguments.
struct PreparedLaunch {
  const void* kernel = nullptr;
  unsigned grid = 0;
  int cluster = 1, smem = 0;
  CUtensorMap tmA, tmB, tmBh, tmD, tmZ;
  TcParams p;
  DualParams d2;
  size_t flag_bytes = 0;              // > 0: p.flags is zeroed on the stream before the launch
  int fin_gy = 0, fin_tile_m = 0, fin_tile_n = 0;   // fin_gy > 0: splitk_finalize_kernel follows
  bool cacheable = true;              // false: the launch ran unsplit only because no scratch could be had right now
};
cudaError_t run_prepared(const PreparedLaunch& L, cudaStream_t s);

struct ProblemMaps { CUtensorMap tmA, tmB, tmD, tmZ, tmAs, tmBs; };   // tmAs / tmBs: the small parts of an x3 problem

// Fills the geometry fields of `p` and the tensor maps of one problem for the given tile configuration.
template <int kElemBytes, bool kAMN, bool kBMN, int kBlockN, int kStages, int kCG>
bool prepare_problem(const GemmProblem& g, TcParams& p, ProblemMaps& m) {
  using Cfg = TcCfg<kElemBytes, kBlockN, kStages, kCG>;
  constexpr int kTileM = kBlockM * kCG;
  constexpr int kLocalN = kBlockN / kCG;
  p.m_blocks = (g.M + kTileM - 1) / kTileM;
  p.n_blocks = (g.N + kBlockN - 1) / kBlockN;
  p.k_blocks = (g.K + Cfg::kBlockK - 1) / Cfg::kBlockK;
  // up to 16 row-blocks: one group, i.e. column after column (measured 2 % faster than groups of 8 at 4096^3;
  // with 32 row-blocks groups of 16 or 32 were not better than 8)
  p.group_m = p.m_blocks <= 16 ? p.m_blocks : kGroupM;
  p.kb_per_slice = 0;
  p.x3_kb = 0;
  if (g.reduce_batch && g.batch > 1) {
    p.kb_per_slice = p.k_blocks;
    p.k_blocks *= g.batch;
  }
  if (g.in_dtype == kF32 && g.math == 2) {
    if (!g.A_small || !g.B_small || p.kb_per_slice > 0) return false;
    p.x3_kb = p.k_blocks;
    p.k_blocks *= 3;
  }
  const int ab_format = g.in_dtype == kF32 ? 2 : (g.in_dtype == kBF16 ? 1 : 0);
  p.idesc = ptx::make_idesc(ab_format, kAMN, kBMN, kTileM, kBlockN);
  p.idesc_half = ptx::make_idesc(ab_format, kAMN, kBMN, kTileM, kBlockN / 2);

  bool ok;
  constexpr bool kWide = (kElemBytes == 4);   // M/N-contiguous 32-bit tiles are swizzled in 32-byte units
  if (!kAMN) ok = make_operand_map(&m.tmA, g.in_dtype, g.A, g.K, g.M, g.lda, g.batch, g.strideA, Cfg::kBlockK, kBlockM, false);
  else       ok = make_operand_map(&m.tmA, g.in_dtype, g.A, g.M, g.K, g.lda, g.batch, g.strideA, Cfg::kBlockK, Cfg::kBlockK, kWide);
  if (!ok) return false;
  if (!kBMN) ok = make_operand_map(&m.tmB, g.in_dtype, g.B, g.K, g.N, g.ldb, g.batch, g.strideB, Cfg::kBlockK, kLocalN, false);
  else       ok = make_operand_map(&m.tmB, g.in_dtype, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, Cfg::kBlockK, Cfg::kBlockK, kWide);
  if (!ok) return false;
  m.tmAs = m.tmA; m.tmBs = m.tmB;
  if (p.x3_kb > 0) {
    if (!kAMN) ok = make_operand_map(&m.tmAs, g.in_dtype, g.A_small, g.K, g.M, g.lda, g.batch, g.strideA, Cfg::kBlockK, kBlockM, false);
    else       ok = make_operand_map(&m.tmAs, g.in_dtype, g.A_small, g.M, g.K, g.lda, g.batch, g.strideA, Cfg::kBlockK, Cfg::kBlockK, kWide);
    if (!ok) return false;
    if (!kBMN) ok = make_operand_map(&m.tmBs, g.in_dtype, g.B_small, g.K, g.N, g.ldb, g.batch, g.strideB, Cfg::kBlockK, kLocalN, false);
    else       ok = make_operand_map(&m.tmBs, g.in_dtype, g.B_small, g.N, g.K, g.ldb, g.batch, g.strideB, Cfg::kBlockK, Cfg::kBlockK, kWide);
    if (!ok) return false;
  }

  // Outputs as tensor maps for the epilogue's bulk stores (when base, pitch and batch stride allow).
  m.tmD = m.tmA; m.tmZ = m.tmA;
  // (the 64-column store pairs two 32-column chunks of one warp: a warp of the 64-wide tile has only one)
  p.store_wide = (p.d_vec && g.epi.Z == nullptr && g.epi.d_dtype != kF32 && kBlockN >= 128) ? 1 : 0;
  if (p.d_vec && !make_output_map(&m.tmD, g.epi.d_dtype, g.epi.D, g.N, g.M, g.epi.ldd, p.batch, g.epi.strideD,
                                  p.store_wide != 0)) {
    p.d_vec = 0;
    p.store_wide = 0;
  }
  if (p.z_vec && !make_output_map(&m.tmZ, g.epi.z_dtype, g.epi.Z, g.N, g.M, g.epi.ldz, p.batch, g.epi.strideZ, false))
    p.z_vec = 0;
  p.store_dbl = (g.epi.d_dtype != kF32 && (g.epi.Z == nullptr || g.epi.z_dtype != kF32)) ? 1 : 0;
  p.plain = (g.epi.C == nullptr && g.epi.bias == nullptr && g.epi.Z == nullptr && g.epi.act == kActNone) ? 1 : 0;
  p.main_tiles = static_cast<int>(static_cast<long long>(p.batch) * p.m_blocks * p.n_blocks);
  p.tail_tiles = 0;
  p.split = 1;
  return true;
}

template <int kElemBytes, bool kAMN, bool kBMN, int kBlockN, int kStages, int kCG>
cudaError_t prepare_cfg(const GemmProblem& g, TcParams& p, cudaStream_t s, PreparedLaunch& L) {
  using Cfg = TcCfg<kElemBytes, kBlockN, kStages, kCG>;
  auto kernel = gemm_tc_kernel<kElemBytes, kAMN, kBMN, kBlockN, kStages, kCG, false>;
  auto kernel_split = gemm_tc_kernel<kElemBytes, kAMN, kBMN, kBlockN, kStages, kCG, true>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(kernel_split, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;

  constexpr int kTileM = kBlockM * kCG;
  constexpr int kLocalN = kBlockN / kCG;
  ProblemMaps pm;
  if (!prepare_problem<kElemBytes, kAMN, kBMN, kBlockN, kStages, kCG>(g, p, pm)) return cudaErrorInvalidValue;
  L.tmA = pm.tmA; L.tmB = pm.tmB; L.tmD = pm.tmD; L.tmZ = pm.tmZ;
  L.d2.tmA = pm.tmAs; L.d2.tmB = pm.tmBs;         // read only when p.x3_kb > 0

  const long long tiles = static_cast<long long>(p.batch) * p.m_blocks * p.n_blocks;
  const long long units = sm_budget() / kCG > 0 ? sm_budget() / kCG : 1;   // one CTA (or CTA pair) per SM (pair of SMs)

  // Split-K: a problem whose tiles fill at most half of the machine is cut along the reduction as well.
  const long long rem = tiles % units;
  static const bool split_off = [] { const char* e = getenv("GE2B_SPLITK"); return e && atoi(e) == 0; }();
  // Only problems smaller than one wave are split: with several waves the measured gain of splitting just the last
  // one (half a wave at 4096^3) was eaten by the exchange of partial sums and the slower full-machine wave.
  if (!split_off && tiles < units && 2 * rem <= units && rem <= kSplitMaxTail) {
    long long sp = units / rem;
    if (sp > 32) sp = 32;
    // Splitting costs a fixed 10 to 18 us (partial tiles out to L2, a fence and a counter per warp, the last warp's
    // reads of every slice), measured on B200 against about 0.27 us per k-block of an unsplit tile: 1024^3 (16
    // k-blocks) ran in 23 us split and 12 us unsplit, 1024 x 1024 x 4096 (64 k-blocks) in 30 and 25.  It pays only for
    // long reductions, which are the HBM-bound skinny-M shapes (128 k-blocks at K = 8192: 32 us split, 42 unsplit).
    if (p.k_blocks < 96) sp = 1;
    if (sp > p.k_blocks / 24) sp = p.k_blocks / 24;             // keep at least 24 k-blocks per slice
    if (sp >= 2) {
      SplitScratch sc;
      if (split_scratch(s, &sc)) {
        size_t ws_bytes = sc.ws_bytes;              // bias-gradient partials of this launch sit at the end of the scratch
        const char* dbp = reinterpret_cast<const char*>(g.db.partial);
        if (dbp >= reinterpret_cast<const char*>(sc.ws) && dbp < reinterpret_cast<const char*>(sc.ws) + sc.ws_bytes)
          ws_bytes = static_cast<size_t>(dbp - reinterpret_cast<const char*>(sc.ws));
        while (sp >= 2 && static_cast<size_t>(sp) * rem * kTileM * kBlockN * sizeof(float) > ws_bytes) --sp;
        if (sp >= 2) {
          p.main_tiles = static_cast<int>(tiles - rem);
          p.tail_tiles = static_cast<int>(rem);
          p.split = static_cast<int>(sp);
          p.ws = sc.ws;
          p.flags = sc.flags;
          p.fin_in_kernel = sp <= kSplitInKernelMax ? 1 : 0;
          // the library's own counters are zero when created and every launch leaves them zero; lent memory holds
          // whatever the caller left there, so it is cleared on the stream first
          if (p.fin_in_kernel && sc.lent) L.flag_bytes = static_cast<size_t>(rem) * kEpiWarps * kCG * sizeof(int);
        }
      } else {
        L.cacheable = false;
      }
    }
  }
  // Narrow tail: several waves whose last one fills at most half of the pairs.
  bool narrow_tail = false;
  static const bool narrow_off = [] { const char* e = getenv("GE2B_NARROW_TAIL"); return e && atoi(e) == 0; }();
  if (kCG == 2 && kBlockN == 256 && !narrow_off && p.x3_kb == 0 && p.split == 1 && tiles > units && rem > 0 &&
      2 * rem <= units) {
    narrow_tail = true;
    p.main_tiles = static_cast<int>(tiles - rem);
    p.tail_tiles = static_cast<int>(rem);
    p.split = 2;
  }
  L.tmBh = L.tmB;
  if (narrow_tail && !kBMN &&
      !make_operand_map(&L.tmBh, g.in_dtype, g.B, g.K, g.N, g.ldb, g.batch, g.strideB, Cfg::kBlockK, kLocalN / 2, false))
    return cudaErrorInvalidValue;
  const long long items = static_cast<long long>(p.main_tiles) + static_cast<long long>(p.tail_tiles) * p.split;
  L.grid = static_cast<unsigned>((items < units ? items : units) * kCG);
  L.cluster = kCG;
  L.smem = Cfg::kSmemBytes;
  L.kernel = reinterpret_cast<const void*>(kernel);
  if (p.split > 1 && !narrow_tail) {
    L.kernel = reinterpret_cast<const void*>(kernel_split);
    if (!p.fin_in_kernel) {
      const int quads = kBlockN / 4, rows_per_pass = 256 / quads;
      int gy = kTileM / rows_per_pass;                    // one pass per block when the grid is small ...
      while (gy > 1 && static_cast<long long>(p.tail_tiles) * gy > 8ll * units) gy >>= 1;   // ... fewer blocks when it is not
      L.fin_gy = gy; L.fin_tile_m = kTileM; L.fin_tile_n = kBlockN;
    }
  }
  L.p = p;
  return cudaSuccess;
}

// Two independent problems in one persistent launch (CTA pairs, 256 x 256 tiles, no split-K, no narrow tail): the
// tiles of the second follow those of the first in one list.  Both must be 16-bit or both 32-bit, and both must leave
// through the same kind of store (checked by the caller through the filled TcParams).
template <int kElemBytes, bool kAMN1, bool kBMN1, bool kAMN2, bool kBMN2>
cudaError_t prepare_dual_cfg(const GemmProblem& g1, TcParams& p1, const GemmProblem& g2, TcParams& p2, PreparedLaunch& L) {
  constexpr int kBlockN = 256, kStages = 6, kCG = 2;
  using Cfg = TcCfg<kElemBytes, kBlockN, kStages, kCG>;
  auto kernel = gemm_tc_kernel<kElemBytes, kAMN1, kBMN1, kBlockN, kStages, kCG, false, true, kAMN2, kBMN2>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;
  ProblemMaps m1, m2;
  if (!prepare_problem<kElemBytes, kAMN1, kBMN1, kBlockN, kStages, kCG>(g1, p1, m1)) return cudaErrorInvalidValue;
  if (!prepare_problem<kElemBytes, kAMN2, kBMN2, kBlockN, kStages, kCG>(g2, p2, m2)) return cudaErrorInvalidValue;
  if (p1.store_wide != p2.store_wide || p1.store_dbl != p2.store_dbl || g2.epi.Z != nullptr) return cudaErrorNotSupported;
  L.d2.tmA = m2.tmA; L.d2.tmB = m2.tmB; L.d2.tmD = m2.tmD;
  L.d2.p = p2;
  const long long items = static_cast<long long>(p1.main_tiles) + p2.main_tiles;
  const long long units = sm_budget() / kCG > 0 ? sm_budget() / kCG : 1;
  L.tmA = m1.tmA; L.tmB = m1.tmB; L.tmBh = m1.tmB; L.tmD = m1.tmD; L.tmZ = m1.tmZ;
  L.p = p1;
  L.grid = static_cast<unsigned>((items < units ? items : units) * kCG);
  L.cluster = kCG;
  L.smem = Cfg::kSmemBytes;
  L.kernel = reinterpret_cast<const void*>(kernel);
  return cudaSuccess;
}

struct TileChoice { int block_n, cta_group; };

template <int kElemBytes, bool kAMN, bool kBMN>
cudaError_t prepare_bn(const GemmProblem& g, TcParams& p, TileChoice t, cudaStream_t s, PreparedLaunch& L) {
  if (t.cta_group == 2 && t.block_n == 256) return prepare_cfg<kElemBytes, kAMN, kBMN, 256, 6, 2>(g, p, s, L);
  if (t.block_n == 128) return prepare_cfg<kElemBytes, kAMN, kBMN, 128, 6, 1>(g, p, s, L);
  if (t.block_n == 64) return prepare_cfg<kElemBytes, kAMN, kBMN, 64, 8, 1>(g, p, s, L);
  return prepare_cfg<kElemBytes, kAMN, kBMN, 256, 4, 1>(g, p, s, L);
}

// Defined (explicitly instantiated) in the gemm_tc_inst_*.cu files.
#define GE2B_TC_DECLARE(E, A, B) \
  extern template cudaError_t prepare_bn<E, A, B>(const GemmProblem&, TcParams&, TileChoice, cudaStream_t, PreparedLaunch&);
GE2B_TC_DECLARE(2, false, false) GE2B_TC_DECLARE(2, false, true) GE2B_TC_DECLARE(2, true, false) GE2B_TC_DECLARE(2, true, true)
GE2B_TC_DECLARE(4, false, false) GE2B_TC_DECLARE(4, false, true) GE2B_TC_DECLARE(4, true, false) GE2B_TC_DECLARE(4, true, true)
#undef GE2B_TC_DECLARE
extern template cudaError_t prepare_dual_cfg<2, false, false, true, true>(const GemmProblem&, TcParams&, const GemmProblem&,
                                                                           TcParams&, PreparedLaunch&);
extern template cudaError_t prepare_dual_cfg<4, false, false, true, true>(const GemmProblem&, TcParams&, const GemmProblem&,
                                                                           TcParams&, PreparedLaunch&);

}  // namespace tc
}  // namespace ge2b
