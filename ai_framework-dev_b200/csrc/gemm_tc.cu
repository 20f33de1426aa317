// Tensor-core GEMM: host-side helpers (tensor maps, split-K scratch), tile choice and dispatch.  The kernel template
// lives in gemm_tc_kernel.cuh and is instantiated by the gemm_tc_inst_*.cu files.
#include <atomic>
#include <cstring>
#include <map>
#include <utility>
#include <vector>

#include "gemm_tc_kernel.cuh"

namespace ge2b {
namespace tc {

// ------------------------------------------------------------------------------------------------
// Host side: tensor maps, configuration choice, launch.
// ------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn_impl() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 3-D map {inner, rows, batch} over a row-major operand; box {box_inner, box_rows, 1}, 128-byte swizzle,
// out-of-range elements read as zero (which makes ragged K, M and N tiles correct without special code).
bool make_operand_map(CUtensorMap* map, int dtype, const void* base, long long inner, long long rows, long long ld,
                      long long batch, long long batch_stride, int box_inner, int box_rows, bool swizzle_32b_units) {
  EncodeTiledFn enc = encode_tiled_fn_impl();
  if (!enc) return false;
  const int esz = dtype_bytes(dtype);
  const CUtensorMapDataType dt = dtype == kF32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (batch_stride <= 0 || batch <= 1) { batch = 1; batch_stride = rows * ld; }
  cuuint64_t dims[3]    = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * esz, static_cast<cuuint64_t>(batch_stride) * esz};
  cuuint32_t box[3]     = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows), 1u};
  cuuint32_t estr[3]    = {1u, 1u, 1u};
  const CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle_32b_units ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 3-D map {columns, rows, batch} over a row-major output for the epilogue's bulk stores: box of 32 x 32 elements
// (64 x 32 in the `wide` form of 16-bit single-output launches), swizzled the way the epilogue lays its staging
// buffer out (64-byte rows for 32 16-bit elements, 128-byte rows otherwise).
bool make_output_map(CUtensorMap* map, int dtype, const void* base, long long cols, long long rows, long long ld,
                     long long batch, long long batch_stride, bool wide) {
  EncodeTiledFn enc = encode_tiled_fn_impl();
  if (!enc) return false;
  const int esz = dtype_bytes(dtype);
  const CUtensorMapDataType dt = dtype == kF32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (batch_stride <= 0 || batch <= 1) { batch = 1; batch_stride = rows * ld; }
  cuuint64_t dims[3]    = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * esz, static_cast<cuuint64_t>(batch_stride) * esz};
  cuuint32_t box[3]     = {wide ? 64u : 32u, 32u, 1u};
  cuuint32_t estr[3]    = {1u, 1u, 1u};
  const CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         (esz == 4 || wide) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool tensor_vec_ok(const void* p, long long ld, long long batch_stride, int dt) {
  if (!p) return false;
  const int esz = dtype_bytes(dt);
  return aligned16(p) && (ld * esz) % 16 == 0 && (batch_stride * esz) % 16 == 0;
}

// Scratch of split-K launches (fp32 partial tiles + one arrival counter per tile and epilogue-warp slot).
//
// Where it comes from, in this order:
//   1. memory the caller lent for the duration of the call (scratch_lease(): the operator API's lt_workspace, the tail
//      of the fixed array of the allocation-free backward entry); nothing is allocated;
//   2. the library's own buffer, one per (device, stream): launches on one stream are ordered, launches on different
//      streams get different buffers.  It is created (cudaMalloc) the first time a split launch arrives on that
//      stream, which cannot happen while the stream is being captured or when the lease forbids allocation; the launch
//      then runs unsplit and `split_unavailable_total()` counts it.  Warm a shape up once, on the stream that will
//      be captured, before capturing it.  release_library_scratch() frees all of them.
namespace {
struct OwnedScratch { float* ws = nullptr; int* flags = nullptr; };
std::mutex g_scratch_mu;
std::map<std::pair<int, cudaStream_t>, OwnedScratch> g_scratch_table;
std::atomic<long long> g_split_unavailable{0};
}  // namespace

bool split_scratch(cudaStream_t s, SplitScratch* out) {
  const ScratchLease& lease = scratch_lease();
  if (lease.base && lease.bytes >= kSplitFlagBytes + (1u << 20)) {
    // flags first (256-byte aligned base), partial tiles after them
    out->flags = static_cast<int*>(lease.base);
    out->ws = reinterpret_cast<float*>(static_cast<unsigned char*>(lease.base) + kSplitFlagBytes);
    out->ws_bytes = lease.bytes - kSplitFlagBytes;
    out->lent = true;
    return true;
  }
  if (lease.no_alloc) { g_split_unavailable.fetch_add(1, std::memory_order_relaxed); return false; }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  OwnedScratch& sc = g_scratch_table[{dev, s}];
  if (!sc.ws) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
      g_split_unavailable.fetch_add(1, std::memory_order_relaxed);
      return false;
    }
    if (cudaMalloc(reinterpret_cast<void**>(&sc.ws), kSplitWsBytes) != cudaSuccess) {
      cudaGetLastError();        // the failed allocation must not surface as the next launch's error
      sc.ws = nullptr;
      g_split_unavailable.fetch_add(1, std::memory_order_relaxed);
      return false;
    }
    if (cudaMalloc(reinterpret_cast<void**>(&sc.flags), kSplitFlagBytes) != cudaSuccess ||
        cudaMemset(sc.flags, 0, kSplitFlagBytes) != cudaSuccess) {
      cudaGetLastError();
      cudaFree(sc.ws); sc.ws = nullptr;
      if (sc.flags) { cudaFree(sc.flags); sc.flags = nullptr; }
      g_split_unavailable.fetch_add(1, std::memory_order_relaxed);
      return false;
    }
  }
  out->ws = sc.ws; out->flags = sc.flags; out->ws_bytes = kSplitWsBytes; out->lent = false;
  return true;
}

bool driver_has_tensor_maps() { return encode_tiled_fn_impl() != nullptr; }

}  // namespace tc

bool borrow_stream_scratch(cudaStream_t s, float** ws, size_t* ws_bytes, int** flags, size_t* flag_bytes, bool* lent) {
  tc::SplitScratch sc;
  if (!tc::split_scratch(s, &sc)) return false;
  *ws = sc.ws; *ws_bytes = sc.ws_bytes; *flags = sc.flags; *flag_bytes = tc::kSplitFlagBytes; *lent = sc.lent;
  return true;
}

long long split_unavailable_total() { return tc::g_split_unavailable.load(std::memory_order_relaxed); }

void release_library_scratch() {
  cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lk(tc::g_scratch_mu);
  int cur = 0;
  cudaGetDevice(&cur);
  for (auto& kv : tc::g_scratch_table) {
    if (!kv.second.ws) continue;
    cudaSetDevice(kv.first.first);
    cudaFree(kv.second.ws);
    cudaFree(kv.second.flags);
  }
  tc::g_scratch_table.clear();
  cudaSetDevice(cur);
  plan_cache_generation().fetch_add(1, std::memory_order_relaxed);   // cached launches may point into freed scratch
}

// GE2B_PDL=1 switches programmatic dependent launch on for the GEMM and prologue kernels.  Off by default: replayed
// from a CUDA graph the benchmark step measured the same with and without it (0.3021 / 0.3022 ms), since a graph's
// kernel-to-kernel dependencies already cost about as little; it is left in for eagerly launched sequences.
bool early_start_enabled() {
  static const bool on = [] { const char* e = getenv("GE2B_PDL"); return e && atoi(e) == 1; }();
  return on;
}

ScratchLease& scratch_lease() {
  thread_local ScratchLease lease;
  return lease;
}

std::atomic<unsigned long long>& plan_cache_generation() {
  static std::atomic<unsigned long long> gen{1};
  return gen;
}

namespace tc {

cudaError_t run_prepared(const PreparedLaunch& L, cudaStream_t s) {
  if (L.flag_bytes && cudaMemsetAsync(L.p.flags, 0, L.flag_bytes, s) != cudaSuccess) return cudaErrorUnknown;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(L.grid, 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(L.smem);
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(L.cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (early_start_enabled() && L.flag_bytes == 0) {     // (a memset before the launch is an ordinary dependency)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  void* args[] = {const_cast<CUtensorMap*>(&L.tmA), const_cast<CUtensorMap*>(&L.tmB), const_cast<CUtensorMap*>(&L.tmBh),
                  const_cast<CUtensorMap*>(&L.tmD), const_cast<CUtensorMap*>(&L.tmZ), const_cast<TcParams*>(&L.p),
                  const_cast<DualParams*>(&L.d2)};
  const cudaError_t e = cudaLaunchKernelExC(&cfg, L.kernel, args);
  if (e != cudaSuccess || L.fin_gy == 0) return e;
  splitk_finalize_kernel<<<dim3(L.p.tail_tiles, L.fin_gy), 256, 0, s>>>(L.p, L.fin_tile_m, L.fin_tile_n);
  return cudaGetLastError();
}

}  // namespace tc

namespace {
using namespace tc;

// ---- per-thread cache of prepared launches ----
// A launch is fully determined by the problem description (pointers, shapes, pitches, epilogue), the stream (whose
// split-K scratch it may use), the lent scratch, the device and the SM budget.  Encoding tensor maps costs several
// microseconds per map; a training step repeats the same few launches, so they are kept ready.  Tensor maps hold
// addresses and shapes only, so an entry stays valid even if the buffers behind the pointers are freed and given out
// again: the key then simply matches a problem with the same geometry at the same addresses.
struct PlanKey {
  static constexpr int kWords = 96;
  unsigned long long w[kWords];
  int n = 0;
  void add(unsigned long long v) { if (n < kWords) w[n++] = v; }
  void add_ptr(const void* p) { add(reinterpret_cast<unsigned long long>(p)); }
  void add_f(float f) { unsigned u; std::memcpy(&u, &f, 4); add(u); }
  unsigned long long hash() const {
    unsigned long long h = 1469598103934665603ull;
    for (int i = 0; i < n; ++i) { h ^= w[i]; h *= 1099511628211ull; }
    return h;
  }
  bool same(const PlanKey& o) const { return n == o.n && std::memcmp(w, o.w, sizeof(unsigned long long) * n) == 0; }
};

void key_problem(PlanKey& k, const GemmProblem& g) {
  k.add((static_cast<unsigned long long>(static_cast<unsigned>(g.M)) << 32) | static_cast<unsigned>(g.N));
  k.add((static_cast<unsigned long long>(static_cast<unsigned>(g.K)) << 32) | static_cast<unsigned>(g.batch));
  k.add(static_cast<unsigned long long>(g.in_dtype) | (static_cast<unsigned long long>(g.math) << 8) |
        (static_cast<unsigned long long>(g.a_mn) << 16) | (static_cast<unsigned long long>(g.b_mn) << 17) |
        (static_cast<unsigned long long>(g.reduce_batch) << 18) | (static_cast<unsigned long long>(g.epi.bias_kind) << 24) |
        (static_cast<unsigned long long>(g.epi.act) << 32) | (static_cast<unsigned long long>(g.epi.d_dtype) << 40) |
        (static_cast<unsigned long long>(g.epi.z_dtype) << 48));
  k.add_ptr(g.A); k.add(g.lda); k.add(g.strideA);
  k.add_ptr(g.B); k.add(g.ldb); k.add(g.strideB);
  k.add_ptr(g.epi.D); k.add(g.epi.ldd); k.add(g.epi.strideD);
  k.add_ptr(g.epi.Z); k.add(g.epi.ldz); k.add(g.epi.strideZ);
  k.add_ptr(g.epi.C); k.add(g.epi.ldc); k.add(g.epi.strideC);
  k.add_ptr(g.epi.bias);
  k.add_ptr(g.A_small); k.add_ptr(g.B_small);
  k.add_ptr(g.db.partial); k.add_ptr(g.db.out); k.add(g.db.pitch);
  k.add((static_cast<unsigned long long>(static_cast<unsigned>(g.db.blocks)) << 32) | static_cast<unsigned>(g.db.n));
  k.add_f(g.epi.leaky); k.add_f(g.epi.alpha); k.add_f(g.epi.beta);
}

void key_context(PlanKey& k, cudaStream_t s, int extra) {
  int dev = -1;
  cudaGetDevice(&dev);
  const ScratchLease& lease = scratch_lease();
  k.add_ptr(s); k.add_ptr(lease.base); k.add(lease.bytes);
  k.add(static_cast<unsigned long long>(dev + 1) | (static_cast<unsigned long long>(lease.no_alloc) << 16) |
        (static_cast<unsigned long long>(sm_budget()) << 32));
  k.add(static_cast<unsigned long long>(extra));
  k.add(plan_cache_generation().load(std::memory_order_relaxed));
}

struct PlanEntry { unsigned long long hash = 0, stamp = 0; PlanKey key; PreparedLaunch L; bool used = false; };
constexpr int kPlanEntries = 64;

struct PlanCache {
  std::vector<PlanEntry> e;
  unsigned long long clock = 0;
  PlanEntry* find(const PlanKey& k, unsigned long long h) {
    for (auto& x : e)
      if (x.used && x.hash == h && x.key.same(k)) { x.stamp = ++clock; return &x; }
    return nullptr;
  }
  PlanEntry* slot() {
    if (e.empty()) e.resize(kPlanEntries);
    PlanEntry* best = &e[0];
    for (auto& x : e) {
      if (!x.used) { best = &x; break; }
      if (x.stamp < best->stamp) best = &x;
    }
    return best;
  }
};
PlanCache& plan_cache() { thread_local PlanCache c; return c; }
const bool g_plan_cache_off = [] { const char* e = getenv("GE2B_PLAN_CACHE"); return e && atoi(e) == 0; }();

template <int kElemBytes>
cudaError_t prepare_major(const GemmProblem& g, TcParams& p, TileChoice t, cudaStream_t s, PreparedLaunch& L) {
  if (g.a_mn) return g.b_mn ? prepare_bn<kElemBytes, true, true>(g, p, t, s, L)
                            : prepare_bn<kElemBytes, true, false>(g, p, t, s, L);
  return g.b_mn ? prepare_bn<kElemBytes, false, true>(g, p, t, s, L)
                : prepare_bn<kElemBytes, false, false>(g, p, t, s, L);
}

// Tile choice.  Wide (256) tiles run the tensor pipe at full rate; narrow (128) tiles quantise better onto the
// SMs.  CTA pairs need at least two row blocks to be worth their while.  GE2B_BLOCK_N / GE2B_CTA_GROUP (read once)
// override.
TileChoice choose_tile(const GemmProblem& g) {
  TileChoice t{256, 1};
  static const int force_bn = [] { const char* e = getenv("GE2B_BLOCK_N"); const int v = e ? atoi(e) : 0; return (v == 64 || v == 128 || v == 256) ? v : 0; }();
  static const int force_cg = [] { const char* e = getenv("GE2B_CTA_GROUP"); const int v = e ? atoi(e) : 0; return (v == 1 || v == 2) ? v : 0; }();
  // A CTA pair (256 rows per tile, half of B per CTA, deeper ring) is the faster form whenever the problem has at
  // least two 128-row blocks; below that the second CTA of a pair would only compute padding.
  t.cta_group = force_cg ? force_cg : (g.M > 128 ? 2 : 1);
  const double sms = sm_budget();
  auto cost = [&](int bn, int cg, double rate) {
    const long long mb = (g.M + 128 * cg - 1) / (128 * cg);
    const long long tiles = static_cast<long long>(g.reduce_batch ? 1 : g.batch) * mb * ((g.N + bn - 1) / bn);
    const long long units = static_cast<long long>(sms) / cg;
    const double waves = static_cast<double>((tiles + units - 1) / units);
    return waves * bn / rate;      // time units: one 128-wide tile at full rate = 128
  };
  // measured on B200: a 128-wide tile reaches about 0.72 of the 256-wide tile's rate (single CTA; the pair form
  // of the narrow tile was slower still and is not built)
  if (force_bn) { t.block_n = force_bn; if (t.block_n <= 128) t.cta_group = 1; return t; }
  // Skinny M with a long reduction (decode-like: M <= 128, N = K = 8192) streams the weight matrix once and is bound
  // by HBM.  256-wide tiles give too few CTAs to pull it at full rate unless the reduction is split, and the split
  // costs 10 us or more; 64-wide tiles give N / 64 CTAs that each stream their own panel of B with nothing to
  // exchange (eight-deep ring).
  // Measured on B200 (M = 16 .. 128, N = K = 8192, graph replay): 40 us, against 32 us for 256-wide tiles with the
  // reduction split four ways -- eight stages of 10 KB of real data per SM are not enough bytes in flight to pull
  // HBM at full rate, and the 128-row A box fills most of every stage with zeros.  Off unless GE2B_SKINNY_64=1.
  static const bool skinny64 = [] { const char* e = getenv("GE2B_SKINNY_64"); return e && atoi(e) == 1; }();
  if (skinny64 && g.M <= 128 && !g.reduce_batch && g.K >= 2048) {
    const long long tiles64 = static_cast<long long>(g.batch) * ((g.N + 63) / 64);
    const long long tiles256 = static_cast<long long>(g.batch) * ((g.N + 255) / 256);
    if (tiles256 < static_cast<long long>(sms) && 10 * tiles64 >= 6 * static_cast<long long>(sms)) {
      t.block_n = 64; t.cta_group = 1;
      return t;
    }
  }
  if (g.N <= 128) { t.block_n = 128; t.cta_group = 1; return t; }
  if (cost(256, t.cta_group, 1.0) > cost(128, 1, 0.72)) { t.block_n = 128; t.cta_group = 1; }
  return t;
}

void fill_common(const GemmProblem& g, tc::TcParams& p) {
  p.M = g.M; p.N = g.N; p.K = g.K; p.batch = g.reduce_batch ? 1 : g.batch;
  p.a_bcast = (g.batch > 1 && g.strideA == 0) ? 1 : 0;
  p.b_bcast = (g.batch > 1 && g.strideB == 0) ? 1 : 0;
  p.epi = g.epi;
  p.d_vec = tensor_vec_ok(g.epi.D, g.epi.ldd, g.epi.strideD, g.epi.d_dtype);
  p.z_vec = tensor_vec_ok(g.epi.Z, g.epi.ldz, g.epi.strideZ, g.epi.z_dtype);
  p.c_vec = tensor_vec_ok(g.epi.C, g.epi.ldc, g.epi.strideC, g.epi.d_dtype);
  p.bias_vec = g.epi.bias && aligned16(g.epi.bias);
  p.db = g.db;
  p.status = device_status_ptr();
}

}  // namespace

bool gemm_tc_supported(const GemmProblem& g, const char** why) {
  auto fail = [&](const char* m) { if (why) *why = m; return false; };
  if (g.M < 1 || g.N < 1 || g.K < 1 || g.batch < 1) return fail("empty problem");
  if (g.in_dtype == kF32 && g.math != 1 && g.math != 2) return fail("fp32 operands without a tensor-core math mode");
  if (g.in_dtype == kF32 && g.math == 2 && (!g.A_small || !g.B_small || !aligned16(g.A_small) || !aligned16(g.B_small)))
    return fail("split operands of the compensated mode missing or unaligned");
  const int esz = dtype_bytes(g.in_dtype);
  if (!aligned16(g.A) || !aligned16(g.B)) return fail("operand base not 16-byte aligned");
  if ((g.lda * esz) % 16 || (g.ldb * esz) % 16) return fail("operand row pitch not a multiple of 16 bytes");
  if ((g.strideA * esz) % 16 || (g.strideB * esz) % 16) return fail("batch stride not a multiple of 16 bytes");
  if (g.strideA < 0 || g.strideB < 0) return fail("negative batch stride");
  if (!tc::driver_has_tensor_maps()) return fail("driver lacks cuTensorMapEncodeTiled");
  if (!g.epi.D) return fail("no output");
  return true;
}

cudaError_t launch_gemm_tc_dual(const GemmProblem& dx, const GemmProblem& dw, cudaStream_t s) {
  static const bool off = [] { const char* e = getenv("GE2B_DUAL_BWD"); return e && atoi(e) == 0; }();
  if (off) return cudaErrorNotSupported;
  // the pair form: both problems unbatched, same element size, the orders of a dense backward, large enough for
  // CTA pairs, plain epilogues with TMA-storable 16-byte aligned outputs
  if (dx.batch != 1 || dw.batch != 1 || dx.in_dtype != dw.in_dtype) return cudaErrorNotSupported;
  if (dx.math == 2 || dw.math == 2) return cudaErrorNotSupported;   // the compensated mode uses the second-problem slot
  if (dx.a_mn || dx.b_mn || !dw.a_mn || !dw.b_mn) return cudaErrorNotSupported;
  if (dx.M <= 128 || dw.M <= 128 || dx.N <= 128 || dw.N <= 128) return cudaErrorNotSupported;
  // worth it only when the combined list quantises better than the two lists do separately
  const long long units = sm_budget() / 2 > 0 ? sm_budget() / 2 : 1;
  auto tiles = [](const GemmProblem& g) { return static_cast<long long>((g.M + 255) / 256) * ((g.N + 255) / 256); };
  auto waves = [&](long long t) { return (t + units - 1) / units; };
  if (tiles(dx) + tiles(dw) < units) return cudaErrorNotSupported;   // small problems are better off with split-K each
  if (waves(tiles(dx) + tiles(dw)) >= waves(tiles(dx)) + waves(tiles(dw))) return cudaErrorNotSupported;

  PlanKey key;
  PlanEntry* hit = nullptr;
  unsigned long long h = 0;
  if (!g_plan_cache_off) {
    key_problem(key, dx); key_problem(key, dw); key_context(key, s, 2);
    h = key.hash();
    hit = plan_cache().find(key, h);
    if (hit) return run_prepared(hit->L, s);
  }
  if (!gemm_tc_supported(dx, nullptr) || !gemm_tc_supported(dw, nullptr)) return cudaErrorNotSupported;
  if (dx.epi.Z || dw.epi.Z || dx.epi.d_dtype != dw.epi.d_dtype) return cudaErrorNotSupported;
  TcParams p1{}, p2{};
  fill_common(dx, p1);
  fill_common(dw, p2);
  if (!p1.status || !p1.d_vec || !p2.d_vec) return cudaErrorNotSupported;
  PreparedLaunch L;
  const cudaError_t e = dx.in_dtype == kF32 ? tc::prepare_dual_cfg<4, false, false, true, true>(dx, p1, dw, p2, L)
                                            : tc::prepare_dual_cfg<2, false, false, true, true>(dx, p1, dw, p2, L);
  if (e != cudaSuccess) return e;
  if (!g_plan_cache_off && L.cacheable) {
    PlanEntry* slot = plan_cache().slot();
    slot->key = key; slot->hash = h; slot->L = L; slot->used = true; slot->stamp = ++plan_cache().clock;
  }
  return run_prepared(L, s);
}

cudaError_t launch_gemm_tc(const GemmProblem& g, cudaStream_t s) {
  PlanKey key;
  unsigned long long h = 0;
  if (!g_plan_cache_off) {
    key_problem(key, g); key_context(key, s, 1);
    h = key.hash();
    if (PlanEntry* hit = plan_cache().find(key, h)) return run_prepared(hit->L, s);
  }
  TcParams p{};
  fill_common(g, p);
  if (!p.status) return cudaErrorInvalidDevice;
  const TileChoice t = choose_tile(g);
  PreparedLaunch L;
  const cudaError_t e = g.in_dtype == kF32 ? prepare_major<4>(g, p, t, s, L) : prepare_major<2>(g, p, t, s, L);
  if (e != cudaSuccess) return e;
  if (!g_plan_cache_off && L.cacheable) {
    PlanEntry* slot = plan_cache().slot();
    slot->key = key; slot->hash = h; slot->L = L; slot->used = true; slot->stamp = ++plan_cache().clock;
  }
  return run_prepared(L, s);
}

}  // namespace ge2b
