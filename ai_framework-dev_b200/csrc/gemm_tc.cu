// Tensor-core GEMM: host-side helpers (tensor maps, split-K scratch), tile choice and dispatch.  The kernel template
// lives in gemm_tc_kernel.cuh and is instantiated by the gemm_tc_inst_*.cu files.
#include <map>
#include <utility>

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

// Scratch of split-K launches (fp32 partial tiles + one arrival counter per tile and epilogue-warp slot).  One buffer per
// (device, stream), created the first time a launch on that stream needs it and kept for the life of the process:
// launches on one stream are ordered, launches on different streams get different buffers.  Creating it allocates
// device memory, so the first split launch on a stream must happen outside stream capture (warm the shape up once).

SplitScratch* split_scratch(cudaStream_t s) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, SplitScratch> table;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  SplitScratch& sc = table[{dev, s}];
  if (!sc.ws) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&sc.ws), kSplitWsBytes) != cudaSuccess) { sc.ws = nullptr; return nullptr; }
    if (cudaMalloc(reinterpret_cast<void**>(&sc.flags), kSplitMaxTail * kEpiWarps * 2 * sizeof(int)) != cudaSuccess) {
      cudaFree(sc.ws); sc.ws = nullptr; return nullptr;
    }
    sc.ws_bytes = kSplitWsBytes;
  }
  return &sc;
}


bool driver_has_tensor_maps() { return encode_tiled_fn_impl() != nullptr; }

}  // namespace tc

namespace {
using namespace tc;

template <int kElemBytes>
cudaError_t launch_major(const GemmProblem& g, TcParams& p, TileChoice t, cudaStream_t s) {
  if (g.a_mn) return g.b_mn ? launch_bn<kElemBytes, true, true>(g, p, t, s)
                            : launch_bn<kElemBytes, true, false>(g, p, t, s);
  return g.b_mn ? launch_bn<kElemBytes, false, true>(g, p, t, s)
                : launch_bn<kElemBytes, false, false>(g, p, t, s);
}

// Tile choice.  Wide (256) tiles run the tensor pipe at full rate; narrow (128) tiles quantise better onto the
// SMs.  CTA pairs need at least two row blocks to be worth their while.  GE2B_BLOCK_N / GE2B_CTA_GROUP override.
TileChoice choose_tile(const GemmProblem& g) {
  TileChoice t{256, 1};
  int force_bn = 0, force_cg = 0;
  if (const char* e = getenv("GE2B_BLOCK_N")) { const int v = atoi(e); if (v == 128 || v == 256) force_bn = v; }
  if (const char* e = getenv("GE2B_CTA_GROUP")) { const int v = atoi(e); if (v == 1 || v == 2) force_cg = v; }
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
  if (force_bn) { t.block_n = force_bn; if (t.block_n == 128) t.cta_group = 1; return t; }
  if (g.N <= 128) { t.block_n = 128; t.cta_group = 1; return t; }
  if (cost(256, t.cta_group, 1.0) > cost(128, 1, 0.72)) { t.block_n = 128; t.cta_group = 1; }
  return t;
}

}  // namespace

bool gemm_tc_supported(const GemmProblem& g, const char** why) {
  auto fail = [&](const char* m) { if (why) *why = m; return false; };
  if (g.M < 1 || g.N < 1 || g.K < 1 || g.batch < 1) return fail("empty problem");
  if (g.in_dtype == kF32 && g.math != 1) return fail("fp32 operands without TF32 opt-in");
  const int esz = dtype_bytes(g.in_dtype);
  if (!aligned16(g.A) || !aligned16(g.B)) return fail("operand base not 16-byte aligned");
  if ((g.lda * esz) % 16 || (g.ldb * esz) % 16) return fail("operand row pitch not a multiple of 16 bytes");
  if ((g.strideA * esz) % 16 || (g.strideB * esz) % 16) return fail("batch stride not a multiple of 16 bytes");
  if (g.strideA < 0 || g.strideB < 0) return fail("negative batch stride");
  if (!tc::driver_has_tensor_maps()) return fail("driver lacks cuTensorMapEncodeTiled");
  if (!g.epi.D) return fail("no output");
  return true;
}

namespace {
void fill_common(const GemmProblem& g, tc::TcParams& p) {
  p.M = g.M; p.N = g.N; p.K = g.K; p.batch = g.reduce_batch ? 1 : g.batch;
  p.a_bcast = (g.batch > 1 && g.strideA == 0) ? 1 : 0;
  p.b_bcast = (g.batch > 1 && g.strideB == 0) ? 1 : 0;
  p.epi = g.epi;
  p.d_vec = tensor_vec_ok(g.epi.D, g.epi.ldd, g.epi.strideD, g.epi.d_dtype);
  p.z_vec = tensor_vec_ok(g.epi.Z, g.epi.ldz, g.epi.strideZ, g.epi.z_dtype);
  p.c_vec = tensor_vec_ok(g.epi.C, g.epi.ldc, g.epi.strideC, g.epi.d_dtype);
  p.bias_vec = g.epi.bias && aligned16(g.epi.bias);
  p.status = device_status_ptr();
}
}  // namespace

cudaError_t launch_gemm_tc_dual(const GemmProblem& dx, const GemmProblem& dw, cudaStream_t s) {
  static const bool off = [] { const char* e = getenv("GE2B_DUAL_BWD"); return e && atoi(e) == 0; }();
  if (off) return cudaErrorNotSupported;
  // the pair form: both problems unbatched, same element size, the orders of a dense backward, large enough for
  // CTA pairs, plain epilogues with TMA-storable 16-byte aligned outputs
  if (dx.batch != 1 || dw.batch != 1 || dx.in_dtype != dw.in_dtype) return cudaErrorNotSupported;
  if (dx.a_mn || dx.b_mn || !dw.a_mn || !dw.b_mn) return cudaErrorNotSupported;
  if (dx.M <= 128 || dw.M <= 128 || dx.N <= 128 || dw.N <= 128) return cudaErrorNotSupported;
  if (!gemm_tc_supported(dx, nullptr) || !gemm_tc_supported(dw, nullptr)) return cudaErrorNotSupported;
  if (dx.epi.Z || dw.epi.Z || dx.epi.d_dtype != dw.epi.d_dtype) return cudaErrorNotSupported;
  TcParams p1{}, p2{};
  fill_common(dx, p1);
  fill_common(dw, p2);
  if (!p1.status || !p1.d_vec || !p2.d_vec) return cudaErrorNotSupported;
  // worth it only when the combined list quantises better than the two lists do separately
  const long long units = sm_budget() / 2 > 0 ? sm_budget() / 2 : 1;
  auto tiles = [](const GemmProblem& g) { return static_cast<long long>((g.M + 255) / 256) * ((g.N + 255) / 256); };
  auto waves = [&](long long t) { return (t + units - 1) / units; };
  if (tiles(dx) + tiles(dw) < units) return cudaErrorNotSupported;   // small problems are better off with split-K each
  if (waves(tiles(dx) + tiles(dw)) >= waves(tiles(dx)) + waves(tiles(dw))) return cudaErrorNotSupported;
  return dx.in_dtype == kF32 ? tc::launch_dual_cfg<4, false, false, true, true>(dx, p1, dw, p2, s)
                             : tc::launch_dual_cfg<2, false, false, true, true>(dx, p1, dw, p2, s);
}

cudaError_t launch_gemm_tc(const GemmProblem& g, cudaStream_t s) {
  TcParams p{};
  p.M = g.M; p.N = g.N; p.K = g.K; p.batch = g.reduce_batch ? 1 : g.batch;
  p.a_bcast = (g.batch > 1 && g.strideA == 0) ? 1 : 0;
  p.b_bcast = (g.batch > 1 && g.strideB == 0) ? 1 : 0;
  p.epi = g.epi;
  p.d_vec = tensor_vec_ok(g.epi.D, g.epi.ldd, g.epi.strideD, g.epi.d_dtype);
  p.z_vec = tensor_vec_ok(g.epi.Z, g.epi.ldz, g.epi.strideZ, g.epi.z_dtype);
  p.c_vec = tensor_vec_ok(g.epi.C, g.epi.ldc, g.epi.strideC, g.epi.d_dtype);
  p.bias_vec = g.epi.bias && aligned16(g.epi.bias);
  p.status = device_status_ptr();
  if (!p.status) return cudaErrorInvalidDevice;
  const TileChoice t = choose_tile(g);
  return g.in_dtype == kF32 ? launch_major<4>(g, p, t, s) : launch_major<2>(g, p, t, s);
}

}  // namespace ge2b
