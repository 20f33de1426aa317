// Internal parameter blocks shared by the host launch layer and the CUDA kernels of the
// dense-layer path  D = act(alpha * A.B + beta * C + bias)  and its backward.
//
// Numbering of ActKind / BiasKind / DType follows the reference's ABI-anchored enums
// (backends/cuda/ops/_common/shim/enums.hpp:10-24, ai_device.hpp:14-16) so that values
// can be passed through unchanged from the operator API.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

// Profiler ranges with the reference's names ("gemm.fwd", "gemm.bwd", "bwd.epilogue", "bwd.gemms":
// backends/cuda/ops/gemm/launcher.cu:154,287, kernels/regemm_backward.cu:201,262), compiled in under the reference's
// own switch AI_USE_NVTX (backends/cuda/ops/_common/shim/ai_nvtx.hpp:8-16).  Header-only NVTX: without a profiler
// attached a range costs a few nanoseconds.
#if defined(AI_USE_NVTX) || defined(USE_NVTX) || defined(AI_ENABLE_NVTX)
#include <nvtx3/nvToolsExt.h>
namespace ge2b {
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};
}  // namespace ge2b
#else
namespace ge2b {
struct NvtxRange { explicit NvtxRange(const char*) {} };
}  // namespace ge2b
#endif

namespace ge2b {

enum : int { kActNone = 0, kActReLU = 1, kActLeaky = 2, kActGELU = 3, kActSigmoid = 4, kActTanh = 5 };
enum : int { kBiasNone = 0, kBiasScalar = 1, kBiasPerM = 2, kBiasPerN = 3 };
enum : int { kF32 = 0, kF16 = 1, kBF16 = 2 };

// Error bits written by device code into the per-device status word (never cleared by kernels).
enum : int {
  kErrWaitTimeout = 1,   // a bounded mbarrier wait ran out
  kErrAborted     = 2    // a role left its loop because another role timed out
};

__host__ __device__ inline int dtype_bytes(int dt) { return dt == kF32 ? 4 : 2; }

// The second half of a deterministic per-column bias gradient: out[c] = sum over row blocks (ascending) of
// partial[block * pitch + c].  It rides along with the GEMM launch that follows the prologue (idle lanes of the
// producer warp do it while the tensor pipe works) or, where no such launch follows, runs as a small kernel.
struct DbFinish {
  const float* partial = nullptr; long long pitch = 0; int blocks = 0;
  float* out = nullptr; int n = 0;
};

// Everything the fused epilogue needs.  Pointers may be null where stated.
struct EpilogueArgs {
  void*        D;    long long ldd, strideD;      // output, row-major [M,N] per batch slice
  void*        Z;    long long ldz, strideZ;      // pre-activation stash (null = not saved)
  const void*  C;    long long ldc, strideC;      // addend scaled by beta (null = none)
  const float* bias;                              // always fp32 (null = none)
  int   bias_kind;                                // kBias*
  int   act;                                      // kAct*
  float leaky;
  float alpha, beta;
  int   d_dtype;                                  // dtype of D and C
  int   z_dtype;                                  // dtype of Z
};

// One (optionally strided-batched) GEMM  D[b] = epi(A[b] (M x K) . B[b] (K x N)).
//   a_mn == false : A is stored with the reduction index contiguous  (memory rows = M,  row length K)
//   a_mn == true  : A is stored with the M index contiguous          (memory rows = K,  row length M)
//   b_mn == false : B is stored with the reduction index contiguous  (memory rows = N,  row length K)
//   b_mn == true  : B is stored with the N index contiguous          (memory rows = K,  row length N)
// Strides are in elements; a batch stride of 0 broadcasts the operand to every slice.
struct GemmProblem {
  int M, N, K, batch;
  int in_dtype;                                   // kBF16 / kF16 / kF32
  int math;                                       // for kF32: 0 = exact fp32 FMA, 1 = TF32 tensor cores,
                                                  // 2 = error-compensated TF32 (three products of split operands)
  bool a_mn, b_mn;
  const void* A; long long lda, strideA;
  const void* B; long long ldb, strideB;
  EpilogueArgs epi;
  // math == 2: A and B hold the TF32-representable "big" parts of the fp32 operands and these the remainders
  // (operand = big + small exactly), same geometry.  The launch computes big.big + big.small + small.big in one fp32
  // accumulator: every product is exact in TF32 arithmetic and only small.small (2^-22 relative) is dropped.
  const void* A_small = nullptr;
  const void* B_small = nullptr;
  DbFinish db;                                    // tensor-core path only: bias-gradient finish carried by this launch
  // The batch index joins the reduction: D = act(alpha * sum_b A[b].B[b] + ...), one output matrix.  Tensor-core
  // path only (used by the convolution's weight gradient, which sums over the images of a batch).
  bool reduce_batch = false;
};

// gZ = gY * act'(Z) with the column/row/total reduction into gBias.
struct BwdPrologueArgs {
  int M, N;
  const void* gY; long long ldgY; int gy_dtype;
  const void* Z;  long long ldZ;  int z_dtype;
  void* gZ; long long ldgZ; int gz_dtype;         // scratch that the two backward GEMMs read
  void* gC; long long ldgC; int gc_dtype; float beta;   // optional gC = beta * gZ
  float* gBias; int bias_kind;                    // fp32, zeroed by the launcher before the kernel
  int act; float leaky;
  // Per-column bias gradient without atomics (filled in by launch_bwd_prologue when stream scratch is to be had):
  // every CTA leaves the column sums of its rows in db_partial[row block][column]; the row blocks are added in a
  // fixed order afterwards (see DbFinish).  Null: fp32 atomics.
  float* db_partial = nullptr; long long db_pitch = 0;
};


// ---- launchers (each returns cudaSuccess or the launch error) ----
cudaError_t launch_gemm_simt(const GemmProblem& g, cudaStream_t s);      // exact fp32-accumulate FMA path (any dtype, any ld)
bool        gemm_tc_supported(const GemmProblem& g, const char** why);   // alignment / dtype rules of the TMA + tcgen05 path
cudaError_t launch_gemm_tc(const GemmProblem& g, cudaStream_t s);        // TMA + tcgen05 + TMEM path
// dX = gZ.W^T and dW = X^T.gZ of one dense layer as ONE persistent launch (their tiles form one list, so only the
// combined list's last wave is partly filled).  Returns cudaErrorNotSupported when the pair does not qualify; the
// caller then launches the two problems one after the other.
cudaError_t launch_gemm_tc_dual(const GemmProblem& dx, const GemmProblem& dw, cudaStream_t s);
// `pending` (may be null): receives the finish of a deterministic per-column bias gradient that the caller must
// attach to the next tensor-core GEMM launch on the stream or run with launch_db_finish; without it (or when no
// scratch is to be had) the kernel adds with atomics and nothing is pending.
// zero_gbias: the launcher zeroes gBias on the stream first where the kernel adds into it with atomics (it does not
// when the deterministic form overwrites it).
cudaError_t launch_bwd_prologue(const BwdPrologueArgs& a, cudaStream_t s, DbFinish* pending = nullptr,
                                bool zero_gbias = false);
cudaError_t launch_db_finish(const DbFinish& f, cudaStream_t s);
// big = src with the 13 low mantissa bits cleared (exactly representable in TF32), small = src - big (exact in fp32);
// src is rows x cols with pitch ld_src, big and small are written with pitch cols.
cudaError_t launch_split_tf32(const float* src, long long ld_src, float* big, float* small, long long rows, long long cols,
                              cudaStream_t s);
// up to three such splits in one launch (a backward splits gZ, W and X)
struct SplitItem { const float* src; long long ld; float* big; float* small; long long rows, cols; };
cudaError_t launch_split_tf32_multi(const SplitItem* items, int n, cudaStream_t s);

// Reads (and optionally clears) the device status word of the current device. Synchronises.
int  device_status_word(bool clear);
int* device_status_ptr();   // device address of the status word for the current device

// Device memory a caller lends to the launch layer for the duration of one call on this thread (split-K partial tiles
// and arrival counters are placed in it).  `no_alloc`: the launch layer must not create scratch of its own during the
// call; what does not fit the lent memory runs unsplit.  Set through ScopedLease.
struct ScratchLease { void* base = nullptr; size_t bytes = 0; bool no_alloc = false; };
ScratchLease& scratch_lease();                       // thread-local
struct ScopedLease {
  ScratchLease saved;
  ScopedLease(void* base, size_t bytes, bool no_alloc) : saved(scratch_lease()) {
    // the launch layer wants a 256-byte aligned base
    uintptr_t a = reinterpret_cast<uintptr_t>(base);
    const uintptr_t up = (a + 255u) & ~static_cast<uintptr_t>(255u);
    if (base && bytes > up - a) { scratch_lease().base = reinterpret_cast<void*>(up); scratch_lease().bytes = bytes - (up - a); }
    else { scratch_lease().base = nullptr; scratch_lease().bytes = 0; }
    scratch_lease().no_alloc = no_alloc;
  }
  ~ScopedLease() { scratch_lease() = saved; }
  ScopedLease(const ScopedLease&) = delete;
  ScopedLease& operator=(const ScopedLease&) = delete;
};
// The calling thread's scratch for launches on stream `s` (lent memory first, else the library's per-stream buffer;
// see split_scratch in gemm_tc.cu).  `flags` are zero and every user leaves them zero, unless `*lent`.
bool borrow_stream_scratch(cudaStream_t s, float** ws, size_t* ws_bytes, int** flags, size_t* flag_bytes, bool* lent);
long long split_unavailable_total();   // split-K launches that ran unsplit because no scratch could be had (capture, no_alloc)
void release_library_scratch();        // synchronises the device and frees every split-K scratch the library created
std::atomic<unsigned long long>& plan_cache_generation();   // bumping it invalidates every thread's cached launches

bool early_start_enabled(); // programmatic dependent launch for the GEMM and prologue kernels (GE2B_PDL=1: on)
int  sm_count();            // cached multiprocessor count of the current device
int  sm_budget();           // SMs the persistent GEMM may occupy: sm_count() unless lowered by set_sm_limit()
void keep_async_pool_cached();   // call before cudaMallocAsync: the default pool then keeps freed scratch for reuse
void set_sm_limit(int n);   // n <= 0 restores "all SMs"; process-wide

}  // namespace ge2b
