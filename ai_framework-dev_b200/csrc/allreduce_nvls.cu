// Sum all-reduce of the dense layer's weight / bias gradients across the GPUs of one node, written for NVLink 5 /
// NVSwitch: every rank reduces ITS slice of the buffer with multimem.ld_reduce (the switch reads the slice from every
// GPU and returns the sum: in-switch reduction) and publishes the result with multimem.st (the switch writes it to
// every GPU).  Each byte crosses each GPU's links once in each direction, which is the bandwidth optimum, and the
// whole exchange is one kernel per rank.  This is the data-parallel step of the path: dW = sum_r X_r^T.gZ_r,
// db = sum_r colsum(gZ_r); the reference has no multi-GPU form of it.
//
// The buffer must be "symmetric": the same allocation size on every rank, mapped into one multicast object, with a
// small signal pad per rank that the peers can write (any allocator that can do this will do; the tests and the
// benchmark take it from torch.distributed's symmetric memory).  The kernel is handed plain addresses:
//   mc_base      multicast address of the buffer (multimem.* only)
//   sig_ptrs[r]  address, valid on THIS GPU, of rank r's signal pad
// Ranks meet twice, through the signal pads: before reading (every rank's local partial sums are complete: they
// were written by earlier kernels of the same stream) and after writing (every rank's results have landed
// everywhere).  A signal is a 32-bit word that the sender flips 0 -> 1 on the receiver and the receiver flips back
// 1 -> 0, so the pads return to all-zero after every call and the same launch can be replayed from a CUDA graph.
// Every wait is bounded (two seconds of wall time); on expiry the block records kErrWaitTimeout in the device
// status word and returns without touching the buffer again.
//
// One kernel per GPU and one rank per GPU: ranks never share a GPU (kernels that wait on each other must not).
// No TMA, no multicast LOADS into shared memory: only multimem.ld_reduce / multimem.st on global memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"

using namespace ge2b;

namespace {

constexpr int kArThreads = 512;
constexpr int kArUnroll = 4;                   // 16-byte reductions in flight per thread
constexpr int kArMaxBlocks = 64;
constexpr int kArMaxWorld = 16;
constexpr int kArExclusiveSmem = 120 * 1024;   // more than half of an SM's shared memory: one block per SM
constexpr unsigned long long kWaitNs = 2000000000ull;   // a rank that is two seconds late is not coming

struct ArSegment {
  unsigned long long offset;    // bytes from the buffer base, 16-byte aligned
  unsigned long long bytes;     // multiple of 16
  int dtype;                    // kBF16 or kF32
};

struct ArParams {
  unsigned long long mc_base;
  unsigned long long sig_ptrs[kArMaxWorld];
  int world, rank;
  ArSegment seg[2];
  int n_seg;
  int* status;
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Both polls give up after kWaitNs of wall time (checked every 64 polls).
__device__ __forceinline__ bool put_signal(uint32_t* addr) {
  unsigned long long t0 = 0;
  uint32_t seen, spins = 0;
  for (;;) {
    asm volatile("atom.global.release.sys.cas.b32 %0, [%1], 0, 1;" : "=r"(seen) : "l"(addr) : "memory");
    if (seen == 0u) return true;
    if ((++spins & 63u) == 0u) {
      const unsigned long long t = now_ns();
      if (t0 == 0) t0 = t;
      else if (t - t0 > kWaitNs) return false;
    }
  }
}

__device__ __forceinline__ bool wait_signal(uint32_t* addr) {
  unsigned long long t0 = 0;
  uint32_t seen, spins = 0;
  for (;;) {
    asm volatile("atom.global.acquire.sys.cas.b32 %0, [%1], 1, 0;" : "=r"(seen) : "l"(addr) : "memory");
    if (seen == 1u) return true;
    if ((++spins & 63u) == 0u) {
      const unsigned long long t = now_ns();
      if (t0 == 0) t0 = t;
      else if (t - t0 > kWaitNs) return false;
    }
  }
}

// All ranks' block `blockIdx.x` meet: thread p signals rank p's pad slot [block][my rank] and waits for its own
// slot [block][p].  Returns false (to every thread of the block) when a wait ran out.
__device__ __forceinline__ bool block_barrier(const ArParams& p, int* ok_smem) {
  __syncthreads();
  if (threadIdx.x == 0) *ok_smem = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    uint32_t* theirs = reinterpret_cast<uint32_t*>(p.sig_ptrs[peer]) + blockIdx.x * kArMaxWorld + p.rank;
    uint32_t* mine = reinterpret_cast<uint32_t*>(p.sig_ptrs[p.rank]) + blockIdx.x * kArMaxWorld + peer;
    bool ok = put_signal(theirs);
    ok = ok && wait_signal(mine);
    if (!ok) *ok_smem = 0;
  }
  __syncthreads();
  return *ok_smem != 0;
}

template <bool kBf16>
__device__ __forceinline__ void reduce_16(unsigned long long addr, uint32_t (&r)[4]) {
  if constexpr (kBf16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(addr) : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(addr) : "memory");
  }
}

template <bool kBf16>
__device__ __forceinline__ void publish_16(unsigned long long addr, const uint32_t (&r)[4]) {
  if constexpr (kBf16) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
  } else {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
  }
}

// This rank's share of one segment: 16-byte units [u0, u1), walked by all blocks together.
template <bool kBf16>
__device__ __forceinline__ void reduce_segment(const ArParams& p, const ArSegment& s) {
  const unsigned long long units = s.bytes >> 4;
  const unsigned long long per = (units + p.world - 1) / p.world;
  const unsigned long long u0 = per * p.rank < units ? per * p.rank : units;
  const unsigned long long u1 = u0 + per < units ? u0 + per : units;
  const unsigned long long base = p.mc_base + s.offset;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kArThreads;
  unsigned long long u = u0 + static_cast<unsigned long long>(blockIdx.x) * kArThreads + threadIdx.x;
  for (; u + (kArUnroll - 1) * stride < u1; u += kArUnroll * stride) {
    uint32_t r[kArUnroll][4];
#pragma unroll
    for (int j = 0; j < kArUnroll; ++j) reduce_16<kBf16>(base + ((u + j * stride) << 4), r[j]);
#pragma unroll
    for (int j = 0; j < kArUnroll; ++j) publish_16<kBf16>(base + ((u + j * stride) << 4), r[j]);
  }
  for (; u < u1; u += stride) {
    uint32_t r[4];
    reduce_16<kBf16>(base + (u << 4), r);
    publish_16<kBf16>(base + (u << 4), r);
  }
}

__global__ void __launch_bounds__(kArThreads) allreduce_nvls_kernel(const ArParams p) {
  __shared__ int ok_smem;
  if (!block_barrier(p, &ok_smem)) {            // every rank's partial sums are in place
    if (threadIdx.x == 0) atomicOr(p.status, kErrWaitTimeout);
    return;
  }
  for (int i = 0; i < p.n_seg; ++i) {
    if (p.seg[i].dtype == kBF16) reduce_segment<true>(p, p.seg[i]);
    else                         reduce_segment<false>(p, p.seg[i]);
  }
  __threadfence_system();                       // this thread's multimem.st are performed before it signals
  if (!block_barrier(p, &ok_smem)) {            // every rank's results have landed on every GPU
    if (threadIdx.x == 0) atomicOr(p.status, kErrWaitTimeout);
  }
}

}  // namespace

extern "C" {

int ge2b_allreduce_nvls_pad_bytes(void) { return kArMaxBlocks * kArMaxWorld * static_cast<int>(sizeof(uint32_t)); }

int ge2b_allreduce_nvls(const ge2b_allreduce_nvls_t* a, void* stream) {
  if (!a || !a->multicast_base || !a->signal_pads || a->world < 2 || a->world > kArMaxWorld || a->rank < 0 ||
      a->rank >= a->world || a->n_segments < 1 || a->n_segments > 2)
    return kBadArgs;
  ArParams p{};
  p.mc_base = reinterpret_cast<unsigned long long>(a->multicast_base);
  for (int r = 0; r < a->world; ++r) {
    if (!a->signal_pads[r]) return kBadArgs;
    p.sig_ptrs[r] = reinterpret_cast<unsigned long long>(a->signal_pads[r]);
  }
  p.world = a->world; p.rank = a->rank; p.n_seg = a->n_segments;
  unsigned long long total = 0;
  for (int i = 0; i < a->n_segments; ++i) {
    const auto& s = a->segments[i];
    if ((s.offset_bytes & 15u) || (s.bytes & 15u) || s.bytes == 0) return kBadArgs;
    if (s.dtype != GE2_DT_BF16 && s.dtype != GE2_DT_F32) return kBadArgs;
    p.seg[i].offset = s.offset_bytes; p.seg[i].bytes = s.bytes; p.seg[i].dtype = s.dtype;
    total += s.bytes;
  }
  p.status = device_status_ptr();
  if (!p.status) return kCudaError;
  int blocks = a->blocks > 0 ? a->blocks : 32;
  if (blocks > kArMaxBlocks) blocks = kArMaxBlocks;
  // small buffers: no more blocks than there are 16-byte units for
  const unsigned long long want = (total / 16 / a->world + kArThreads - 1) / kArThreads;
  if (static_cast<unsigned long long>(blocks) > want) blocks = want > 0 ? static_cast<int>(want) : 1;
  if (blocks > 1 && blocks % 2) --blocks;
  // Placement.  The exchange usually runs beside a GEMM whose CTAs come in pairs that need both SMs of a TPC.  Blocks
  // scattered one per TPC would break twice as many pairs as there are blocks, so the blocks are launched as clusters
  // of two (co-scheduled on neighbouring SMs) and each asks for enough shared memory to have its SM to itself:
  // `blocks` blocks then occupy exactly `blocks` SMs of blocks / 2 TPCs, whichever kernel is scheduled first.
  static cudaError_t attr_err = cudaFuncSetAttribute(allreduce_nvls_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     kArExclusiveSmem);
  if (attr_err != cudaSuccess) return kCudaError;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
  cfg.blockDim = dim3(kArThreads, 1, 1);
  cfg.dynamicSmemBytes = kArExclusiveSmem;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (blocks % 2 == 0) ? 2u : 1u;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel, p) == cudaSuccess ? kOk : kCudaError;
}

}  // extern "C"
