// Operand split of the error-compensated fp32 mode: x = big + small with `big` exactly representable in TF32
// (the 13 low mantissa bits cleared) and `small` = x - big, which is exact in fp32 and below 2^-10 |x|.
// The tensor-core GEMM then forms big.big + big.small + small.big in one fp32 accumulator (see GemmProblem::A_small):
// fp32 inputs, fp32-grade results, at a third of the TF32 rate -- which replaces the cublasSgemm calls of the
// reference's backward (backends/cuda/ops/gemm/kernels/regemm_backward.cu:265-291) on the tensor cores.
#include <cuda_runtime.h>

#include "ge2_internal.hpp"

namespace ge2b {
namespace {

__device__ __forceinline__ void split1(float x, float& big, float& small) {
  big = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
  small = x - big;
}

__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ src, long long ld, float* __restrict__ big, float* __restrict__ small,
                  long long rows, long long cols, int vec) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (vec) {                                   // cols % 4 == 0, ld % 4 == 0, 16-byte aligned bases
    const long long q = cols >> 2, total = rows * q;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
      const long long r = i / q, c = (i - r * q) << 2;
      const float4 x = *reinterpret_cast<const float4*>(src + r * ld + c);
      float4 b, s;
      split1(x.x, b.x, s.x); split1(x.y, b.y, s.y); split1(x.z, b.z, s.z); split1(x.w, b.w, s.w);
      *reinterpret_cast<float4*>(big + r * cols + c) = b;
      *reinterpret_cast<float4*>(small + r * cols + c) = s;
    }
  } else {
    const long long total = rows * cols;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
      const long long r = i / cols, c = i - r * cols;
      float b, s;
      split1(src[r * ld + c], b, s);
      big[i] = b; small[i] = s;
    }
  }
}

struct SplitMulti { SplitItem it[3]; int first_block[4]; int n; };

// Several splits in one launch: block b works on a 16384-element span of one tensor.
constexpr long long kSplitSpan = 16384;
__global__ void __launch_bounds__(256) split_tf32_multi_kernel(const SplitMulti m) {
  int t = 0;
  while (t + 1 < m.n && static_cast<int>(blockIdx.x) >= m.first_block[t + 1]) ++t;
  const SplitItem it = m.it[t];
  const long long total = it.rows * it.cols;
  const long long begin = static_cast<long long>(blockIdx.x - m.first_block[t]) * kSplitSpan;
  const long long end = begin + kSplitSpan < total ? begin + kSplitSpan : total;
  const bool vec = it.cols % 4 == 0 && it.ld % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(it.src) | reinterpret_cast<uintptr_t>(it.big) |
                     reinterpret_cast<uintptr_t>(it.small)) & 15u) == 0;
  if (vec) {
    for (long long i = begin + 4ll * threadIdx.x; i < end; i += 4 * 256) {
      const long long r = i / it.cols, c = i - r * it.cols;
      const float4 x = *reinterpret_cast<const float4*>(it.src + r * it.ld + c);
      float4 b, s;
      split1(x.x, b.x, s.x); split1(x.y, b.y, s.y); split1(x.z, b.z, s.z); split1(x.w, b.w, s.w);
      *reinterpret_cast<float4*>(it.big + i) = b;
      *reinterpret_cast<float4*>(it.small + i) = s;
    }
  } else {
    for (long long i = begin + threadIdx.x; i < end; i += 256) {
      const long long r = i / it.cols, c = i - r * it.cols;
      float b, s;
      split1(it.src[r * it.ld + c], b, s);
      it.big[i] = b; it.small[i] = s;
    }
  }
}

}  // namespace

cudaError_t launch_split_tf32_multi(const SplitItem* items, int n, cudaStream_t s) {
  if (!items || n < 1 || n > 3) return cudaErrorInvalidValue;
  SplitMulti m{};
  int blocks = 0;
  for (int i = 0; i < n; ++i) {
    m.it[i] = items[i];
    m.first_block[i] = blocks;
    blocks += static_cast<int>((items[i].rows * items[i].cols + kSplitSpan - 1) / kSplitSpan);
  }
  m.first_block[n] = blocks;
  m.n = n;
  if (blocks == 0) return cudaSuccess;
  split_tf32_multi_kernel<<<blocks, 256, 0, s>>>(m);
  return cudaGetLastError();
}

cudaError_t launch_split_tf32(const float* src, long long ld_src, float* big, float* small, long long rows, long long cols,
                              cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  const bool vec = cols % 4 == 0 && ld_src % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(big) | reinterpret_cast<uintptr_t>(small)) & 15u) == 0;
  const long long work = vec ? rows * (cols >> 2) : rows * cols;
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  split_tf32_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(src, ld_src, big, small, rows, cols, vec ? 1 : 0);
  return cudaGetLastError();
}

}  // namespace ge2b
