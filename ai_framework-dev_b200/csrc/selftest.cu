// Self-test of the bounded wait every role of the tensor-core GEMM relies on (ptx::mbar_wait): a one-warp kernel
// initialises an mbarrier that nothing will ever arrive at, waits on it with a small clock budget, and reports what
// the wait returned.  The wait must give up, set the CTA's abort flag and the kernel must OR kErrWaitTimeout into the
// device status word -- the path a stuck pipeline takes -- and return normally: no trap, no TMA or TMEM in flight, the
// context stays usable.
#include <cuda_runtime.h>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"
#include "sm100_ptx.cuh"

using namespace ge2b;

namespace {

__global__ void __launch_bounds__(32) wait_expiry_kernel(long long budget_cycles, int* status, int* report) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(bar_addr, 1);
    ptx::fence_barrier_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = ptx::mbar_wait(bar_addr, 0u, &abort_flag, budget_cycles);   // phase 0 never completes
    const long long waited = clock64() - t0;
    report[0] = ok ? 1 : 0;
    report[1] = abort_flag;
    report[2] = static_cast<int>(waited > 0x7fffffffll ? 0x7fffffffll : waited);
    if (!ok) atomicOr(status, kErrWaitTimeout);
  }
  __syncwarp();
  // a second waiter sees the abort flag the first one set and leaves at once
  if (threadIdx.x == 1) report[3] = ptx::mbar_wait(bar_addr, 0u, &abort_flag, budget_cycles) ? 1 : 0;
}

}  // namespace

extern "C" int ge2b_selftest_wait_expiry(long long budget_cycles, int* report4, void* stream) {
  if (budget_cycles <= 0 || budget_cycles > 200000000ll || !report4) return kBadArgs;   // at most about 0.1 s
  int* status = device_status_ptr();
  if (!status) return kCudaError;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int* d_report = nullptr;
  if (cudaMallocAsync(reinterpret_cast<void**>(&d_report), 4 * sizeof(int), s) != cudaSuccess) return kCudaError;
  cudaMemsetAsync(d_report, 0xff, 4 * sizeof(int), s);
  wait_expiry_kernel<<<1, 32, 0, s>>>(budget_cycles, status, d_report);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyAsync(report4, d_report, 4 * sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFreeAsync(d_report, s);
  return e == cudaSuccess ? kOk : kCudaError;
}
