// Small per-device runtime state of the launch layer: the device status word that bounded waits
// report into, and the cached multiprocessor count used to size persistent grids.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "ge2_internal.hpp"

namespace ge2b {
namespace {

__device__ int g_status_word = 0;

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int* g_status_addr[kMaxDevices] = {};
int  g_sm_count[kMaxDevices]    = {};

int current_device() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return -1;
  return d;
}

}  // namespace

int* device_status_ptr() {
  const int d = current_device();
  if (d < 0) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_addr[d]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status_addr[d] = static_cast<int*>(p);
  }
  return g_status_addr[d];
}

int device_status_word(bool clear) {
  int* p = device_status_ptr();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (clear && v != 0) {
    const int zero = 0;
    cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

int sm_count() {
  const int d = current_device();
  if (d < 0) return 1;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_sm_count[d] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 1;
    g_sm_count[d] = n;
  }
  return g_sm_count[d];
}

namespace {
std::atomic<int> g_sm_limit{0};
}

void set_sm_limit(int n) { g_sm_limit.store(n > 0 ? n : 0, std::memory_order_relaxed); }

// Stream-ordered scratch (cudaMallocAsync) comes from the device's default memory pool, which by default hands its
// memory back to the driver at every synchronisation; a step that allocates the same scratch again and again would
// pay for fresh physical memory each time.  Raising the pool's release threshold (once per device) keeps it cached.
void keep_async_pool_cached() {
  static bool done[kMaxDevices] = {};
  const int d = current_device();
  if (d < 0 || d >= kMaxDevices || done[d]) return;
  done[d] = true;
  cudaMemPool_t pool = nullptr;
  if (cudaDeviceGetDefaultMemPool(&pool, d) != cudaSuccess || !pool) { cudaGetLastError(); return; }
  unsigned long long keep = ~0ull;
  if (cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) cudaGetLastError();
}

int sm_budget() {
  const int all = sm_count();
  const int lim = g_sm_limit.load(std::memory_order_relaxed);
  return (lim > 0 && lim < all) ? lim : all;
}

}  // namespace ge2b
