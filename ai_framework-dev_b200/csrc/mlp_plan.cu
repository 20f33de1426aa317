// The captured training-step driver around the dense layers, in C++ behind a C ABI: a stack of Dense layers ->
// softmax cross-entropy (mean) -> SGD on fp32 master weights, with pointer-stable buffers allocated once, the step
// warmed up, captured into a CUDA graph and replayed.
//
// What it restates, for this path only, from the reference's Python graph runtime:
//   * graph/capture_plan.py:250-287  one pre-allocated y, z, gA, gW, gB and gZ work buffer per Dense layer
//   * graph/runtime.py:24-148        forward layer by layer -> loss -> backward from the last layer to the first
//                                    (dX is computed for the first layer too) -> optimizer, all on one stream
//   * graph/graph_exec.py:51-231     warm-up outside capture, capture, instantiate, replay
//   * layers/sequential.py:416-497   compile() / one_step()
// and adds what the reference does not have: a batch sharded along M over several GPUs, each layer's dW and db summed
// across them on a side stream as soon as they are written (under the dX GEMM and the backward of the layers below),
// either by this library's NVLink kernel over caller-provided symmetric memory or by the collective library (loaded
// at run time; the plan builds its own communicator from a unique id the caller distributes).
// No PyTorch, no Python: buffers are cudaMalloc'ed here, the caller hands over host or device pointers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <new>
#include <vector>

#include "../../include/ge2_b200.h"
#include "dense_ops.hpp"

using namespace ge2b;

extern "C" int ge2_launch_softmax_ce_fused(const ge2_uintptr* bufs, int n, void* stream);

namespace ge2b {
int launch_sgd_multi(const SgdTensor* t, int n, float lr, cudaStream_t s);   // train_step.cu
}

namespace {

constexpr int kMaxLayers = GE2B_MLP_MAX_LAYERS;
constexpr size_t kAlign = 256;
size_t round_up(size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

// ---- the collective library, bound at run time (no link dependency; single-GPU users never load it) ----
struct NcclApi {
  using comm_t = void*;
  struct unique_id { char internal[128]; };
  int (*GetUniqueId)(unique_id*) = nullptr;
  int (*CommInitRank)(comm_t*, int, unique_id, int) = nullptr;
  int (*CommDestroy)(comm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, comm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  bool ok = false;
};
constexpr int kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclFloat16 = 6, kNcclSum = 0;   // public enum values of nccl.h

NcclApi& nccl() {
  static NcclApi api = [] {
    NcclApi a;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return a;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(dlsym(h, "ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(dlsym(h, "ncclGroupEnd"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.GroupStart && a.GroupEnd;
    return a;
  }();
  return api;
}

struct Layer {
  int in = 0, out = 0, act = 0;
  float* W32 = nullptr;      // [in, out] fp32 master
  void* W = nullptr;         // [in, out] in the compute dtype (the fp32 master itself when dtype is fp32)
  float* b = nullptr;        // [out]
  void *y = nullptr, *z = nullptr, *work = nullptr, *gA = nullptr;
  void* gW = nullptr;        // inside the gradient buffer
  float* gB = nullptr;       // inside the gradient buffer
  size_t gw_off = 0, gb_off = 0, end_off = 0;
};

}  // namespace

struct ge2b_mlp_plan {
  ge2b_mlp_config_t cfg;
  int n = 0, esz = 2;
  std::vector<Layer> L;
  void* X = nullptr;
  int* labels = nullptr;
  void* dlogits = nullptr;
  float* loss = nullptr;
  unsigned char* grads = nullptr;       // gradient buffer (own allocation, or the caller's symmetric one)
  bool own_grads = false;
  size_t grad_data_bytes = 0;
  std::vector<void*> pads;              // exchange 1: every rank's signal pad as mapped here
  void* nccl_comm = nullptr;            // exchange 2
  cudaStream_t s_main = nullptr, s_comm = nullptr;
  cudaEvent_t ev_layer[kMaxLayers] = {}, ev_join = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  std::vector<void*> owned;             // every cudaMalloc of the plan
  long long launches_per_step = 0;
};

namespace {

bool ok(cudaError_t e) { return e == cudaSuccess; }

size_t grad_layout(const ge2b_mlp_config_t& c, std::vector<Layer>* L) {
  const size_t esz = dtype_bytes(c.dtype);
  size_t off = 0;
  for (int i = 0; i < c.n_layers; ++i) {
    const size_t gw = static_cast<size_t>(c.dims[i]) * c.dims[i + 1] * esz, gb = static_cast<size_t>(c.dims[i + 1]) * 4;
    if (L) { (*L)[i].gw_off = off; }
    off = round_up(off + gw);
    if (L) { (*L)[i].gb_off = off; }
    off = round_up(off + gb);
    if (L) { (*L)[i].end_off = off; }
  }
  return off;
}

bool config_ok(const ge2b_mlp_config_t* c) {
  if (!c || c->n_layers < 1 || c->n_layers > kMaxLayers || c->batch < 1) return false;
  if (c->dtype != GE2_DT_F32 && c->dtype != GE2_DT_F16 && c->dtype != GE2_DT_BF16) return false;
  for (int i = 0; i <= c->n_layers; ++i)
    if (c->dims[i] < 1) return false;
  for (int i = 0; i < c->n_layers; ++i)
    if (c->acts[i] < 0 || c->acts[i] > 5) return false;
  if (c->world < 1 || c->rank < 0 || c->rank >= (c->world > 0 ? c->world : 1)) return false;
  if (c->world > 1 && (c->exchange < 1 || c->exchange > 2)) return false;
  if (c->world > 1 && c->exchange == 1 && (c->dtype == GE2_DT_F16 || !c->grad_base || !c->grad_multicast || !c->peer_grad_bases))
    return false;                        // the NVLink kernel sums bf16 and fp32
  if (c->world > 1 && c->exchange == 2 && !c->nccl_unique_id) return false;
  return c->lr > 0.f;
}

void* dmalloc(ge2b_mlp_plan* p, size_t bytes) {
  void* q = nullptr;
  if (!ok(cudaMalloc(&q, bytes ? bytes : 16))) return nullptr;
  p->owned.push_back(q);
  return q;
}

int exchange_layer(ge2b_mlp_plan* p, int i, cudaStream_t s) {
  const Layer& l = p->L[i];
  if (p->cfg.exchange == 1) {
    ge2b_allreduce_nvls_t a{};
    a.multicast_base = p->cfg.grad_multicast;
    a.signal_pads = p->pads.data();
    a.world = p->cfg.world; a.rank = p->cfg.rank;
    a.n_segments = 2;
    a.segments[0].offset_bytes = l.gw_off; a.segments[0].bytes = l.gb_off - l.gw_off; a.segments[0].dtype = static_cast<ge2_dtype_t>(p->cfg.dtype);
    a.segments[1].offset_bytes = l.gb_off; a.segments[1].bytes = l.end_off - l.gb_off; a.segments[1].dtype = GE2_DT_F32;
    a.blocks = p->cfg.comm_blocks;
    return ge2b_allreduce_nvls(&a, s);
  }
  NcclApi& api = nccl();
  const int dt = p->cfg.dtype == GE2_DT_F32 ? kNcclFloat32 : (p->cfg.dtype == GE2_DT_BF16 ? kNcclBfloat16 : kNcclFloat16);
  // one group: the two tensors of a layer travel as one fused operation
  if (api.GroupStart() != 0) return kCudaError;
  int rc = api.AllReduce(l.gW, l.gW, static_cast<size_t>(l.in) * l.out, dt, kNcclSum, p->nccl_comm, s);
  rc |= api.AllReduce(l.gB, l.gB, static_cast<size_t>(l.out), kNcclFloat32, kNcclSum, p->nccl_comm, s);
  rc |= api.GroupEnd();
  return rc == 0 ? kOk : kCudaError;
}

// One training step on s_main (the exchange on s_comm, forked and joined by events, so that the whole step can be
// captured as one graph).
int run_step(ge2b_mlp_plan* p) {
  const int n = p->n, B = p->cfg.batch, dt = p->cfg.dtype;
  cudaStream_t s = p->s_main;
  const long long l0 = launches_total();
  const void* cur = p->X;
  for (int i = 0; i < n; ++i) {
    Layer& l = p->L[i];
    DenseForward f;
    f.M = B; f.K = l.in; f.N = l.out;
    f.dtype = dt; f.z_dtype = dt; f.math = dt == kF32 ? default_fp32_math() : 1;
    f.A = cur; f.lda = l.in; f.B = l.W; f.ldb = l.out; f.D = l.y; f.ldd = l.out; f.Z = l.z; f.ldz = l.out;
    f.bias = l.b; f.bias_kind = kBiasPerN; f.act = l.act;
    const int rc = dense_forward(f, s);
    if (rc != kOk) return rc;
    cur = l.y;
  }
  {
    ge2_softmax_ce_params_t q{};
    q.M = B; q.C = p->cfg.dims[n];
    q.dtype = static_cast<ge2_dtype_t>(dt); q.grad_dtype = static_cast<ge2_dtype_t>(dt);
    q.reduction = 1; q.ignore_index = -1;
    const int gb = p->cfg.global_batch > 0 ? p->cfg.global_batch : B;
    q.grad_scale = 1.f / static_cast<float>(gb);      // mean over the GLOBAL batch: the replicas' gradients add up
    q.mean_denominator = gb;
    ge2_uintptr bufs[5] = {reinterpret_cast<ge2_uintptr>(p->L[n - 1].y), reinterpret_cast<ge2_uintptr>(p->labels),
                           reinterpret_cast<ge2_uintptr>(p->dlogits), reinterpret_cast<ge2_uintptr>(p->loss),
                           reinterpret_cast<ge2_uintptr>(&q)};
    const int rc = ge2_launch_softmax_ce_fused(bufs, 5, s);
    if (rc != kOk) return rc;
  }
  const void* g = p->dlogits;
  const bool dp = p->cfg.world > 1;
  struct LimitGuard { bool on; ~LimitGuard() { if (on) set_sm_limit(0); } } guard{dp};   // also on the error returns
  for (int i = n - 1; i >= 0; --i) {
    Layer& l = p->L[i];
    DenseBackward b;
    b.M = B; b.K = l.in; b.N = l.out;
    b.dtype = dt; b.z_dtype = dt; b.math = dt == kF32 ? default_fp32_math() : 1;
    b.A = i == 0 ? p->X : p->L[i - 1].y; b.lda = l.in;
    b.B = l.W; b.ldb = l.out;
    b.gY = g; b.ldgY = l.out; b.Z = l.z; b.ldZ = l.out;
    b.act = l.act;
    b.scratch = l.work; b.scratch_bytes = static_cast<size_t>(B) * l.out * p->esz;
    b.gB = l.gW; b.ldgB = l.out; b.gBias = l.gB; b.bias_kind = kBiasPerN;
    if (!dp) {                              // one call: prologue, then dX and dW (one launch when that fills the machine better)
      b.gA = l.gA; b.ldgA = l.in;
      const int rc = dense_backward(b, s);
      if (rc != kOk) return rc;
    } else {                                // gZ, db and dW first, so that their exchange starts before dX is computed
      int rc = dense_backward(b, s);
      if (rc != kOk) return rc;
      if (!ok(cudaEventRecord(p->ev_layer[i], s)) || !ok(cudaStreamWaitEvent(p->s_comm, p->ev_layer[i], 0))) return kCudaError;
      rc = exchange_layer(p, i, p->s_comm);
      if (rc != kOk) return rc;
      // from here to the join an exchange may be running beside the GEMMs: they leave it its SMs (a persistent grid
      // that wanted every SM would have to wait for the exchange kernel's blocks to finish)
      set_sm_limit(sm_count() - (p->cfg.comm_blocks > 0 ? p->cfg.comm_blocks : 16));
      b.gB = nullptr; b.gBias = nullptr; b.bias_kind = kBiasNone;
      b.gA = l.gA; b.ldgA = l.in; b.reuse_gz = true;
      rc = dense_backward(b, s);
      if (rc != kOk) return rc;
    }
    g = l.gA;
  }
  if (dp) set_sm_limit(0);
  if (dp && (!ok(cudaEventRecord(p->ev_join, p->s_comm)) || !ok(cudaStreamWaitEvent(s, p->ev_join, 0)))) return kCudaError;
  SgdTensor t[2 * kMaxLayers];
  for (int i = 0; i < n; ++i) {
    Layer& l = p->L[i];
    t[2 * i] = SgdTensor{l.W32, l.gW, dt == kF32 ? nullptr : l.W, static_cast<long long>(l.in) * l.out, dt, dt};
    t[2 * i + 1] = SgdTensor{l.b, l.gB, nullptr, static_cast<long long>(l.out), kF32, kF32};
  }
  const int rc = launch_sgd_multi(t, 2 * n, p->cfg.lr, s);
  p->launches_per_step = launches_total() - l0 + 2 + (dp ? n : 0);   // + loss, optimizer and exchange kernels
  return rc;
}

void destroy(ge2b_mlp_plan* p) {
  if (!p) return;
  if (p->s_main) cudaStreamSynchronize(p->s_main);
  if (p->s_comm) cudaStreamSynchronize(p->s_comm);
  if (p->exec) cudaGraphExecDestroy(p->exec);
  if (p->graph) cudaGraphDestroy(p->graph);
  if (p->nccl_comm && nccl().ok) nccl().CommDestroy(p->nccl_comm);
  for (void* q : p->owned) cudaFree(q);
  for (int i = 0; i < kMaxLayers; ++i)
    if (p->ev_layer[i]) cudaEventDestroy(p->ev_layer[i]);
  if (p->ev_join) cudaEventDestroy(p->ev_join);
  if (p->s_main) cudaStreamDestroy(p->s_main);
  if (p->s_comm) cudaStreamDestroy(p->s_comm);
  delete p;
}

}  // namespace

extern "C" {

size_t ge2b_mlp_plan_grad_bytes(const ge2b_mlp_config_t* c) {
  if (!c || c->n_layers < 1 || c->n_layers > kMaxLayers) return 0;
  return grad_layout(*c, nullptr) + static_cast<size_t>(ge2b_allreduce_nvls_pad_bytes());
}

int ge2b_nccl_unique_id(void* id128) {
  if (!id128 || !nccl().ok) return kCudaError;
  NcclApi::unique_id id;
  if (nccl().GetUniqueId(&id) != 0) return kCudaError;
  std::memcpy(id128, id.internal, 128);
  return kOk;
}

int ge2b_mlp_plan_create(ge2b_mlp_plan** out, const ge2b_mlp_config_t* c) {
  if (!out || !config_ok(c)) return kBadArgs;
  ge2b_mlp_plan* p = new (std::nothrow) ge2b_mlp_plan();
  if (!p) return kCudaError;
  p->cfg = *c;
  if (p->cfg.world < 1) p->cfg.world = 1;
  p->n = c->n_layers;
  p->esz = dtype_bytes(c->dtype);
  p->L.resize(p->n);
  const size_t B = static_cast<size_t>(c->batch);
  bool good = ok(cudaStreamCreateWithFlags(&p->s_main, cudaStreamNonBlocking)) &&
              ok(cudaStreamCreateWithFlags(&p->s_comm, cudaStreamNonBlocking)) &&
              ok(cudaEventCreateWithFlags(&p->ev_join, cudaEventDisableTiming));
  for (int i = 0; good && i < p->n; ++i) good = ok(cudaEventCreateWithFlags(&p->ev_layer[i], cudaEventDisableTiming));
  p->grad_data_bytes = grad_layout(*c, &p->L);
  if (good && c->world > 1 && c->exchange == 1) {
    p->grads = static_cast<unsigned char*>(c->grad_base);
    for (int r = 0; r < c->world; ++r) {
      if (!c->peer_grad_bases[r]) { good = false; break; }
      p->pads.push_back(static_cast<unsigned char*>(c->peer_grad_bases[r]) + p->grad_data_bytes);
    }
  } else if (good) {
    p->grads = static_cast<unsigned char*>(dmalloc(p, p->grad_data_bytes));
    p->own_grads = true;
    good = p->grads != nullptr && ok(cudaMemset(p->grads, 0, p->grad_data_bytes));
  }
  if (good && c->world > 1 && c->exchange == 2) {
    NcclApi& api = nccl();
    NcclApi::unique_id id;
    std::memcpy(id.internal, c->nccl_unique_id, 128);
    good = api.ok && api.CommInitRank(&p->nccl_comm, c->world, id, c->rank) == 0;
  }
  p->X = good ? dmalloc(p, B * c->dims[0] * p->esz) : nullptr;
  p->labels = good ? static_cast<int*>(dmalloc(p, B * sizeof(int))) : nullptr;
  p->dlogits = good ? dmalloc(p, B * c->dims[p->n] * p->esz) : nullptr;
  p->loss = good ? static_cast<float*>(dmalloc(p, sizeof(float))) : nullptr;
  good = good && p->X && p->labels && p->dlogits && p->loss && ok(cudaMemset(p->X, 0, B * c->dims[0] * p->esz)) &&
         ok(cudaMemset(p->labels, 0, B * sizeof(int))) && ok(cudaMemset(p->loss, 0, sizeof(float)));
  for (int i = 0; good && i < p->n; ++i) {
    Layer& l = p->L[i];
    l.in = c->dims[i]; l.out = c->dims[i + 1]; l.act = c->acts[i];
    const size_t w = static_cast<size_t>(l.in) * l.out, a = B * l.out;
    l.W32 = static_cast<float*>(dmalloc(p, w * 4));
    l.W = c->dtype == GE2_DT_F32 ? l.W32 : dmalloc(p, w * p->esz);
    l.b = static_cast<float*>(dmalloc(p, static_cast<size_t>(l.out) * 4));
    l.y = dmalloc(p, a * p->esz); l.z = dmalloc(p, a * p->esz); l.work = dmalloc(p, a * p->esz);
    l.gA = dmalloc(p, B * l.in * p->esz);
    l.gW = p->grads + l.gw_off;
    l.gB = reinterpret_cast<float*>(p->grads + l.gb_off);
    good = l.W32 && l.W && l.b && l.y && l.z && l.work && l.gA && ok(cudaMemset(l.W32, 0, w * 4)) &&
           ok(cudaMemset(l.b, 0, static_cast<size_t>(l.out) * 4)) && (c->dtype == GE2_DT_F32 || ok(cudaMemset(l.W, 0, w * p->esz)));
  }
  if (!good) { cudaGetLastError(); destroy(p); return kCudaError; }
  *out = p;
  return kOk;
}

void ge2b_mlp_plan_destroy(ge2b_mlp_plan* p) { destroy(p); }

// fp32 host arrays in: W [in, out] row-major, b [out] (either may be null = leave as is).  Also writes the
// compute-dtype copy of W that the forward pass reads.
int ge2b_mlp_plan_set_params(ge2b_mlp_plan* p, int layer, const float* W, const float* b) {
  if (!p || layer < 0 || layer >= p->n) return kBadArgs;
  Layer& l = p->L[layer];
  const size_t w = static_cast<size_t>(l.in) * l.out;
  if (W) {
    if (!ok(cudaMemcpyAsync(l.W32, W, w * 4, cudaMemcpyHostToDevice, p->s_main))) return kCudaError;
    if (p->cfg.dtype != GE2_DT_F32) {
      // lr = 0 update against any finite gradient: rounds the master into the low-precision copy
      if (!ok(cudaMemsetAsync(l.gW, 0, w * p->esz, p->s_main))) return kCudaError;
      SgdTensor t{l.W32, l.gW, l.W, static_cast<long long>(w), p->cfg.dtype, p->cfg.dtype};
      if (launch_sgd_multi(&t, 1, 0.f, p->s_main) != kOk) return kCudaError;
    }
  }
  if (b && !ok(cudaMemcpyAsync(l.b, b, static_cast<size_t>(l.out) * 4, cudaMemcpyHostToDevice, p->s_main))) return kCudaError;
  return ok(cudaStreamSynchronize(p->s_main)) ? kOk : kCudaError;
}

int ge2b_mlp_plan_get_params(ge2b_mlp_plan* p, int layer, float* W, float* b, void* W_low) {
  if (!p || layer < 0 || layer >= p->n) return kBadArgs;
  Layer& l = p->L[layer];
  const size_t w = static_cast<size_t>(l.in) * l.out;
  bool good = ok(cudaStreamSynchronize(p->s_main));
  if (W) good = good && ok(cudaMemcpy(W, l.W32, w * 4, cudaMemcpyDeviceToHost));
  if (b) good = good && ok(cudaMemcpy(b, l.b, static_cast<size_t>(l.out) * 4, cudaMemcpyDeviceToHost));
  if (W_low) good = good && ok(cudaMemcpy(W_low, l.W, w * p->esz, cudaMemcpyDeviceToHost));
  return good ? kOk : kCudaError;
}

// Gradients as the last step left them (after the exchange): gW in the compute dtype, gb fp32.
int ge2b_mlp_plan_get_grads(ge2b_mlp_plan* p, int layer, void* gW, float* gb) {
  if (!p || layer < 0 || layer >= p->n) return kBadArgs;
  Layer& l = p->L[layer];
  bool good = ok(cudaStreamSynchronize(p->s_main));
  if (gW) good = good && ok(cudaMemcpy(gW, l.gW, static_cast<size_t>(l.in) * l.out * p->esz, cudaMemcpyDeviceToHost));
  if (gb) good = good && ok(cudaMemcpy(gb, l.gB, static_cast<size_t>(l.out) * 4, cudaMemcpyDeviceToHost));
  return good ? kOk : kCudaError;
}

// Warm-up (the step runs twice eagerly on the plan's stream: function attributes, per-stream scratch, communicator
// channels), with the parameters saved and put back so that training starts from the weights that were set; then,
// with `capture`, the step is captured into a graph and instantiated.
int ge2b_mlp_plan_compile(ge2b_mlp_plan* p, int capture) {
  if (!p) return kBadArgs;
  std::vector<void*> backup;
  std::vector<std::pair<void*, size_t>> live;
  for (Layer& l : p->L) {
    const size_t w = static_cast<size_t>(l.in) * l.out;
    live.push_back({l.W32, w * 4});
    if (l.W != l.W32) live.push_back({l.W, w * p->esz});
    live.push_back({l.b, static_cast<size_t>(l.out) * 4});
  }
  bool good = true;
  for (auto& kv : live) {
    void* q = nullptr;
    good = good && ok(cudaMalloc(&q, kv.second)) && ok(cudaMemcpyAsync(q, kv.first, kv.second, cudaMemcpyDeviceToDevice, p->s_main));
    backup.push_back(q);
  }
  int rc = good ? kOk : kCudaError;
  for (int k = 0; rc == kOk && k < 2; ++k) rc = run_step(p);
  for (size_t i = 0; i < backup.size(); ++i) {
    if (backup[i] && rc == kOk && !ok(cudaMemcpyAsync(live[i].first, backup[i], live[i].second, cudaMemcpyDeviceToDevice, p->s_main)))
      rc = kCudaError;
  }
  if (!ok(cudaStreamSynchronize(p->s_main)) || !ok(cudaStreamSynchronize(p->s_comm))) rc = rc == kOk ? kCudaError : rc;
  for (void* q : backup)
    if (q) cudaFree(q);
  if (rc != kOk || !capture) return rc;
  if (p->exec) { cudaGraphExecDestroy(p->exec); p->exec = nullptr; }
  if (p->graph) { cudaGraphDestroy(p->graph); p->graph = nullptr; }
  // thread-local mode: other threads of the process (a collective library's watchdog) may use the CUDA API meanwhile
  if (!ok(cudaStreamBeginCapture(p->s_main, cudaStreamCaptureModeThreadLocal))) return kCudaError;
  rc = run_step(p);
  cudaGraph_t g = nullptr;
  const cudaError_t e = cudaStreamEndCapture(p->s_main, &g);
  if (rc != kOk || e != cudaSuccess || !g) { if (g) cudaGraphDestroy(g); cudaGetLastError(); return rc != kOk ? rc : kCudaError; }
  p->graph = g;
  if (!ok(cudaGraphInstantiate(&p->exec, p->graph, 0))) { p->exec = nullptr; return kCudaError; }
  return kOk;
}

// Device-resident step: replays the graph (or runs the step eagerly when the plan was not captured).  Asynchronous.
int ge2b_mlp_plan_launch(ge2b_mlp_plan* p) {
  if (!p) return kBadArgs;
  if (p->exec) return ok(cudaGraphLaunch(p->exec, p->s_main)) ? kOk : kCudaError;
  return run_step(p);
}

// One step from HOST data: X [batch, dims[0]] in the compute dtype and int32 labels are copied up (page-locked buffers
// copy asynchronously), the step runs, and with loss_out the scalar loss of this rank's rows (their sum over the
// global batch size) is copied back and the call waits for it.
int ge2b_mlp_plan_step(ge2b_mlp_plan* p, const void* X_host, const int* labels_host, float* loss_out) {
  if (!p) return kBadArgs;
  const size_t B = static_cast<size_t>(p->cfg.batch);
  if (X_host && !ok(cudaMemcpyAsync(p->X, X_host, B * p->cfg.dims[0] * p->esz, cudaMemcpyHostToDevice, p->s_main))) return kCudaError;
  if (labels_host && !ok(cudaMemcpyAsync(p->labels, labels_host, B * sizeof(int), cudaMemcpyHostToDevice, p->s_main))) return kCudaError;
  const int rc = ge2b_mlp_plan_launch(p);
  if (rc != kOk) return rc;
  if (!loss_out) return kOk;
  if (!ok(cudaMemcpyAsync(loss_out, p->loss, sizeof(float), cudaMemcpyDeviceToHost, p->s_main))) return kCudaError;
  return ok(cudaStreamSynchronize(p->s_main)) ? kOk : kCudaError;
}

int ge2b_mlp_plan_sync(ge2b_mlp_plan* p) {
  if (!p) return kBadArgs;
  return ok(cudaStreamSynchronize(p->s_main)) && ok(cudaStreamSynchronize(p->s_comm)) ? kOk : kCudaError;
}

// Device addresses of the plan's static buffers and its stream, for callers that fill the batch on the device or time
// the step with their own events: what = 0 input X, 1 labels, 2 loss, 3 stream handle, 4 logits (last layer's output).
void* ge2b_mlp_plan_buffer(ge2b_mlp_plan* p, int what) {
  if (!p) return nullptr;
  switch (what) {
    case 0: return p->X;
    case 1: return p->labels;
    case 2: return p->loss;
    case 3: return p->s_main;
    case 4: return p->L[p->n - 1].y;
    default: return nullptr;
  }
}

long long ge2b_mlp_plan_launches_per_step(ge2b_mlp_plan* p) { return p ? p->launches_per_step : 0; }

}  // extern "C"
