/*
 * C ABI of the B200 dense-layer launch layer (libge2_b200.so).
 *
 * The first five entry points are the reference's own C ABI for this path, unchanged: same names,
 * same `bufs[]` conventions (device pointers as uintptr_t, LAST entry a HOST pointer to the parameter
 * struct, read during the call), same return codes (0 ok, -1 bad arguments, -2 CUDA error,
 * -99 not implemented).  The remaining entry points are additions behind the same convention for the
 * 16-bit / TF32 tensor-core paths, the strided-batched form and host-buffer calls.
 *
 * All launches are asynchronous on `stream` (a cudaStream_t cast to void*; NULL = default stream).
 * Nothing is retained after a call returns.  There is no CPU fallback: without a CUDA device every
 * launch returns -2.
 */
#ifndef GE2_B200_H_
#define GE2_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uintptr_t ge2_uintptr;

/* ---- enums: numbering of the reference's C ABI (dev/backend/graph_executor_v2/include/ge_v2_api_ex.h:15-28).
 *      Note GE2_BIAS_* differs from the C++ BiasKind numbering (None=0, Scalar=1, PerM=2, PerN=3). ---- */
typedef enum { GE2_BIAS_SCALAR = 0, GE2_BIAS_PER_M = 1, GE2_BIAS_PER_N = 2 } ge2_bias_kind_t;
typedef enum {
  GE2_ACT_NONE = 0, GE2_ACT_RELU = 1, GE2_ACT_LEAKY_RELU = 2, GE2_ACT_GELU = 3, GE2_ACT_SIGMOID = 4, GE2_ACT_TANH = 5
} ge2_act_kind_t;

/* dtype numbering of the reference's DType (backends/cuda/ops/_common/shim/ai_device.hpp:15) */
typedef enum { GE2_DT_F32 = 0, GE2_DT_F16 = 1, GE2_DT_BF16 = 2 } ge2_dtype_t;
/* arithmetic for fp32 tensors: exact fp32 FMA (parity with the reference's fp32 path) or TF32 tensor cores */
/* fp32 tensors only.  FP32: exact fp32 FMA chains in the forward (bit-identical pre-activation to the reference
 * kernel); the backward GEMMs, which the reference hands to cuBLAS, run error-compensated on the tensor cores.
 * TENSOR: TF32 tensor cores (inputs truncated to 10 mantissa bits).  FP32X3: error-compensated TF32 everywhere (three
 * TF32 products of operands split into big + small parts, fp32-grade results; needs stream-ordered scratch, so outside
 * stream capture). */
typedef enum { GE2_MATH_FP32 = 0, GE2_MATH_TENSOR = 1, GE2_MATH_FP32X3 = 2 } ge2_math_t;

/* ---- replaces dev/backend/graph_executor_v2/include/ge_v2_api.h:12-18 ---- */
typedef struct {
  int M, N, K;
  int has_bias; /* 0/1 */
  int act;      /* 0 none, 1 ReLU */
} ge2_gemm_bias_act_params_t;

/* ---- replaces dev/backend/graph_executor_v2/include/ge_v2_api_ex.h:37-62 ---- */
typedef struct {
  int M, N, K;
  int lda, ldb, ldc, ldd;     /* <= 0: row-major default (K, N, N, N) */
  float alpha;                /* 0 is read as 1 */
  float beta;
  int use_C, has_bias;        /* 0/1: whether bufs[] carries C / bias */
  ge2_bias_kind_t bias_kind;
  ge2_act_kind_t act_kind;
  float leaky_slope;
  int save_preact;            /* 1: bufs[] carries Z and the pre-activation is written there */
  int ldZ;                    /* <= 0: ldd */
} ge2_gemm_bias_act_params_ex_t;

/* ---- replaces dev/backend/graph_executor_v2/include/ge_v2_api_ex.h:94-113 ---- */
typedef struct {
  int M, N, K;
  int lda, ldb, ldc;
  int ldgY, ldZ;
  int ldgA, ldgB, ldgC;       /* <= 0: row-major default */
  float alpha, beta;
  ge2_bias_kind_t bias_kind;
  ge2_act_kind_t act_kind;
  float leaky_slope;
} ge2_gemm_bias_act_bwd_params_t;

/* Name-keyed dispatcher.  Replaces dev/backend/graph_executor_v2/src/launch_table.cpp:31-96 (declared again
 * in graph_executor_v2/include/ai/legacy_ge2_api.h:7-13).  Names: "gemm_bias_act_f32", "gemm_bias_act_tc_f16",
 * "gemm_bias_act_f32_ex" | "gemm_bias_act_ex", "gemm_bias_act_bwd_f32_ex" | "gemm_bias_act_bwd", and the
 * additions "gemm_bias_act_typed" | "gemm_strided_batched", "gemm_bias_act_bwd_typed".  Unknown name: -1. */
int ge2_launch(const char* name, const ge2_uintptr* bufs, int n, void* stream);

/* fp32, D = act(A.B + bias).  bufs = [A, B, (bias), D, &ge2_gemm_bias_act_params_t].
 * Replaces dev/backend/graph_executor_v2/src/my_kernels.cu:36-73. */
int ge2_launch_gemm_bias_act_f32(const ge2_uintptr* bufs, int n, void* stream);

/* fp16 tensor-core form of the call above: A, B, D are IEEE half, bias fp32, fp32 accumulation.
 * The reference ships this slot as a stub returning -99 (my_kernels.cu:76-80); here it runs on tcgen05. */
int ge2_launch_gemm_bias_act_tc_f16(const ge2_uintptr* bufs, int n, void* stream);

/* fp32, D = act(alpha*A.B + beta*C + bias) with optional pre-activation stash.
 * bufs = [A, B, (C), D, (bias), (Z), &ge2_gemm_bias_act_params_ex_t].
 * Replaces dev/backend/graph_executor_v2/src/my_kernels.cu:117-195. */
int ge2_launch_gemm_bias_act_f32_ex(const ge2_uintptr* bufs, int n, void* stream);

/* fp32 backward.  bufs = [A, B, C|0, gY, Z, gA|0, gB|0, gC|0, gBias|0, &ge2_gemm_bias_act_bwd_params_t]
 * (fixed 10 slots).  The gZ scratch is taken from the stream-ordered allocator, as the reference does
 * when it is given no workspace.  Replaces dev/backend/graph_executor_v2/src/my_kernels.cu:199-254. */
int ge2_launch_gemm_bias_act_bwd_f32_ex(const ge2_uintptr* bufs, int n, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Additions: typed + strided-batched forward, typed backward.
 * ------------------------------------------------------------------------------------------------ */
typedef struct {
  ge2_gemm_bias_act_params_ex_t base;
  ge2_dtype_t dtype;          /* of A, B, C and D */
  ge2_dtype_t z_dtype;        /* of Z */
  ge2_math_t math;            /* fp32 tensors only */
  int trans_b;                /* 1: B is given as [N,K] row-major (the Q.K^T form); ldb default becomes K */
  int batch;                  /* <= 1: a single GEMM */
  long long strideA, strideB, strideC, strideD, strideZ; /* elements between slices; 0 broadcasts an input */
  int trans_a;                /* 1: A is given as [K,M] row-major (the X^T.gZ form); lda default becomes M */
} ge2_gemm_typed_params_t;

/* Same bufs layout as ge2_launch_gemm_bias_act_f32_ex with &ge2_gemm_typed_params_t last.  Stands in for the
 * per-(batch, head) loops of 2-D GEMM calls in backends/cuda/ops/sdpa/launcher.cu:185-222,236-270, the per-image
 * loop of backends/cuda/ops/conv2d/launcher.cu:180-227 and dev/backend/graph_executor/ge/gemm_rm.cuh:38-66. */
int ge2_launch_gemm_bias_act_typed(const ge2_uintptr* bufs, int n, void* stream);

typedef struct {
  ge2_gemm_bias_act_bwd_params_t base;
  ge2_dtype_t dtype;          /* of A, B, C, gY, gA, gB, gC */
  ge2_dtype_t z_dtype;        /* of Z */
  ge2_math_t math;
  size_t scratch_bytes;       /* size of the scratch in slot 9 (0 = not stated) */
  int reuse_gz;               /* 1: the scratch already holds gZ from an earlier call on the same gY and Z: only the
                                 requested GEMMs run (lets a caller launch dW, start its all-reduce, then launch dX) */
} ge2_gemm_bwd_typed_params_t;

/* bufs = [A, B, C|0, gY, Z, gA|0, gB|0, gC|0, gBias|0, scratch|0, &ge2_gemm_bwd_typed_params_t] (fixed 11 slots).
 * `scratch` holds gZ (M*N elements of `dtype`); with scratch == 0 it is taken from the stream-ordered allocator.
 * Typed form of backends/cuda/ops/gemm/kernels/regemm_backward.cu:151-301. */
int ge2_launch_gemm_bias_act_bwd_typed(const ge2_uintptr* bufs, int n, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Host-buffer plan: forward + backward of one dense layer with inputs and results in HOST memory.
 * Counterpart of the reference's GemmPlan (graph_executor_v2/src/bindings/py_api.cpp:403-523): device buffers
 * are allocated at creation; a step copies inputs up, runs Y = act(X.W + b) and (dX, dW, db) from dY, and copies
 * the results down, pipelined over internal streams.  A step returns when the results are in host memory.
 * Null result pointers are skipped.  Use page-locked host memory for full PCIe speed.  One plan serves one
 * thread at a time.
 * ------------------------------------------------------------------------------------------------ */
typedef struct ge2b_dense_plan ge2b_dense_plan;
int ge2b_dense_plan_create(ge2b_dense_plan** out, int M, int K, int N, ge2_dtype_t dtype, ge2_act_kind_t act,
                           float leaky_slope, int has_bias, ge2_math_t math);
int ge2b_dense_plan_step(ge2b_dense_plan* plan, const void* X, const void* W, const float* bias, const void* dY,
                         void* Y, void* dX, void* dW, float* db);
/* The same step split in two: `submit` enqueues the copies and kernels and returns; `wait` blocks until the OLDEST
 * submitted step's results are in its host buffers.  Up to two steps may be in flight (a third submit first waits
 * for the oldest); the host buffers of a step must stay untouched until its wait returns. */
int ge2b_dense_plan_submit(ge2b_dense_plan* plan, const void* X, const void* W, const float* bias, const void* dY,
                           void* Y, void* dX, void* dW, float* db);
int ge2b_dense_plan_wait(ge2b_dense_plan* plan);
void ge2b_dense_plan_destroy(ge2b_dense_plan* plan);

/* ------------------------------------------------------------------------------------------------
 * The two passes either side of the dense layers in a training step.
 * ------------------------------------------------------------------------------------------------ */
typedef struct {
  int M, C;                   /* rows (samples), classes */
  int ld_logits, ld_dlogits;  /* <= 0: C */
  ge2_dtype_t dtype;          /* of the logits */
  ge2_dtype_t grad_dtype;     /* of dlogits */
  int reduction;              /* 0 none (loss[M]), 1 mean, 2 sum (loss[1]) */
  int ignore_index;           /* rows with this label give zero loss and zero gradient; -1 disables */
  float grad_scale;           /* dlogits = (softmax - onehot) * grad_scale; pass 1/batch for a mean loss */
  int mean_denominator;       /* <= 0: M.  The global batch when the rows are one shard of it. */
  float label_smoothing;      /* target = (1 - ls) * onehot + ls / C, as the reference's separate CE ops
                                 (cross_entropy/kernels.cu:96-101,188-195); 0 = off */
} ge2_softmax_ce_params_t;

/* Fused softmax + cross-entropy from logits, forward and backward in one pass.
 * bufs = [logits, labels(int32), dlogits, loss|0, &ge2_softmax_ce_params_t].
 * Replaces SoftmaxCEFusedForwardBackwardCudaLaunch (backends/cuda/ops/cross_entropy/api.hpp:46-56,
 * kernels.cu:287-372).  Like the reference's native op, a mean divides by the row count including ignored rows. */
int ge2_launch_softmax_ce_fused(const ge2_uintptr* bufs, int n, void* stream);

typedef struct {
  long long n;                /* elements */
  ge2_dtype_t grad_dtype;     /* of the gradient */
  ge2_dtype_t low_dtype;      /* of the optional low-precision copy of the parameters */
  float lr, momentum, dampening;
  int nesterov;
  float weight_decay;
  int decay_mode;             /* 0 none, 1 L2 (added to the gradient), 2 decoupled */
  float grad_scale;           /* 0 is read as 1 */
} ge2_sgd_params_t;

/* SGD step on fp32 master parameters.  bufs = [param(fp32), grad, velocity(fp32)|0, param_low|0, &ge2_sgd_params_t].
 * Replaces SGDCudaLaunch's kernel (backends/cuda/ops/optimizer/kernels.cu:33-66; L2 decay) and the Python optimizer's
 * element-wise kernel (python/graph_executor_v2/optim/sgd.py:16-64; decoupled decay); param_low receives the updated
 * parameters rounded to `low_dtype` for the next forward pass. */
int ge2_launch_sgd_update(const ge2_uintptr* bufs, int n, void* stream);

/* Backward for callers that may not allocate device memory and have no scratch of their own to pass: the gZ
 * scratch is a fixed GE2B_NOALLOC_SCRATCH_BYTES array inside the library's device image (held by every GPU that
 * loads the library, until the process exits).  This entry point has no counterpart in the reference, whose
 * backward either receives a workspace or calls cudaMallocAsync.
 * bufs = [A, B, C|0, gY, Z, gA|0, gB|0, gC|0, gBias|0, &ge2_gemm_bwd_typed_params_t]  (10 slots; scratch_bytes and
 * reuse_gz of the struct are ignored).  Returns -1 when M*N*sizeof(element) > GE2B_NOALLOC_SCRATCH_BYTES.
 * All calls on one GPU share the array: calls whose kernels may overlap on the GPU must be ordered by the caller.
 * What the array has left after gZ holds the GEMMs' split-K partial sums; the library creates no scratch of its own
 * during the call (a problem whose split does not fit runs unsplit).
 * The first call on a device performs a one-time address lookup, and with lazy module loading it is also when the
 * driver reserves the array's 16 MiB; make it before any stream capture begins and before a pool takes the
 * whole GPU. */
#define GE2B_NOALLOC_SCRATCH_BYTES (16u << 20)
int ge2_launch_gemm_bias_act_bwd_noalloc(const ge2_uintptr* bufs, int n, void* stream);

/* Bytes of gZ scratch the backward needs (mirrors GemmRequiredBackwardScratchBytes,
 * backends/cuda/ops/gemm/api.hpp:107-112, which always counts fp32). */
size_t ge2b_backward_scratch_bytes(long long M, long long N);

/* Device status word of the current device: 0, or a bit set when a bounded wait inside a kernel ran out.
 * Synchronises the device.  clear != 0 resets it. */
int ge2b_device_status(int clear);
int ge2b_sm_count(void);
/* The tensor-core GEMM is a persistent kernel sized to every SM of the device.  A caller that runs a collective
 * (NCCL) concurrently with a GEMM can leave it room: subsequent GEMM launches of this process occupy at most
 * `n` SMs.  n <= 0 restores the default.  No counterpart in the reference (single GPU, single stream). */
void ge2b_set_sm_limit(int n);
const char* ge2b_version(void);

/* Fills the C++ kernel registries of include/ge2_dispatch.hpp with this library's entries (idempotent).  Stands where
 * the reference declares, and never defines, ai_backend_cuda_register_all (src/bindings/py_api.cpp:43). */
void ge2b_register_gemm_kernels(void);

/* ---- 2-D convolution on the GEMM kernels (NCHW tensors, OIHW weight, groups = 1) ----
 * Replaces Conv2DCudaLaunch / Conv2DCudaBackwardLaunch (backends/cuda/ops/conv2d/api.hpp:44-64, launcher.cu:115-462):
 * same attributes (Conv2DAttrs, api.hpp:6-16) and the same output-size rule, but one im2col pass and one batched
 * GEMM launch for the whole batch instead of a per-image loop, and no caller-provided workspace (scratch is
 * allocated and freed in stream order).  dtype tags every tensor (GE2_DT_*); bias and dB stay fp32; Z may be fp32
 * or dtype.  math as in ge2_params_typed_t.  dB is the sum over the whole batch (the reference's per-image
 * GemmCudaBackward zeroes the bias gradient on every call, launcher.cu:420-431 with regemm_backward.cu:196, so its
 * dB holds the last image only). */
typedef struct {
  int N, Cin, H, W;          /* input  [N, Cin, H, W] */
  int Cout, Kh, Kw;          /* weight [Cout, Cin, Kh, Kw] */
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int groups;                /* must be 1 (anything else: -99, as the reference returns Unimplemented) */
  int act_kind;              /* GE2_ACT_* */
  float leaky_slope;
  int with_bias;
  int save_z;                /* forward: also write the pre-activation to Z */
  int dtype, z_dtype, math;
} ge2b_conv2d_params_t;

/* Y [N, Cout, Ho, Wo] = act(conv(X, W) + bias[co]).  Returns 0, -1 (bad arguments), -2 (CUDA error), -99. */
int ge2b_conv2d_forward(const ge2b_conv2d_params_t* p, const void* X, const void* W, const float* bias, void* Y, void* Z,
                        void* stream);
/* (X, W, dY, Z) -> dW [Cout, Cin, Kh, Kw], dB [Cout] fp32, dX [N, Cin, H, W]; any output may be null.  Outputs are
 * overwritten (not accumulated into). */
int ge2b_conv2d_backward(const ge2b_conv2d_params_t* p, const void* X, const void* W, const void* dY, const void* Z,
                         void* dW, float* dB, void* dX, void* stream);
/* Ho, Wo for the geometry in p (conv2d/launcher.cu:137-138). */
int ge2b_conv2d_output_size(const ge2b_conv2d_params_t* p, int* Ho, int* Wo);

/* ------------------------------------------------------------------------------------------------
 * Fused scaled-dot-product attention forward, the caller of the batched GEMM pair S = scale.Q.K^T, O = softmax(S).V
 * with the scores kept on chip.  Replaces SDPACudaLaunch's per-(batch, head) transpose / GEMM / scale / mask /
 * softmax / GEMM sequence (backends/cuda/ops/sdpa/api.hpp:18-26, launcher.cu:129-270).
 * ------------------------------------------------------------------------------------------------ */
typedef struct {
  int B, H;                   /* batch, heads */
  int M, N;                   /* queries, keys per (batch, head) */
  int D;                      /* head dimension: 64 or 128 */
  ge2_dtype_t dtype;          /* of Q, K, V and O: GE2_DT_BF16 */
  float scale;                /* 0: 1/sqrt(D), as SDPAAttrs::scale */
  int causal;                 /* keys n > m are masked for query m */
  int mask_kind;              /* of the optional mask [B,1,M,N]: 1 fp32 additive, 2 int8, 3 int32 (non-zero = masked) */
  float dropout_p;            /* must be 0 (-99 otherwise) */
} ge2b_sdpa_params_t;

/* Q [B,H,M,D], K, V [B,H,N,D], O [B,H,M,D] contiguous; mask may be null; lse (fp32 [B,H,M], the log-sum-exp of every
 * row's scaled and masked scores) may be null.  A row with every key masked gives zeros.  Returns 0, -1, -2 or -99
 * (a dtype, head dimension or dropout this kernel does not cover). */
int ge2b_sdpa_forward(const ge2b_sdpa_params_t* p, const void* Q, const void* K, const void* V, const void* mask, void* O,
                      float* lse, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Data-parallel gradient exchange: sum all-reduce over NVLink / NVSwitch in one kernel per rank.
 * No counterpart in the reference (it has no multi-GPU path); this is the "dW / db are combined across the GPUs"
 * step of the sharded dense layer.  Every rank reduces its slice of a symmetric buffer inside the switch
 * (multimem.ld_reduce) and writes the sums to every GPU (multimem.st).  bf16 values are summed in fp32.
 * ------------------------------------------------------------------------------------------------ */
typedef struct {
  unsigned long long offset_bytes;   /* from the buffer base; multiple of 16 */
  unsigned long long bytes;          /* multiple of 16 */
  ge2_dtype_t dtype;                 /* GE2_DT_BF16 or GE2_DT_F32 */
} ge2b_allreduce_segment_t;

typedef struct {
  void* multicast_base;              /* multicast address of the symmetric buffer (same offset layout on every rank) */
  void* const* signal_pads;          /* [world] addresses, valid on this GPU, of every rank's signal pad: at least
                                        ge2b_allreduce_nvls_pad_bytes() bytes each, zero before the first call */
  int world, rank;                   /* 2..16 ranks, one per GPU */
  int n_segments;                    /* 1 or 2 regions of the buffer (e.g. bf16 dW and fp32 db in one bucket) */
  ge2b_allreduce_segment_t segments[2];
  int blocks;                        /* thread blocks (SMs) to use; <= 0: 32 */
} ge2b_allreduce_nvls_t;

/* Launches the exchange on `stream`.  Every rank must call it with the same segments; the kernels of the ranks wait
 * for each other (bounded: a wait that runs out sets bit 1 of ge2b_device_status and the kernel returns), so one rank
 * per GPU.  The signal pads are left all-zero again, so the launch may be captured into a CUDA graph and replayed.
 * Returns 0, -1 (bad arguments) or -2. */
int ge2b_allreduce_nvls(const ge2b_allreduce_nvls_t* args, void* stream);
int ge2b_allreduce_nvls_pad_bytes(void);

/* ------------------------------------------------------------------------------------------------
 * The captured training step around the dense layers: Dense stack -> softmax cross-entropy (mean) -> SGD.
 * C++ counterpart of the reference's Python graph runtime for this path (graph/capture_plan.py:250-287 buffers per
 * layer, graph/runtime.py:24-148 step order, graph/graph_exec.py:51-231 warm-up / capture / replay,
 * layers/sequential.py:416-497 compile / one_step).  Buffers are allocated once; the step is replayed from a CUDA
 * graph.  With world > 1 the rows are one shard of the global batch and every layer's dW / db are summed over the
 * ranks on a side stream under the rest of the backward pass.
 * ------------------------------------------------------------------------------------------------ */
#define GE2B_MLP_MAX_LAYERS 8
typedef struct ge2b_mlp_plan ge2b_mlp_plan;
typedef struct {
  int n_layers;                          /* 1..GE2B_MLP_MAX_LAYERS */
  int dims[GE2B_MLP_MAX_LAYERS + 1];     /* dims[i] -> dims[i+1] is layer i */
  int acts[GE2B_MLP_MAX_LAYERS];         /* GE2_ACT_* per layer */
  int batch;                             /* rows on this rank */
  int global_batch;                      /* rows over all ranks (<= 0: batch): denominator of the mean loss */
  ge2_dtype_t dtype;                     /* compute dtype of weights / activations (fp32 master weights are kept) */
  float lr;
  int world, rank;                       /* data-parallel replicas; world 1 = single GPU */
  int exchange;                          /* world > 1: 1 = ge2b_allreduce_nvls over the symmetric memory below,
                                            2 = the collective library (NCCL), communicator built from nccl_unique_id */
  void* grad_base;                       /* exchange 1: this rank's mapping of the symmetric gradient buffer of
                                            ge2b_mlp_plan_grad_bytes() bytes, zero-filled ... */
  void* grad_multicast;                  /* ... its multicast address ... */
  void* const* peer_grad_bases;          /* ... and every rank's buffer as mapped on this GPU [world] */
  const void* nccl_unique_id;            /* exchange 2: 128 bytes from ge2b_nccl_unique_id() on rank 0, sent to all */
  int comm_blocks;                       /* exchange 1: thread blocks of the exchange kernel (<= 0: default) */
} ge2b_mlp_config_t;

size_t ge2b_mlp_plan_grad_bytes(const ge2b_mlp_config_t* cfg);
int ge2b_nccl_unique_id(void* id128);
int ge2b_mlp_plan_create(ge2b_mlp_plan** out, const ge2b_mlp_config_t* cfg);
void ge2b_mlp_plan_destroy(ge2b_mlp_plan* plan);
/* fp32 HOST arrays: W [dims[l], dims[l+1]] row-major and b [dims[l+1]]; null = leave unchanged. */
int ge2b_mlp_plan_set_params(ge2b_mlp_plan* plan, int layer, const float* W, const float* b);
/* Any of W (fp32 master), b, W_low (the compute-dtype copy) may be null. */
int ge2b_mlp_plan_get_params(ge2b_mlp_plan* plan, int layer, float* W, float* b, void* W_low);
/* Gradients of the last step, after the exchange: gW in the compute dtype, gb fp32. */
int ge2b_mlp_plan_get_grads(ge2b_mlp_plan* plan, int layer, void* gW, float* gb);
/* Warm-up (parameters are saved and restored around it) and, with capture != 0, graph capture + instantiation. */
int ge2b_mlp_plan_compile(ge2b_mlp_plan* plan, int capture);
/* One step on the batch already in the plan's device buffers (asynchronous). */
int ge2b_mlp_plan_launch(ge2b_mlp_plan* plan);
/* One step from HOST data (X in the compute dtype, int32 labels; null = keep the batch in place); with loss_out the
 * call waits for the step and returns this rank's share of the mean loss. */
int ge2b_mlp_plan_step(ge2b_mlp_plan* plan, const void* X_host, const int* labels_host, float* loss_out);
int ge2b_mlp_plan_sync(ge2b_mlp_plan* plan);
/* what: 0 input X, 1 labels (int32), 2 loss (fp32 scalar), 3 the plan's stream (cudaStream_t), 4 logits. */
void* ge2b_mlp_plan_buffer(ge2b_mlp_plan* plan, int what);
long long ge2b_mlp_plan_launches_per_step(ge2b_mlp_plan* plan);

/* Introspection for tests and benchmarks: which kernel family the calling thread's most recent GEMM went to
 * (0 none, 1 exact-fp32 CUDA-core kernel, 2 tcgen05 tensor-core kernel) and how many kernels this library
 * has launched in the process. */
int ge2b_last_route(void);
long long ge2b_launches_total(void);
/* Split-K launches that ran unsplit because no scratch could be had: the stream was being captured before any split
 * launch had warmed it up, or the call was one that must not allocate and lent too little.  A step whose captured
 * form differs from its eager form shows up here. */
long long ge2b_split_unavailable_total(void);
/* Self-test of the kernels' bounded waits: launches a one-warp kernel that waits, with a budget of `budget_cycles` SM
 * clocks (at most 2e8), on an mbarrier nothing arrives at.  The wait gives up, the kernel ORs the "wait timed out" bit
 * (1) into the device status word and returns; report4 (host memory, 4 ints) receives {wait result (0 = gave up),
 * abort flag, cycles waited, result of a second waiter that found the abort flag set}.  Synchronises the stream.
 * Clear the status word with ge2b_device_status(1) afterwards. */
int ge2b_selftest_wait_expiry(long long budget_cycles, int* report4, void* stream);
/* Synchronises the current device and frees every split-K scratch buffer the library created (64 MiB per
 * (device, stream) that ever ran a split launch).  The buffers come back on demand. */
void ge2b_release_scratch(void);

#ifdef __cplusplus
}
#endif
#endif /* GE2_B200_H_ */
