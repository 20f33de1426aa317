"""ctypes binding of libge2_b200.so (declarations follow include/ge2_b200.h)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB = None


def library_path() -> Path:
    return _PKG / "lib" / "libge2_b200.so"


class ParamsLegacy(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("has_bias", C.c_int), ("act", C.c_int)]


class ParamsEx(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
                ("lda", C.c_int), ("ldb", C.c_int), ("ldc", C.c_int), ("ldd", C.c_int),
                ("alpha", C.c_float), ("beta", C.c_float),
                ("use_C", C.c_int), ("has_bias", C.c_int),
                ("bias_kind", C.c_int), ("act_kind", C.c_int),
                ("leaky_slope", C.c_float),
                ("save_preact", C.c_int), ("ldZ", C.c_int)]


class ParamsBwd(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
                ("lda", C.c_int), ("ldb", C.c_int), ("ldc", C.c_int),
                ("ldgY", C.c_int), ("ldZ", C.c_int),
                ("ldgA", C.c_int), ("ldgB", C.c_int), ("ldgC", C.c_int),
                ("alpha", C.c_float), ("beta", C.c_float),
                ("bias_kind", C.c_int), ("act_kind", C.c_int),
                ("leaky_slope", C.c_float)]


class ParamsTyped(C.Structure):
    _fields_ = [("base", ParamsEx),
                ("dtype", C.c_int), ("z_dtype", C.c_int), ("math", C.c_int),
                ("trans_b", C.c_int), ("batch", C.c_int),
                ("strideA", C.c_longlong), ("strideB", C.c_longlong), ("strideC", C.c_longlong),
                ("strideD", C.c_longlong), ("strideZ", C.c_longlong), ("trans_a", C.c_int)]


class ParamsSoftmaxCE(C.Structure):
    _fields_ = [("M", C.c_int), ("C", C.c_int), ("ld_logits", C.c_int), ("ld_dlogits", C.c_int),
                ("dtype", C.c_int), ("grad_dtype", C.c_int), ("reduction", C.c_int), ("ignore_index", C.c_int),
                ("grad_scale", C.c_float), ("mean_denominator", C.c_int), ("label_smoothing", C.c_float)]


class ParamsSGD(C.Structure):
    _fields_ = [("n", C.c_longlong), ("grad_dtype", C.c_int), ("low_dtype", C.c_int),
                ("lr", C.c_float), ("momentum", C.c_float), ("dampening", C.c_float), ("nesterov", C.c_int),
                ("weight_decay", C.c_float), ("decay_mode", C.c_int), ("grad_scale", C.c_float)]


class AllreduceSegment(C.Structure):
    _fields_ = [("offset_bytes", C.c_ulonglong), ("bytes", C.c_ulonglong), ("dtype", C.c_int)]


class AllreduceNvls(C.Structure):
    _fields_ = [("multicast_base", C.c_void_p), ("signal_pads", C.POINTER(C.c_void_p)), ("world", C.c_int),
                ("rank", C.c_int), ("n_segments", C.c_int), ("segments", AllreduceSegment * 2), ("blocks", C.c_int)]


MLP_MAX_LAYERS = 8


class MlpConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("dims", C.c_int * (MLP_MAX_LAYERS + 1)), ("acts", C.c_int * MLP_MAX_LAYERS),
                ("batch", C.c_int), ("global_batch", C.c_int), ("dtype", C.c_int), ("lr", C.c_float),
                ("world", C.c_int), ("rank", C.c_int), ("exchange", C.c_int),
                ("grad_base", C.c_void_p), ("grad_multicast", C.c_void_p), ("peer_grad_bases", C.POINTER(C.c_void_p)),
                ("nccl_unique_id", C.c_void_p), ("comm_blocks", C.c_int)]


class ParamsSdpa(C.Structure):
    _fields_ = [("B", C.c_int), ("H", C.c_int), ("M", C.c_int), ("N", C.c_int), ("D", C.c_int), ("dtype", C.c_int),
                ("scale", C.c_float), ("causal", C.c_int), ("mask_kind", C.c_int), ("dropout_p", C.c_float)]


class ParamsBwdTyped(C.Structure):
    _fields_ = [("base", ParamsBwd),
                ("dtype", C.c_int), ("z_dtype", C.c_int), ("math", C.c_int),
                ("scratch_bytes", C.c_size_t), ("reuse_gz", C.c_int)]


class ParamsConv2D(C.Structure):
    _fields_ = [("N", C.c_int), ("Cin", C.c_int), ("H", C.c_int), ("W", C.c_int),
                ("Cout", C.c_int), ("Kh", C.c_int), ("Kw", C.c_int),
                ("stride_h", C.c_int), ("stride_w", C.c_int), ("pad_h", C.c_int), ("pad_w", C.c_int),
                ("dil_h", C.c_int), ("dil_w", C.c_int), ("groups", C.c_int),
                ("act_kind", C.c_int), ("leaky_slope", C.c_float), ("with_bias", C.c_int), ("save_z", C.c_int),
                ("dtype", C.c_int), ("z_dtype", C.c_int), ("math", C.c_int)]


# numbering of the C ABI
BIAS_SCALAR, BIAS_PER_M, BIAS_PER_N = 0, 1, 2
ACT = {"none": 0, "relu": 1, "leaky_relu": 2, "leakyrelu": 2, "lrelu": 2, "gelu": 3, "sigmoid": 4, "tanh": 5}
DT_F32, DT_F16, DT_BF16 = 0, 1, 2
MATH_FP32, MATH_TENSOR, MATH_FP32X3 = 0, 1, 2
NOALLOC_SCRATCH_BYTES = 16 << 20

# every symbol include/ge2_b200.h declares
EXPORTS = [
    "ge2_launch", "ge2_launch_gemm_bias_act_f32", "ge2_launch_gemm_bias_act_tc_f16",
    "ge2_launch_gemm_bias_act_f32_ex", "ge2_launch_gemm_bias_act_bwd_f32_ex",
    "ge2_launch_gemm_bias_act_typed", "ge2_launch_gemm_bias_act_bwd_typed",
    "ge2b_backward_scratch_bytes", "ge2b_device_status", "ge2b_sm_count", "ge2b_set_sm_limit", "ge2b_version",
    "ge2b_last_route", "ge2b_launches_total", "ge2b_register_gemm_kernels",
    "ge2b_split_unavailable_total", "ge2b_release_scratch", "ge2b_selftest_wait_expiry",
    "ge2b_allreduce_nvls", "ge2b_allreduce_nvls_pad_bytes", "ge2b_sdpa_forward",
    "ge2b_mlp_plan_grad_bytes", "ge2b_nccl_unique_id", "ge2b_mlp_plan_create", "ge2b_mlp_plan_destroy",
    "ge2b_mlp_plan_set_params", "ge2b_mlp_plan_get_params", "ge2b_mlp_plan_get_grads", "ge2b_mlp_plan_compile",
    "ge2b_mlp_plan_launch", "ge2b_mlp_plan_step", "ge2b_mlp_plan_sync", "ge2b_mlp_plan_buffer",
    "ge2b_mlp_plan_launches_per_step",
    "ge2b_dense_plan_create", "ge2b_dense_plan_step", "ge2b_dense_plan_destroy",
    "ge2b_dense_plan_submit", "ge2b_dense_plan_wait",
    "ge2_launch_gemm_bias_act_bwd_noalloc",
    "ge2_launch_softmax_ce_fused", "ge2_launch_sgd_update",
    "ge2b_conv2d_forward", "ge2b_conv2d_backward", "ge2b_conv2d_output_size",
]


def load_library() -> C.CDLL:
    """Loads the CUDA launch layer.  Raises if it has not been built: there is nothing to fall back to."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python __graft_entry__.py` (nvcc, sm_100a). "
            "This package has no CPU or eager fallback.")
    lib = C.CDLL(str(path))
    launch_sig = [C.POINTER(C.c_size_t), C.c_int, C.c_void_p]
    for name in ("ge2_launch_gemm_bias_act_f32", "ge2_launch_gemm_bias_act_tc_f16",
                 "ge2_launch_gemm_bias_act_f32_ex", "ge2_launch_gemm_bias_act_bwd_f32_ex",
                 "ge2_launch_gemm_bias_act_typed", "ge2_launch_gemm_bias_act_bwd_typed",
                 "ge2_launch_gemm_bias_act_bwd_noalloc", "ge2_launch_softmax_ce_fused", "ge2_launch_sgd_update"):
        fn = getattr(lib, name)
        fn.argtypes = launch_sig
        fn.restype = C.c_int
    lib.ge2_launch.argtypes = [C.c_char_p] + launch_sig
    lib.ge2_launch.restype = C.c_int
    lib.ge2b_backward_scratch_bytes.argtypes = [C.c_longlong, C.c_longlong]
    lib.ge2b_backward_scratch_bytes.restype = C.c_size_t
    lib.ge2b_device_status.argtypes = [C.c_int]
    lib.ge2b_device_status.restype = C.c_int
    lib.ge2b_sm_count.restype = C.c_int
    lib.ge2b_set_sm_limit.argtypes = [C.c_int]
    lib.ge2b_set_sm_limit.restype = None
    lib.ge2b_version.restype = C.c_char_p
    lib.ge2b_last_route.restype = C.c_int
    lib.ge2b_launches_total.restype = C.c_longlong
    lib.ge2b_split_unavailable_total.restype = C.c_longlong
    lib.ge2b_release_scratch.restype = None
    lib.ge2b_selftest_wait_expiry.argtypes = [C.c_longlong, C.POINTER(C.c_int), C.c_void_p]
    lib.ge2b_selftest_wait_expiry.restype = C.c_int
    lib.ge2b_allreduce_nvls.argtypes = [C.POINTER(AllreduceNvls), C.c_void_p]
    lib.ge2b_allreduce_nvls.restype = C.c_int
    lib.ge2b_allreduce_nvls_pad_bytes.restype = C.c_int
    lib.ge2b_sdpa_forward.argtypes = [C.POINTER(ParamsSdpa)] + [C.c_void_p] * 7
    lib.ge2b_sdpa_forward.restype = C.c_int
    vp = C.c_void_p
    lib.ge2b_mlp_plan_grad_bytes.argtypes = [C.POINTER(MlpConfig)]
    lib.ge2b_mlp_plan_grad_bytes.restype = C.c_size_t
    lib.ge2b_nccl_unique_id.argtypes = [vp]
    lib.ge2b_mlp_plan_create.argtypes = [C.POINTER(vp), C.POINTER(MlpConfig)]
    lib.ge2b_mlp_plan_destroy.argtypes = [vp]
    lib.ge2b_mlp_plan_destroy.restype = None
    lib.ge2b_mlp_plan_set_params.argtypes = [vp, C.c_int, vp, vp]
    lib.ge2b_mlp_plan_get_params.argtypes = [vp, C.c_int, vp, vp, vp]
    lib.ge2b_mlp_plan_get_grads.argtypes = [vp, C.c_int, vp, vp]
    lib.ge2b_mlp_plan_compile.argtypes = [vp, C.c_int]
    lib.ge2b_mlp_plan_launch.argtypes = [vp]
    lib.ge2b_mlp_plan_step.argtypes = [vp, vp, vp, vp]
    lib.ge2b_mlp_plan_sync.argtypes = [vp]
    lib.ge2b_mlp_plan_buffer.argtypes = [vp, C.c_int]
    lib.ge2b_mlp_plan_buffer.restype = vp
    lib.ge2b_mlp_plan_launches_per_step.argtypes = [vp]
    lib.ge2b_mlp_plan_launches_per_step.restype = C.c_longlong
    for name in ("ge2b_nccl_unique_id", "ge2b_mlp_plan_create", "ge2b_mlp_plan_set_params", "ge2b_mlp_plan_get_params",
                 "ge2b_mlp_plan_get_grads", "ge2b_mlp_plan_compile", "ge2b_mlp_plan_launch", "ge2b_mlp_plan_step",
                 "ge2b_mlp_plan_sync"):
        getattr(lib, name).restype = C.c_int
    lib.ge2b_dense_plan_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_float, C.c_int, C.c_int]
    lib.ge2b_dense_plan_create.restype = C.c_int
    lib.ge2b_dense_plan_step.argtypes = [C.c_void_p] * 9
    lib.ge2b_dense_plan_step.restype = C.c_int
    lib.ge2b_dense_plan_submit.argtypes = [C.c_void_p] * 9
    lib.ge2b_dense_plan_submit.restype = C.c_int
    lib.ge2b_dense_plan_wait.argtypes = [C.c_void_p]
    lib.ge2b_dense_plan_wait.restype = C.c_int
    lib.ge2b_dense_plan_destroy.argtypes = [C.c_void_p]
    lib.ge2b_dense_plan_destroy.restype = None
    lib.ge2b_conv2d_forward.argtypes = [C.POINTER(ParamsConv2D)] + [C.c_void_p] * 6
    lib.ge2b_conv2d_forward.restype = C.c_int
    lib.ge2b_conv2d_backward.argtypes = [C.POINTER(ParamsConv2D)] + [C.c_void_p] * 8
    lib.ge2b_conv2d_backward.restype = C.c_int
    lib.ge2b_conv2d_output_size.argtypes = [C.POINTER(ParamsConv2D), C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.ge2b_conv2d_output_size.restype = C.c_int
    _LIB = lib
    return lib


def make_bufs(ptrs, params) -> "C.Array":
    """bufs[] of the C ABI: device pointers as uintptr_t, then the HOST address of the parameter struct."""
    vals = [int(p) for p in ptrs] + [C.addressof(params)]
    return (C.c_size_t * len(vals))(*vals)


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = {-1: "bad arguments", -2: "CUDA error", -99: "not implemented"}.get(rc, "error")
    raise RuntimeError(f"[ge2_b200::{what}] {msg} (code {rc})")
