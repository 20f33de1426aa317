"""GEMM + bias + activation glue over the C ABI, mirroring the reference's Python op module
(graph_executor_v2/python/graph_executor_v2/ops/gemm.py:99-509): `forward`, `backward` (allocating) and
`forward_into`, `backward_into` (no allocation, usable while a CUDA graph is being captured), plus
`forward_batched` for the strided-batched form.

Differences from the reference glue, all additive: device arrays are torch tensors (CuPy is what the
reference uses), tensors may be float32, bfloat16 or float16, and fp32 tensors take `math="fp32"` (default: exact
forward, error-compensated tensor-core backward), `math="tf32"` (TF32 tensor cores) or `math="fp32x3"`
(error-compensated tensor cores in the forward too).  Bias and bias gradients are always float32.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple, Union

import torch

from . import _lib
from ._lib import ACT, BIAS_PER_M, BIAS_PER_N, BIAS_SCALAR, DT_BF16, DT_F16, DT_F32, MATH_FP32, MATH_FP32X3, MATH_TENSOR

_DT = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}


def _dt(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise ValueError(f"{name}: dtype must be float32, float16 or bfloat16, got {t.dtype}")
    return _DT[t.dtype]


def _check_2d(t: torch.Tensor, name: str) -> Tuple[int, int]:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA torch.Tensor")
    if t.dim() != 2:
        raise ValueError(f"{name}: expected 2D, got shape {tuple(t.shape)}")
    if t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        raise ValueError(f"{name}: expected row-major with unit inner stride")
    return int(t.shape[0]), int(t.shape[1])


def _act_code(act: Optional[str]) -> int:
    key = (act or "none").lower()
    if key not in ACT:
        raise ValueError(f"Unsupported act: {act}")
    return ACT[key]


def _math_code(math: str) -> int:
    if math not in ("fp32", "tf32", "fp32x3"):
        raise ValueError("math must be 'fp32', 'tf32' or 'fp32x3'")
    return {"fp32": MATH_FP32, "tf32": MATH_TENSOR, "fp32x3": MATH_FP32X3}[math]


def _stream_ptr(stream, device=None) -> int:
    if stream is None:
        return int(torch.cuda.current_stream(device).cuda_stream)
    if isinstance(stream, torch.cuda.Stream):
        return int(stream.cuda_stream)
    return int(stream)


def _one_device(*tensors) -> torch.device:
    """All tensors of a call must live on ONE GPU: the launch layer builds tensor maps over their addresses and
    launches on that device.  Raises before anything is launched."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise ValueError("expected CUDA tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors of one call are on different devices: {dev} and {t.device}")
    return dev


def _bias_kind(bias: torch.Tensor, M: int, N: int) -> int:
    """Shape rule of the reference launcher (backends/cuda/ops/gemm/launcher.cu:47-77):
    1-D length 1 -> scalar, N -> per-column, M -> per-row; then (1,N), (M,1), (1,1)."""
    s = tuple(bias.shape)
    if len(s) == 1:
        if s[0] == 1:
            return BIAS_SCALAR
        if s[0] == N:
            return BIAS_PER_N
        if s[0] == M:
            return BIAS_PER_M
    if s == (1, N):
        return BIAS_PER_N
    if s == (M, 1):
        return BIAS_PER_M
    if s == (1, 1):
        return BIAS_SCALAR
    n = bias.numel()
    if n == N:
        return BIAS_PER_N
    if n == M:
        return BIAS_PER_M
    if n == 1:
        return BIAS_SCALAR
    raise ValueError(f"bias shape {s} matches none of scalar / (N,) / (M,) / (1,N) / (M,1)")


def _prep_bias(bias, M: int, N: int) -> Optional[torch.Tensor]:
    if bias is None:
        return None
    if not isinstance(bias, torch.Tensor):
        bias = torch.tensor([float(bias)], dtype=torch.float32, device="cuda")
    if bias.dtype != torch.float32:
        bias = bias.float()
    return bias.contiguous()


def forward_into(A, B, *, out, bias=None, act="none", with_bias=False, leaky_slope=0.01, save_z=False, z_out=None,
                 stream=None, math="fp32", alpha=1.0, trans_b=False, trans_a=False) -> None:
    """out = act(alpha * op(A) @ op(B) + bias); with save_z the pre-activation goes to z_out (which may be `out`
    itself only when act is 'none').  trans_a / trans_b read A as [K,M] / B as [N,K] in place (no copy).
    Allocates nothing."""
    if trans_a:
        K, M = _check_2d(A, "A")
    else:
        M, K = _check_2d(A, "A")
    if trans_b:
        N, K2 = _check_2d(B, "B")
    else:
        K2, N = _check_2d(B, "B")
    if K != K2:
        raise ValueError(f"K mismatch: A(K={K}) vs B(K={K2})")
    if _check_2d(out, "out") != (M, N):
        raise ValueError(f"out must be [{M},{N}]")
    dt = _dt(A, "A")
    if _dt(B, "B") != dt or _dt(out, "out") != dt:
        raise ValueError("A, B and out must share one dtype")
    if bias is not None and with_bias is False:
        raise ValueError("bias provided but with_bias=False")
    if with_bias and bias is None:
        raise ValueError("with_bias=True but bias is None")
    if save_z and z_out is None:
        raise ValueError("save_z=True requires z_out")
    if z_out is not None and _check_2d(z_out, "z_out") != (M, N):
        raise ValueError(f"z_out must be [{M},{N}]")

    device = _one_device(A, B, out, bias, z_out)
    lib = _lib.load_library()
    p = _lib.ParamsTyped()
    b = p.base
    b.M, b.N, b.K = M, N, K
    b.lda, b.ldb, b.ldd = A.stride(0), B.stride(0), out.stride(0)
    b.alpha, b.beta = float(alpha), 0.0
    b.use_C, b.has_bias = 0, 1 if bias is not None else 0
    b.bias_kind = _bias_kind(bias, M, N) if bias is not None else BIAS_SCALAR
    b.act_kind = _act_code(act)
    b.leaky_slope = float(leaky_slope)
    b.save_preact = 1 if (save_z and z_out is not None) else 0
    b.ldZ = z_out.stride(0) if z_out is not None else 0
    p.dtype = dt
    p.z_dtype = _dt(z_out, "z_out") if z_out is not None else dt
    p.math = _math_code(math)
    p.trans_b = 1 if trans_b else 0
    p.trans_a = 1 if trans_a else 0
    p.batch = 1
    ptrs = [A.data_ptr(), B.data_ptr(), out.data_ptr()]
    if bias is not None:
        ptrs.append(bias.data_ptr())
    if b.save_preact:
        ptrs.append(z_out.data_ptr())
    bufs = _lib.make_bufs(ptrs, p)
    with torch.cuda.device(device):
        _lib.check(lib.ge2_launch_gemm_bias_act_typed(bufs, len(bufs), _stream_ptr(stream, device)), "forward")


def forward(A, B, bias=None, *, act="none", with_bias=False, leaky_slope=0.01, stream=None, out=None, save_z=False,
            z_out=None, return_z=False, math="fp32", z_dtype=None
            ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Allocating wrapper: returns Y, or (Y, Z) with return_z.  A bias implies with_bias."""
    M, K = _check_2d(A, "A")
    _, N = _check_2d(B, "B")
    if bias is not None:
        with_bias = True
    bias_t = _prep_bias(bias, M, N) if with_bias else None
    if with_bias and bias_t is None:
        raise ValueError("with_bias=True but bias is None")
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype, device=A.device)
    want_z = save_z or return_z or z_out is not None
    if want_z and z_out is None:
        z_out = torch.empty((M, N), dtype=z_dtype or A.dtype, device=A.device)
    forward_into(A, B, out=out, bias=bias_t, act=act, with_bias=with_bias, leaky_slope=leaky_slope, save_z=want_z,
                 z_out=z_out, stream=stream, math=math)
    return (out, z_out) if return_z else out


def backward_into(A, B, gY, Z, *, act="none", with_bias=False, leaky_slope=0.01, C=None, gA_out=None, gB_out=None,
                  gC_out=None, gBias_out=None, stream=None, work_dZ=None, lt_workspace=None, math="fp32",
                  reuse_dZ=False) -> None:
    """(A, B, gY, Z) -> gA_out, gB_out, gBias_out.  `work_dZ` is the gZ scratch (at least M*N elements of the
    tensors' dtype); without it the scratch comes from the stream-ordered allocator, which a graph capture
    does not allow.  `lt_workspace` is accepted for signature compatibility and not used.  With reuse_dZ the
    scratch is taken to hold gZ already (from an earlier call with the same gY and Z) and only the GEMMs run."""
    M, K = _check_2d(A, "A")
    K2, N = _check_2d(B, "B")
    if K != K2:
        raise ValueError(f"K mismatch: A(K={K}) vs B(K={K2})")
    if _check_2d(gY, "gY") != (M, N) or _check_2d(Z, "Z") != (M, N):
        raise ValueError(f"gY/Z must be (M={M}, N={N})")
    dt = _dt(A, "A")
    for t, nm, shp in ((B, "B", (K, N)), (gY, "gY", (M, N)), (gA_out, "gA_out", (M, K)), (gB_out, "gB_out", (K, N)),
                       (gC_out, "gC_out", (M, N))):
        if t is None:
            continue
        if _check_2d(t, nm) != shp:
            raise ValueError(f"{nm} must be {shp}")
        if _dt(t, nm) != dt:
            raise ValueError(f"{nm} must have the dtype of A")
    if gC_out is not None and C is None:
        raise ValueError("gC_out requires C")
    kind = BIAS_SCALAR
    if gBias_out is not None:
        if gBias_out.dtype != torch.float32:
            raise ValueError("gBias_out must be float32")
        kind = _bias_kind(gBias_out, M, N)
        if kind == BIAS_PER_M and tuple(gBias_out.shape) in ((M,), (M, 1)) and M != N:
            # the reference binding refuses a per-row bias gradient (src/bindings/gemm_pybind.cpp:190-203)
            raise ValueError("gBias_out must be per-column (N,) / (1,N) or scalar")
    need = M * N * A.element_size()
    if work_dZ is not None and work_dZ.numel() * work_dZ.element_size() < need:
        raise ValueError(f"work_dZ too small: need {need} bytes")

    device = _one_device(A, B, gY, Z, C, gA_out, gB_out, gC_out, gBias_out, work_dZ)
    lib = _lib.load_library()
    p = _lib.ParamsBwdTyped()
    b = p.base
    b.M, b.N, b.K = M, N, K
    b.lda, b.ldb = A.stride(0), B.stride(0)
    b.ldc = C.stride(0) if C is not None else 0
    b.ldgY, b.ldZ = gY.stride(0), Z.stride(0)
    b.ldgA = gA_out.stride(0) if gA_out is not None else 0
    b.ldgB = gB_out.stride(0) if gB_out is not None else 0
    b.ldgC = gC_out.stride(0) if gC_out is not None else 0
    b.alpha = 1.0
    b.beta = 1.0 if (C is not None and gC_out is not None) else 0.0
    b.bias_kind = kind
    b.act_kind = _act_code(act)
    b.leaky_slope = float(leaky_slope)
    p.dtype, p.z_dtype, p.math = dt, _dt(Z, "Z"), _math_code(math)
    p.scratch_bytes = work_dZ.numel() * work_dZ.element_size() if work_dZ is not None else 0
    if reuse_dZ and work_dZ is None:
        raise ValueError("reuse_dZ needs work_dZ")
    p.reuse_gz = 1 if reuse_dZ else 0
    ptr = lambda t: t.data_ptr() if t is not None else 0   # noqa: E731
    bufs = _lib.make_bufs([ptr(A), ptr(B), ptr(C), ptr(gY), ptr(Z), ptr(gA_out), ptr(gB_out), ptr(gC_out),
                           ptr(gBias_out), ptr(work_dZ)], p)
    with torch.cuda.device(device):
        _lib.check(lib.ge2_launch_gemm_bias_act_bwd_typed(bufs, len(bufs), _stream_ptr(stream, device)), "backward")


def backward(A, B, gY, Z, *, act="none", with_bias=False, leaky_slope=0.01, C=None, want_gA=True, want_gB=True,
             want_gBias=False, stream=None, math="fp32") -> Dict[str, torch.Tensor]:
    """Allocating wrapper: returns {"gA", "gB", "gBias"} for the gradients asked for; gBias has shape (1, N)."""
    M, K = _check_2d(A, "A")
    _, N = _check_2d(B, "B")
    gA = torch.empty((M, K), dtype=A.dtype, device=A.device) if want_gA else None
    gB = torch.empty((K, N), dtype=A.dtype, device=A.device) if want_gB else None
    gBias = torch.empty((1, N), dtype=torch.float32, device=A.device) if (want_gBias or with_bias) else None
    gC = torch.empty((M, N), dtype=A.dtype, device=A.device) if C is not None else None
    backward_into(A, B, gY, Z, act=act, with_bias=with_bias, leaky_slope=leaky_slope, C=C, gA_out=gA, gB_out=gB,
                  gC_out=gC, gBias_out=gBias, stream=stream, math=math)
    out = {}
    if gA is not None:
        out["gA"] = gA
    if gB is not None:
        out["gB"] = gB
    if gBias is not None:
        out["gBias"] = gBias
    if gC is not None:
        out["gC"] = gC
    return out


def forward_batched(A, B, *, out, trans_b=False, alpha=1.0, bias=None, act="none", leaky_slope=0.01, stream=None,
                    math="fp32") -> None:
    """out[i] = act(alpha * A[i] @ op(B[i]) + bias) for tensors [..., rows, cols] whose leading dimensions
    flatten to one batch index with a constant stride.  A leading dimension of size 1 on A or B broadcasts.
    This is the shape of the reference's per-(batch, head) SDPA GEMM loops
    (backends/cuda/ops/sdpa/launcher.cu:185-222,236-270) in a single launch."""
    def flat(t, name):
        if t.dim() < 2 or t.stride(-1) != 1:
            raise ValueError(f"{name}: need [..., rows, cols] with unit inner stride")
        if t.dim() == 3:
            return t
        try:
            # a view or nothing: a silent copy would hide an allocation and, for `out`, lose the result
            return t.view(-1, t.shape[-2], t.shape[-1])
        except RuntimeError:
            raise ValueError(f"{name}: the leading dimensions do not flatten to one batch index with a constant "
                             "stride (pass a contiguous or 3-D tensor)") from None
    A3, B3, O3 = flat(A, "A"), flat(B, "B"), flat(out, "out")
    device = _one_device(A, B, out, bias if isinstance(bias, torch.Tensor) else None)
    batch = O3.shape[0]
    M, K = int(A3.shape[1]), int(A3.shape[2])
    N = int(B3.shape[1] if trans_b else B3.shape[2])
    if int(B3.shape[2] if trans_b else B3.shape[1]) != K or tuple(O3.shape[1:]) != (M, N):
        raise ValueError("shape mismatch")
    dt = _dt(A3, "A")
    if _dt(B3, "B") != dt or _dt(O3, "out") != dt:
        raise ValueError("A, B and out must share one dtype")

    def bstride(t3):
        if t3.shape[0] == 1:
            return 0
        if t3.shape[0] != batch:
            raise ValueError("batch mismatch")
        return t3.stride(0)

    bias_t = _prep_bias(bias, M, N)
    lib = _lib.load_library()
    p = _lib.ParamsTyped()
    b = p.base
    b.M, b.N, b.K = M, N, K
    b.lda, b.ldb, b.ldd = A3.stride(1), B3.stride(1), O3.stride(1)
    b.alpha, b.beta = float(alpha), 0.0
    b.has_bias = 1 if bias_t is not None else 0
    b.bias_kind = _bias_kind(bias_t, M, N) if bias_t is not None else BIAS_SCALAR
    b.act_kind = _act_code(act)
    b.leaky_slope = float(leaky_slope)
    p.dtype, p.z_dtype, p.math = dt, dt, _math_code(math)
    p.trans_b = 1 if trans_b else 0
    p.batch = batch
    p.strideA, p.strideB, p.strideD = bstride(A3), bstride(B3), O3.stride(0) if batch > 1 else M * N
    ptrs = [A3.data_ptr(), B3.data_ptr(), O3.data_ptr()] + ([bias_t.data_ptr()] if bias_t is not None else [])
    bufs = _lib.make_bufs(ptrs, p)
    with torch.cuda.device(device):
        _lib.check(lib.ge2_launch_gemm_bias_act_typed(bufs, len(bufs), _stream_ptr(stream, device)), "forward_batched")
