"""2-D convolution (+ bias + activation) over the C ABI, mirroring the reference's Python op module
(graph_executor_v2/python/graph_executor_v2/ops/conv2d.py:89-520): `forward`, `backward` (allocating) and
`forward_into`, `backward_into` (outputs given by the caller).

NCHW tensors, OIHW weight, groups = 1.  Differences from the reference glue: device arrays are torch tensors; tensors
may be float32, bfloat16 or float16 (bias and its gradient float32); fp32 tensors take `math="fp32"` (exact, default)
or `math="tf32"`; no workspace object is needed (scratch is stream-ordered inside the library), and the bias gradient
is the sum over the whole batch.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .ops_gemm import _act_code, _dt, _math_code, _one_device, _stream_ptr


def _check_4d(t: torch.Tensor, name: str) -> Tuple[int, int, int, int]:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA torch.Tensor")
    if t.dim() != 4:
        raise ValueError(f"{name}: expected 4D, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: must be C-contiguous")
    return tuple(int(v) for v in t.shape)


def out_hw(H: int, W: int, KH: int, KW: int, stride=(1, 1), padding=(0, 0), dilation=(1, 1)) -> Tuple[int, int]:
    """Output size rule of conv2d/launcher.cu:137-138 (the reference's `_out_hw`, ops/conv2d.py:76-86)."""
    Ho = (H + 2 * padding[0] - dilation[0] * (KH - 1) - 1) // stride[0] + 1
    Wo = (W + 2 * padding[1] - dilation[1] * (KW - 1) - 1) // stride[1] + 1
    return Ho, Wo


def _params(X, W, stride, padding, dilation, groups, with_bias, act, leaky_slope, save_z, z_dtype, math):
    N, Cin, H, Win = _check_4d(X, "X")
    Cout, CinW, KH, KW = _check_4d(W, "W")
    if groups != 1:
        raise NotImplementedError("groups != 1 is not supported (the reference returns Unimplemented)")
    if CinW != Cin:
        raise ValueError(f"W.shape[1] ({CinW}) != Cin ({Cin})")
    if W.dtype != X.dtype:
        raise ValueError("X and W must share one dtype")
    p = _lib.ParamsConv2D()
    p.N, p.Cin, p.H, p.W, p.Cout, p.Kh, p.Kw = N, Cin, H, Win, Cout, KH, KW
    p.stride_h, p.stride_w = int(stride[0]), int(stride[1])
    p.pad_h, p.pad_w = int(padding[0]), int(padding[1])
    p.dil_h, p.dil_w = int(dilation[0]), int(dilation[1])
    p.groups = 1
    p.act_kind = _act_code(act)
    p.leaky_slope = float(leaky_slope)
    p.with_bias = 1 if with_bias else 0
    p.save_z = 1 if save_z else 0
    p.dtype = _dt(X, "X")
    p.z_dtype = z_dtype if z_dtype is not None else p.dtype
    p.math = _math_code(math)
    Ho, Wo = out_hw(H, Win, KH, KW, stride, padding, dilation)
    if Ho <= 0 or Wo <= 0:
        raise ValueError("empty output")
    return p, (N, Cout, Ho, Wo)


def _rc(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def forward_into(X, W, *, out, B=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, with_bias=False,
                 act="none", leaky_slope=0.01, save_z=False, Z_saved=None, stream=None, math="fp32") -> None:
    """out = act(conv2d(X, W) + B); with save_z the pre-activation goes to Z_saved (float32 or X's dtype)."""
    lib = _lib.load_library()
    zdt = _dt(Z_saved, "Z_saved") if (save_z and Z_saved is not None) else None
    p, oshape = _params(X, W, stride, padding, dilation, groups, with_bias and B is not None, act, leaky_slope,
                        save_z, zdt, math)
    if tuple(out.shape) != oshape or out.dtype != X.dtype or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous {X.dtype} tensor of shape {oshape}")
    if save_z:
        if Z_saved is None or tuple(Z_saved.shape) != oshape or not Z_saved.is_contiguous():
            raise ValueError(f"Z_saved must be a contiguous tensor of shape {oshape}")
    if p.with_bias and (B.dtype != torch.float32 or B.numel() != p.Cout):
        raise ValueError("B must be float32 with Cout elements")
    device = _one_device(X, W, out, B if p.with_bias else None, Z_saved if save_z else None)
    with torch.cuda.device(device):
        _rc(lib.ge2b_conv2d_forward(C.byref(p), X.data_ptr(), W.data_ptr(), B.data_ptr() if p.with_bias else None,
                                    out.data_ptr(), Z_saved.data_ptr() if save_z else None, _stream_ptr(stream, device)),
            "ge2b_conv2d_forward")


def forward(X, W, B=None, *, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, with_bias=False, act="none",
            leaky_slope=0.01, save_z=False, Z_saved=None, stream=None, out=None, math="fp32", z_dtype=None):
    """Allocating form.  Returns Y, or (Y, Z) when save_z is set."""
    N, Cin, H, Win = _check_4d(X, "X")
    Cout, _, KH, KW = _check_4d(W, "W")
    Ho, Wo = out_hw(H, Win, KH, KW, stride, padding, dilation)
    if out is None:
        out = torch.empty((N, Cout, Ho, Wo), device=X.device, dtype=X.dtype)
    if save_z and Z_saved is None:
        Z_saved = torch.empty((N, Cout, Ho, Wo), device=X.device, dtype=z_dtype or X.dtype)
    forward_into(X, W, out=out, B=B, stride=stride, padding=padding, dilation=dilation, groups=groups,
                 with_bias=with_bias, act=act, leaky_slope=leaky_slope, save_z=save_z, Z_saved=Z_saved, stream=stream,
                 math=math)
    return (out, Z_saved) if save_z else out


def backward_into(X, W, gY, Z, *, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, with_bias=False,
                  act="none", leaky_slope=0.01, gX_out=None, gW_out=None, gB_out=None, stream=None,
                  math="fp32") -> None:
    """(X, W, gY, Z) -> gX_out, gW_out, gB_out (each optional; overwritten)."""
    lib = _lib.load_library()
    p, oshape = _params(X, W, stride, padding, dilation, groups, with_bias, act, leaky_slope, False, _dt(Z, "Z"), math)
    for name, t in (("gY", gY), ("Z", Z)):
        if tuple(_check_4d(t, name)) != oshape:
            raise ValueError(f"{name} must have shape {oshape}")
    if gY.dtype != X.dtype:
        raise ValueError("gY must share X's dtype")
    if gX_out is not None and (gX_out.shape != X.shape or gX_out.dtype != X.dtype or not gX_out.is_contiguous()):
        raise ValueError("gX_out must match X")
    if gW_out is not None and (gW_out.shape != W.shape or gW_out.dtype != W.dtype or not gW_out.is_contiguous()):
        raise ValueError("gW_out must match W")
    if gB_out is not None and (gB_out.dtype != torch.float32 or gB_out.numel() != p.Cout):
        raise ValueError("gB_out must be float32 with Cout elements")
    ptr = lambda t: t.data_ptr() if t is not None else None   # noqa: E731
    device = _one_device(X, W, gY, Z, gX_out, gW_out, gB_out)
    with torch.cuda.device(device):
        _rc(lib.ge2b_conv2d_backward(C.byref(p), X.data_ptr(), W.data_ptr(), gY.data_ptr(), Z.data_ptr(), ptr(gW_out),
                                     ptr(gB_out), ptr(gX_out), _stream_ptr(stream, device)), "ge2b_conv2d_backward")


def backward(X, W, gY, Z, *, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, with_bias=False, act="none",
             leaky_slope=0.01, want_gX=True, want_gW=True, want_gB=False, stream=None,
             math="fp32") -> Dict[str, Optional[torch.Tensor]]:
    """Allocating form; returns {"gX", "gW", "gB"} like the reference."""
    gX = torch.empty_like(X) if want_gX else None
    gW = torch.empty_like(W) if want_gW else None
    gB = torch.empty(W.shape[0], device=X.device, dtype=torch.float32) if want_gB else None
    backward_into(X, W, gY, Z, stride=stride, padding=padding, dilation=dilation, groups=groups, with_bias=with_bias,
                  act=act, leaky_slope=leaky_slope, gX_out=gX, gW_out=gW, gB_out=gB, stream=stream, math=math)
    return {"gX": gX, "gW": gW, "gB": gB}
