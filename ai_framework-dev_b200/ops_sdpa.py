"""Scaled-dot-product attention forward on the fused kernel (csrc/sdpa_fused.cu) through the C ABI.

Counterpart of the reference's SDPA op (backends/cuda/ops/sdpa/api.hpp:8-26: attributes scale, causal, dropout_p;
Q [B,H,M,D], K / V [B,H,N,D], optional mask [B,1,M,N] as int8 / int32 (non-zero = masked) or float32 (additive)).
The scores and probabilities never reach HBM.  bfloat16 tensors, D = 64 or 128, dropout_p = 0.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .ops_gemm import _one_device, _stream_ptr

_MASK_KIND = {torch.float32: 1, torch.int8: 2, torch.int32: 3}


def forward(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *, mask: Optional[torch.Tensor] = None,
            causal: bool = False, scale: float = 0.0, dropout_p: float = 0.0, out: Optional[torch.Tensor] = None,
            lse: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """O = softmax(scale * Q K^T + mask) V per (batch, head); scale 0 means 1/sqrt(D).  `out` ([B,H,M,D]) and `lse`
    (float32 [B,H,M], receives every row's log-sum-exp) are optional pre-allocated outputs."""
    for t, nm in ((Q, "Q"), (K, "K"), (V, "V")):
        if not isinstance(t, torch.Tensor) or t.dim() != 4 or not t.is_contiguous():
            raise ValueError(f"{nm}: expected a contiguous [B,H,L,D] tensor")
    B, H, M, D = Q.shape
    N = K.shape[2]
    if K.shape != (B, H, N, D) or V.shape != (B, H, N, D):
        raise ValueError("K and V must be [B,H,N,D] with Q's B, H and D")
    if Q.dtype != torch.bfloat16 or K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise ValueError("Q, K and V must be bfloat16")
    if out is None:
        out = torch.empty_like(Q)
    if out.shape != Q.shape or out.dtype != Q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor like Q")
    if mask is not None:
        if tuple(mask.shape) != (B, 1, M, N) or mask.dtype not in _MASK_KIND or not mask.is_contiguous():
            raise ValueError("mask must be a contiguous [B,1,M,N] tensor of float32, int8 or int32")
    if lse is not None and (lse.dtype != torch.float32 or tuple(lse.shape) != (B, H, M) or not lse.is_contiguous()):
        raise ValueError("lse must be a contiguous float32 [B,H,M] tensor")
    device = _one_device(Q, K, V, out, mask, lse)
    p = _lib.ParamsSdpa()
    p.B, p.H, p.M, p.N, p.D = B, H, M, N, D
    p.dtype = _lib.DT_BF16
    p.scale, p.causal = float(scale), 1 if causal else 0
    p.mask_kind = _MASK_KIND[mask.dtype] if mask is not None else 0
    p.dropout_p = float(dropout_p)
    lib = _lib.load_library()
    with torch.cuda.device(device):
        rc = lib.ge2b_sdpa_forward(C.byref(p), Q.data_ptr(), K.data_ptr(), V.data_ptr(),
                                   mask.data_ptr() if mask is not None else None, out.data_ptr(),
                                   lse.data_ptr() if lse is not None else None, _stream_ptr(stream, device))
    _lib.check(rc, "sdpa_forward")
    return out
