"""Dense layer over the fused GEMM op, mirroring the reference's
graph_executor_v2/python/graph_executor_v2/layers/dense_gemm.py:40-493: parameters `W:(in_dim, units)` and
`b:(1, units)`, an eager `call`/`backward` pair that caches the pre-activation Z, and the allocation-free
`forward_into`/`backward_into` pair used inside a captured training step.

Unlike the reference layer there is no silent fallback: a failure of the native op raises.
"""
from __future__ import annotations

import math as _math
from typing import List, Optional, Tuple

import torch

from . import ops_gemm


class Dense:
    def __init__(self, units: int, activation: Optional[str] = None, initializer: str = "he", use_bias: bool = True,
                 name: Optional[str] = None, leaky_slope: float = 0.01, dtype: torch.dtype = torch.float32,
                 math: str = "fp32", device: str = "cuda", seed: Optional[int] = None):
        self.units = int(units)
        self.activation = (activation or "none").lower()
        self.initializer = initializer
        self.use_bias = bool(use_bias)
        self.name = name
        self.leaky_slope = float(leaky_slope)
        self.dtype = dtype
        self.math = math
        self.device = device
        self.seed = seed
        self.built = False
        self.W: Optional[torch.Tensor] = None
        self.b: Optional[torch.Tensor] = None
        self.dW: Optional[torch.Tensor] = None
        self.db: Optional[torch.Tensor] = None
        self.last_input: Optional[torch.Tensor] = None
        self.last_z: Optional[torch.Tensor] = None

    # ---- parameters ----
    def _init_weights(self, in_dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
        gen = torch.Generator(device="cpu")
        if self.seed is not None:
            gen.manual_seed(self.seed)
        if self.initializer in ("he", "kaiming", "kaiming_uniform"):
            bound = _math.sqrt(6.0 / in_dim)
        elif self.initializer in ("xavier", "glorot"):
            bound = _math.sqrt(6.0 / (in_dim + self.units))
        elif self.initializer == "zeros":
            bound = 0.0
        else:
            raise ValueError(f"unknown initializer {self.initializer}")
        W = (torch.rand((in_dim, self.units), generator=gen, dtype=torch.float32) * 2.0 - 1.0) * bound
        b = torch.zeros((1, self.units), dtype=torch.float32)
        return W.to(self.device, self.dtype), b.to(self.device)

    def build(self, input_shape: Tuple[int, ...]) -> None:
        if len(input_shape) != 2:
            raise ValueError(f"Dense expects 2D input (batch, in_dim), got {input_shape}")
        self.W, self.b = self._init_weights(int(input_shape[1]))
        self.input_shape = tuple(input_shape)
        self.output_shape = (input_shape[0], self.units)
        self.built = True

    def compute_output_shape(self, input_shape):
        return (input_shape[0], self.units)

    def parameters(self):
        if self.use_bias:
            yield (self.W, self.dW, "W")
            yield (self.b, self.db, "b")
        else:
            yield (self.W, self.dW, "W")

    def grads(self) -> List[Optional[torch.Tensor]]:
        return [self.dW, self.db] if self.use_bias else [self.dW]

    def zero_grad(self) -> None:
        self.dW = None
        self.db = None

    # ---- eager ----
    def call(self, x: torch.Tensor) -> torch.Tensor:
        if not self.built:
            self.build(tuple(x.shape))
        self.last_input = x
        y, z = ops_gemm.forward(x, self.W, self.b if self.use_bias else None, act=self.activation,
                                leaky_slope=self.leaky_slope, return_z=True, math=self.math)
        self.last_z = z
        return y

    __call__ = call

    def backward(self, grad_output: torch.Tensor) -> torch.Tensor:
        if self.last_input is None or self.last_z is None:
            raise RuntimeError("backward called before forward")
        out = ops_gemm.backward(self.last_input, self.W, grad_output, self.last_z, act=self.activation,
                                with_bias=self.use_bias, leaky_slope=self.leaky_slope, want_gA=True, want_gB=True,
                                want_gBias=self.use_bias, math=self.math)
        self.dW = out["gB"]
        self.db = out.get("gBias")
        return out["gA"]

    # ---- allocation-free (graph capture) ----
    def forward_into(self, x: torch.Tensor, *, out: torch.Tensor, z_out: Optional[torch.Tensor] = None,
                     stream=None, work=None) -> None:
        if not self.built:
            raise RuntimeError("forward_into before build")
        ops_gemm.forward_into(x, self.W, out=out, bias=self.b if self.use_bias else None, act=self.activation,
                              with_bias=self.use_bias, leaky_slope=self.leaky_slope, save_z=z_out is not None,
                              z_out=z_out, stream=stream, math=self.math)
        self.last_input = x
        self.last_z = z_out

    def backward_into(self, grad_output: torch.Tensor, *, gA_out: Optional[torch.Tensor], gW_out: torch.Tensor,
                      gB_out: Optional[torch.Tensor] = None, work_dZ: Optional[torch.Tensor] = None,
                      lt_workspace=None, stream=None, x: Optional[torch.Tensor] = None,
                      z: Optional[torch.Tensor] = None) -> None:
        x = x if x is not None else self.last_input
        z = z if z is not None else self.last_z
        if x is None or z is None:
            raise RuntimeError("backward_into needs the forward input and pre-activation")
        ops_gemm.backward_into(x, self.W, grad_output, z, act=self.activation, with_bias=self.use_bias,
                               leaky_slope=self.leaky_slope, gA_out=gA_out, gB_out=gW_out,
                               gBias_out=gB_out if self.use_bias else None, stream=stream, work_dZ=work_dZ,
                               lt_workspace=lt_workspace, math=self.math)
        self.dW = gW_out
        self.db = gB_out
