"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's 2-D convolution
(graph_executor_v2/backends/cuda/ops/conv2d/launcher.cu:115-462, kernels.cu:12-167), on top of the dense oracle.

The reference computes, per image n: Col = im2col(X[n]) as [Ho*Wo, K] with k = (c*Kh + kh)*Kw + kw
(kernels.cu:12-44), rows = act(Col . W_KC + bias) with its fp32 GEMM (launcher.cu:186-225), and transposes the rows
to NCHW (launcher.cu:227-231).  `forward_f32` restates exactly that through dense_oracle.forward_f32 (one ascending-k
fmaf chain per output), so its Z is what the reference's Z is bit for bit; `forward_f64` / `backward_f64` are the
double-precision forms for tolerance checks.  The backward follows launcher.cu:236-462: gZ = dY * act'(Z),
dW[co][k] = sum over images and positions of gZ * Col, dCol = gZ . W, dX = col2im(dCol) (kernels.cu:46-88), with
one deliberate difference: dB sums gZ over the WHOLE batch (the reference zeroes its bias gradient for every image,
regemm_backward.cu:196, and so returns the last image's sum).

Parity pin: tests/test_oracle_conv2d.py checks these functions against torch.nn.functional.conv2d on CPU
(an independent implementation present in this image) and tests/test_gpu_conv2d.py checks the CUDA path against the
reference's own conv2d op compiled for sm_100a (oracle/_ref/libref_conv.so) when that library has been built.
Only tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this module.
"""
from __future__ import annotations

import numpy as np

from . import dense_oracle as D


def out_hw(H, W, Kh, Kw, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """launcher.cu:137-138"""
    Ho = (H + 2 * padding[0] - dilation[0] * (Kh - 1) - 1) // stride[0] + 1
    Wo = (W + 2 * padding[1] - dilation[1] * (Kw - 1) - 1) // stride[1] + 1
    return Ho, Wo


def im2col(x, Kh, Kw, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """x [Cin, H, W] -> Col [Ho*Wo, K], K = Cin*Kh*Kw, zero outside the image (kernels.cu:12-44)."""
    Cin, H, W = x.shape
    Ho, Wo = out_hw(H, W, Kh, Kw, stride, padding, dilation)
    col = np.zeros((Ho * Wo, Cin * Kh * Kw), dtype=x.dtype)
    ho = np.arange(Ho)[:, None]
    wo = np.arange(Wo)[None, :]
    for c in range(Cin):
        for kh in range(Kh):
            for kw in range(Kw):
                hi = ho * stride[0] - padding[0] + kh * dilation[0]
                wi = wo * stride[1] - padding[1] + kw * dilation[1]
                ok = (hi >= 0) & (hi < H) & (wi >= 0) & (wi < W)
                v = np.where(ok, x[c][np.clip(hi, 0, H - 1), np.clip(wi, 0, W - 1)], 0)
                col[:, (c * Kh + kh) * Kw + kw] = v.reshape(-1)
    return col


def col2im(dcol, Cin, H, W, Kh, Kw, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """dCol [Ho*Wo, K] -> dX [Cin, H, W], the adjoint of im2col (kernels.cu:46-88)."""
    Ho, Wo = out_hw(H, W, Kh, Kw, stride, padding, dilation)
    dx = np.zeros((Cin, H, W), dtype=dcol.dtype)
    for c in range(Cin):
        for kh in range(Kh):
            for kw in range(Kw):
                k = (c * Kh + kh) * Kw + kw
                patch = dcol[:, k].reshape(Ho, Wo)
                for ho in range(Ho):
                    hi = ho * stride[0] - padding[0] + kh * dilation[0]
                    if hi < 0 or hi >= H:
                        continue
                    wi = np.arange(Wo) * stride[1] - padding[1] + kw * dilation[1]
                    ok = (wi >= 0) & (wi < W)
                    np.add.at(dx[c, hi], wi[ok], patch[ho][ok])
    return dx


def forward_f32(X, Wt, bias=None, act="none", leaky=0.01, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """(Y, Z) float32 NCHW, per image exactly as the reference: im2col, fp32 GEMM + epilogue, transpose."""
    N, Cin, H, W = X.shape
    Cout, _, Kh, Kw = Wt.shape
    Ho, Wo = out_hw(H, W, Kh, Kw, stride, padding, dilation)
    W_KC = np.ascontiguousarray(Wt.reshape(Cout, -1).T.astype(np.float32))       # pack_w_oihw_to_KC, kernels.cu:121-139
    Y = np.empty((N, Cout, Ho, Wo), np.float32)
    Z = np.empty_like(Y)
    for n in range(N):
        col = im2col(X[n].astype(np.float32), Kh, Kw, stride, padding, dilation)
        y_rows, z_rows = D.forward_f32(col, W_KC, bias, act=act, leaky=leaky)
        Y[n] = y_rows.T.reshape(Cout, Ho, Wo)
        Z[n] = z_rows.T.reshape(Cout, Ho, Wo)
    return Y, Z


def forward_f64(X, Wt, bias=None, act="none", leaky=0.01, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    N, Cin, H, W = X.shape
    Cout, _, Kh, Kw = Wt.shape
    Ho, Wo = out_hw(H, W, Kh, Kw, stride, padding, dilation)
    Wm = Wt.reshape(Cout, -1).astype(np.float64)
    Z = np.empty((N, Cout, Ho, Wo), np.float64)
    for n in range(N):
        col = im2col(X[n].astype(np.float64), Kh, Kw, stride, padding, dilation)
        z = Wm @ col.T
        if bias is not None:
            z = z + np.asarray(bias, np.float64)[:, None]
        Z[n] = z.reshape(Cout, Ho, Wo)
    return D.act_f64(act, Z, leaky), Z


def backward_f64(X, Wt, dY, Z, act="none", leaky=0.01, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """dict(gZ, gW, gB, gX) in float64; gB is the sum over the whole batch."""
    N, Cin, H, W = X.shape
    Cout, _, Kh, Kw = Wt.shape
    Wm = Wt.reshape(Cout, -1).astype(np.float64)
    gZ = dY.astype(np.float64) * D.act_deriv_f64(act, Z.astype(np.float64), leaky)
    gW = np.zeros_like(Wm)
    gX = np.empty(X.shape, np.float64)
    for n in range(N):
        col = im2col(X[n].astype(np.float64), Kh, Kw, stride, padding, dilation)
        gz = gZ[n].reshape(Cout, -1)
        gW += gz @ col
        gX[n] = col2im((Wm.T @ gz).T, Cin, H, W, Kh, Kw, stride, padding, dilation)
    return {"gZ": gZ, "gW": gW.reshape(Wt.shape), "gB": gZ.sum(axis=(0, 2, 3)), "gX": gX}


def conv_inputs(N, Cin, H, W, Cout, Kh, Kw, seed=0, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """X, dY ~ N(0,1); weight ~ U(+-sqrt(6 / fan_in)); bias ~ U(-0.1, 0.1) -- float32."""
    rng = np.random.default_rng(seed)
    Ho, Wo = out_hw(H, W, Kh, Kw, stride, padding, dilation)
    X = rng.standard_normal((N, Cin, H, W), dtype=np.float32)
    lim = np.sqrt(6.0 / (Cin * Kh * Kw))
    Wt = rng.uniform(-lim, lim, (Cout, Cin, Kh, Kw)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, Cout).astype(np.float32)
    dY = rng.standard_normal((N, Cout, Ho, Wo), dtype=np.float32)
    return X, Wt, b, dY
