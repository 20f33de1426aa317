"""Pins the convolution oracle: its float64 forward / backward against torch.nn.functional.conv2d and autograd on the
CPU (an independent implementation), its fp32-exact forward against its own float64 form, and im2col / col2im
against each other (adjoint property).  No GPU."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

GEOMS = [
    # N, Cin, H, W, Cout, Kh, Kw, stride, padding, dilation
    (2, 3, 9, 11, 5, 3, 3, (1, 1), (1, 1), (1, 1)),
    (1, 4, 12, 10, 6, 3, 2, (2, 1), (0, 1), (1, 2)),
    (3, 8, 7, 7, 4, 1, 1, (1, 1), (0, 0), (1, 1)),
    (2, 2, 13, 13, 3, 5, 5, (2, 2), (2, 2), (1, 1)),
    (1, 1, 6, 6, 1, 3, 3, (1, 1), (0, 0), (2, 2)),
]


def _torch_ref(X, Wt, b, dY, act, stride, padding, dilation):
    x = torch.tensor(X, dtype=torch.float64, requires_grad=True)
    w = torch.tensor(Wt, dtype=torch.float64, requires_grad=True)
    bb = torch.tensor(b, dtype=torch.float64, requires_grad=True)
    z = F.conv2d(x, w, bb, stride=stride, padding=padding, dilation=dilation)
    y = {"none": lambda t: t, "relu": torch.relu, "tanh": torch.tanh, "sigmoid": torch.sigmoid,
         "gelu": lambda t: F.gelu(t, approximate="tanh")}[act](z)
    y.backward(torch.tensor(dY, dtype=torch.float64))
    return y.detach().numpy(), z.detach().numpy(), x.grad.numpy(), w.grad.numpy(), bb.grad.numpy()


@pytest.mark.parametrize("geom", GEOMS)
@pytest.mark.parametrize("act", ["none", "relu", "gelu", "tanh"])
def test_float64_oracle_matches_torch(conv_oracle, geom, act):
    N, Cin, H, W, Cout, Kh, Kw, st, pd, dl = geom
    X, Wt, b, dY = conv_oracle.conv_inputs(N, Cin, H, W, Cout, Kh, Kw, seed=1, stride=st, padding=pd, dilation=dl)
    Y, Z = conv_oracle.forward_f64(X, Wt, b, act=act, stride=st, padding=pd, dilation=dl)
    g = conv_oracle.backward_f64(X, Wt, dY, Z, act=act, stride=st, padding=pd, dilation=dl)
    y, z, gx, gw, gb = _torch_ref(X, Wt, b, dY, act, st, pd, dl)
    assert Y.shape == y.shape
    np.testing.assert_allclose(Z, z, rtol=1e-11, atol=1e-11)
    np.testing.assert_allclose(Y, y, rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(g["gX"], gx, rtol=1e-8, atol=1e-9)
    np.testing.assert_allclose(g["gW"], gw, rtol=1e-8, atol=1e-9)
    np.testing.assert_allclose(g["gB"], gb, rtol=1e-8, atol=1e-9)


@pytest.mark.parametrize("geom", GEOMS[:3])
def test_fp32_exact_forward_close_to_float64(conv_oracle, oracle, geom):
    N, Cin, H, W, Cout, Kh, Kw, st, pd, dl = geom
    X, Wt, b, _ = conv_oracle.conv_inputs(N, Cin, H, W, Cout, Kh, Kw, seed=2, stride=st, padding=pd, dilation=dl)
    Y32, Z32 = conv_oracle.forward_f32(X, Wt, b, act="gelu", stride=st, padding=pd, dilation=dl)
    Y64, Z64 = conv_oracle.forward_f64(X, Wt, b, act="gelu", stride=st, padding=pd, dilation=dl)
    assert Y32.dtype == np.float32 and Y32.shape == Y64.shape
    assert oracle.rel_fro(Z32, Z64) < 1e-6
    assert oracle.rel_fro(Y32, Y64) < 1e-6


def test_im2col_col2im_are_adjoint(conv_oracle):
    rng = np.random.default_rng(0)
    Cin, H, W, Kh, Kw, st, pd, dl = 3, 8, 9, 3, 2, (2, 1), (1, 0), (1, 2)
    x = rng.standard_normal((Cin, H, W))
    col = conv_oracle.im2col(x, Kh, Kw, st, pd, dl)
    u = rng.standard_normal(col.shape)
    lhs = float((col * u).sum())
    rhs = float((x * conv_oracle.col2im(u, Cin, H, W, Kh, Kw, st, pd, dl)).sum())
    assert abs(lhs - rhs) <= 1e-10 * max(1.0, abs(lhs))
