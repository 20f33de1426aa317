"""GPU parity tests of the convolution built on the dense-layer kernels.  Every call goes through the C ABI
(ge2b_conv2d_forward / _backward) and is compared with the CPU oracle (oracle/conv2d_oracle.py, pinned against
torch on the CPU by tests/test_oracle_conv2d.py) and, where it was built, with the reference's own conv2d op compiled
for sm_100a (oracle/_ref/libref_conv.so).

Tolerances:
  fp32 tensors, exact path   pre-activation Z bit-identical to the oracle's fp32 restatement and to the reference op;
                             Y identical for none / relu, within 1e-6 relative otherwise; gradients <= 1e-5 relative
                             Frobenius error against float64
  bf16 / TF32 tensor cores   relative Frobenius error <= 2e-2 against float64 on the rounded inputs
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
FRO_TOL = 2e-2
ACT_CODE = {"none": 0, "relu": 1, "leaky_relu": 2, "gelu": 3, "sigmoid": 4, "tanh": 5}

GEOMS = {
    # name: N, Cin, H, W, Cout, Kh, Kw, stride, padding, dilation
    "3x3_same":      (3, 8, 14, 14, 16, 3, 3, (1, 1), (1, 1), (1, 1)),
    "3x3_stride2":   (2, 5, 17, 15, 7, 3, 3, (2, 2), (1, 1), (1, 1)),
    "5x3_dilated":   (2, 4, 16, 18, 6, 5, 3, (1, 2), (2, 1), (1, 2)),
    "1x1_pointwise": (4, 16, 12, 12, 24, 1, 1, (1, 1), (0, 0), (1, 1)),
    "1x1_odd_hw":    (2, 8, 7, 9, 5, 1, 1, (1, 1), (0, 0), (1, 1)),
    "7x7_stem":      (2, 3, 32, 32, 16, 7, 7, (2, 2), (3, 3), (1, 1)),
    "wide":          (2, 64, 20, 20, 96, 3, 3, (1, 1), (1, 1), (1, 1)),
}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.detach().float().cpu().numpy()


@pytest.fixture(autouse=True)
def _status_clean(lib):
    yield
    torch.cuda.synchronize()
    assert lib.ge2b_device_status(1) == 0, "a bounded wait inside a kernel timed out"


def _kw(g):
    return dict(stride=g[7], padding=g[8], dilation=g[9])


# --------------------------------------------------------------------------- fp32, exact path
@pytest.mark.parametrize("act", ["none", "relu", "gelu", "tanh"])
@pytest.mark.parametrize("name", sorted(GEOMS))
def test_fp32_forward_bit_exact_preactivation(pkg, lib, oracle, conv_oracle, name, act):
    g = GEOMS[name]
    X, Wt, b, _ = conv_oracle.conv_inputs(*g[:7], seed=3, **_kw(g))
    Y, Z = pkg.ops_conv2d.forward(dev(X), dev(Wt), dev(b), with_bias=True, act=act, save_z=True, **_kw(g))
    torch.cuda.synchronize()
    Y32, Z32 = conv_oracle.forward_f32(X, Wt, b, act=act, **_kw(g))
    assert np.array_equal(host(Z), Z32)
    if act in ("none", "relu"):
        assert np.array_equal(host(Y), Y32)
    else:
        assert oracle.rel_fro(host(Y), Y32) <= 1e-6


@pytest.mark.parametrize("act", ["none", "gelu", "sigmoid"])
@pytest.mark.parametrize("name", sorted(GEOMS))
def test_fp32_backward_vs_float64(pkg, lib, oracle, conv_oracle, name, act):
    g = GEOMS[name]
    X, Wt, b, dY = conv_oracle.conv_inputs(*g[:7], seed=4, **_kw(g))
    _, Z64 = conv_oracle.forward_f64(X, Wt, b, act=act, **_kw(g))
    Z = Z64.astype(np.float32)
    out = pkg.ops_conv2d.backward(dev(X), dev(Wt), dev(dY), dev(Z), with_bias=True, act=act, want_gB=True, **_kw(g))
    torch.cuda.synchronize()
    ref = conv_oracle.backward_f64(X, Wt, dY, Z, act=act, **_kw(g))
    assert oracle.rel_fro(host(out["gX"]), ref["gX"]) <= 1e-5
    assert oracle.rel_fro(host(out["gW"]), ref["gW"]) <= 1e-5
    assert oracle.rel_fro(host(out["gB"]), ref["gB"]) <= 1e-5


def test_optional_outputs_and_no_bias(pkg, lib, oracle, conv_oracle):
    g = GEOMS["3x3_stride2"]
    X, Wt, _, dY = conv_oracle.conv_inputs(*g[:7], seed=5, **_kw(g))
    Y = pkg.ops_conv2d.forward(dev(X), dev(Wt), None, act="relu", **_kw(g))
    Y64, Z64 = conv_oracle.forward_f64(X, Wt, None, act="relu", **_kw(g))
    assert oracle.rel_fro(host(Y), Y64) <= 1e-6
    Z = dev(Z64.astype(np.float32))
    ref = conv_oracle.backward_f64(X, Wt, dY, Z64.astype(np.float32), act="relu", **_kw(g))
    only_w = pkg.ops_conv2d.backward(dev(X), dev(Wt), dev(dY), Z, act="relu", want_gX=False, **_kw(g))
    assert only_w["gX"] is None and only_w["gB"] is None
    assert oracle.rel_fro(host(only_w["gW"]), ref["gW"]) <= 1e-5
    only_x = pkg.ops_conv2d.backward(dev(X), dev(Wt), dev(dY), Z, act="relu", want_gW=False, **_kw(g))
    assert only_x["gW"] is None
    assert oracle.rel_fro(host(only_x["gX"]), ref["gX"]) <= 1e-5


def test_argument_errors(pkg, lib):
    X = torch.zeros(1, 3, 8, 8, device="cuda")
    W = torch.zeros(4, 3, 3, 3, device="cuda")
    with pytest.raises(NotImplementedError):
        pkg.ops_conv2d.forward(X, W, groups=3)
    with pytest.raises(ValueError):
        pkg.ops_conv2d.forward(X, torch.zeros(4, 2, 3, 3, device="cuda"))
    with pytest.raises(ValueError):
        pkg.ops_conv2d.forward(X, torch.zeros(4, 3, 9, 9, device="cuda"))       # empty output
    p = pkg._lib.ParamsConv2D()
    assert lib.ge2b_conv2d_forward(C.byref(p), None, None, None, None, None, None) == -1
    p.N, p.Cin, p.H, p.W, p.Cout, p.Kh, p.Kw = 1, 3, 8, 8, 4, 3, 3
    p.stride_h = p.stride_w = p.dil_h = p.dil_w = 1
    p.groups = 2
    Y = torch.zeros(1, 4, 6, 6, device="cuda")
    assert lib.ge2b_conv2d_forward(C.byref(p), X.data_ptr(), W.data_ptr(), None, Y.data_ptr(), None, None) == -99


# --------------------------------------------------------------------------- tensor-core paths
@pytest.mark.parametrize("dtype,math", [(torch.bfloat16, "fp32"), (torch.float32, "tf32")])
@pytest.mark.parametrize("name", ["3x3_same", "1x1_pointwise", "7x7_stem", "wide"])
def test_tensor_core_forward_backward(pkg, lib, oracle, conv_oracle, name, dtype, math):
    g = GEOMS[name]
    X, Wt, b, dY = conv_oracle.conv_inputs(*g[:7], seed=6, **_kw(g))
    if dtype == torch.bfloat16:
        X, Wt, dY = (oracle.bf16_round(a) for a in (X, Wt, dY))
    tX, tW, tdY = dev(X, dtype), dev(Wt, dtype), dev(dY, dtype)
    Y, Z = pkg.ops_conv2d.forward(tX, tW, dev(b), with_bias=True, act="gelu", save_z=True, math=math,
                                  z_dtype=torch.float32, **_kw(g))
    out = pkg.ops_conv2d.backward(tX, tW, tdY, Z, with_bias=True, act="gelu", want_gB=True, math=math, **_kw(g))
    torch.cuda.synchronize()
    Y64, Z64 = conv_oracle.forward_f64(X, Wt, b, act="gelu", **_kw(g))
    ref = conv_oracle.backward_f64(X, Wt, dY, host(Z), act="gelu", **_kw(g))
    errs = {"Y": oracle.rel_fro(host(Y), Y64), "Z": oracle.rel_fro(host(Z), Z64),
            "gX": oracle.rel_fro(host(out["gX"]), ref["gX"]), "gW": oracle.rel_fro(host(out["gW"]), ref["gW"]),
            "gB": oracle.rel_fro(host(out["gB"]), ref["gB"])}
    assert all(e <= FRO_TOL for e in errs.values()), errs


def test_bf16_layer_sized_case(pkg, lib, oracle, conv_oracle):
    """A ResNet-like layer (N=8, 64 -> 64 channels, 56 x 56, 3 x 3): the weight gradient's reduction runs over
    8 * 3136 positions in one launch; float64 reference on sampled output channels."""
    N, Cin, H, W, Cout, Kh, Kw = 8, 64, 56, 56, 64, 3, 3
    kw = dict(stride=(1, 1), padding=(1, 1), dilation=(1, 1))
    X, Wt, b, dY = conv_oracle.conv_inputs(N, Cin, H, W, Cout, Kh, Kw, seed=7, **kw)
    X, Wt, dY = (oracle.bf16_round(a) for a in (X, Wt, dY))
    tX, tW, tdY = dev(X, torch.bfloat16), dev(Wt, torch.bfloat16), dev(dY, torch.bfloat16)
    Y, Z = pkg.ops_conv2d.forward(tX, tW, dev(b), with_bias=True, act="relu", save_z=True, **kw)
    assert lib.ge2b_last_route() == 2
    out = pkg.ops_conv2d.backward(tX, tW, tdY, Z, with_bias=True, act="relu", want_gB=True, **kw)
    torch.cuda.synchronize()
    xt = torch.from_numpy(X).double().requires_grad_(True)
    wt = torch.from_numpy(Wt).double().requires_grad_(True)
    z = torch.nn.functional.conv2d(xt, wt, torch.from_numpy(b).double(), padding=1)
    assert oracle.rel_fro(host(Z), z.detach().numpy()) <= FRO_TOL
    gz = torch.from_numpy(dY).double() * (Z.double().cpu() > 0)
    z.backward(gz)
    assert oracle.rel_fro(host(out["gX"]), xt.grad.numpy()) <= FRO_TOL
    assert oracle.rel_fro(host(out["gW"]), wt.grad.numpy()) <= FRO_TOL
    assert oracle.rel_fro(host(out["gB"]), gz.sum(dim=(0, 2, 3)).numpy()) <= FRO_TOL


# --------------------------------------------------------------------------- implicit GEMM against the other routes
IMPLICIT_GEOMS = {
    # rows that are multiples of 8 wide take the aligned 16-byte gather, the others the element-wise one
    "3x3_w16":          (2, 8, 16, 16, 16, 3, 3, (1, 1), (1, 1), (1, 1)),
    "5x5_w24_pad2":     (2, 6, 24, 24, 10, 5, 5, (1, 1), (2, 2), (1, 1)),
    "3x3_w16_dil2":     (2, 4, 16, 16, 8, 3, 3, (1, 1), (2, 2), (2, 2)),
    "3x3_w32_valid":    (1, 5, 12, 32, 9, 3, 3, (1, 1), (0, 0), (1, 1)),      # Wo = 30: general gather on aligned input
    "4x2_w8_even_taps": (3, 3, 9, 8, 4, 4, 2, (1, 1), (2, 1), (1, 1)),
    "3x3_cout_300":     (1, 16, 16, 16, 300, 3, 3, (1, 1), (1, 1), (1, 1)),   # two channel tiles, ragged second one
    "3x3_cout_100":     (2, 12, 10, 16, 100, 3, 3, (1, 1), (1, 1), (1, 1)),   # 128-wide channel tile
    # reductions longer than the operand ring of the 256- and 128-channel tiles (4 and 7 stages): the ring wraps
    "3x3_deep_cout_300": (2, 64, 8, 16, 300, 3, 3, (1, 1), (1, 1), (1, 1)),
    "3x3_deep_cout_100": (4, 64, 16, 16, 100, 3, 3, (1, 1), (1, 1), (1, 1)),
    "3x3_deep_w12":      (3, 72, 10, 12, 130, 3, 3, (1, 1), (1, 1), (1, 1)),   # the same with the element-wise gather
    # several 64-channel blocks per tile (the patch is refilled per block), odd widths for the narrower fill loads
    "3x3_cin_160_w28":   (2, 160, 9, 28, 48, 3, 3, (1, 1), (1, 1), (1, 1)),
    "3x3_cin_128_w14":   (3, 128, 14, 14, 64, 3, 3, (1, 1), (1, 1), (1, 1)),
    "3x3_cin_64_w7":     (5, 64, 7, 7, 96, 3, 3, (1, 1), (1, 1), (1, 1)),
    "5x5_cin_96_pad1":   (2, 96, 13, 20, 40, 5, 5, (1, 1), (1, 1), (1, 1)),
    # strided layers with enough output channels for the per-phase input-gradient launches (one unit-stride
    # correlation per residue of the input pixel modulo the stride); 1x1 / stride 2 leaves three of four phases empty
    "3x3_s2_cout_64":    (2, 24, 18, 20, 64, 3, 3, (2, 2), (1, 1), (1, 1)),
    "3x3_s2_odd_hw":     (2, 16, 17, 15, 40, 3, 3, (2, 2), (1, 1), (1, 1)),
    "5x5_s3x2_dil":      (1, 16, 23, 26, 64, 5, 5, (3, 2), (2, 2), (1, 2)),
    "1x1_s2":            (2, 32, 12, 12, 64, 1, 1, (2, 2), (0, 0), (1, 1)),
    "2x2_s2_tiles":      (2, 16, 12, 16, 32, 2, 2, (2, 2), (0, 0), (1, 1)),
    "3x3_stride2":      GEOMS["3x3_stride2"],
    "5x3_dilated":      GEOMS["5x3_dilated"],
    "7x7_stem":         GEOMS["7x7_stem"],
    "wide":             GEOMS["wide"],
}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", sorted(IMPLICIT_GEOMS))
def test_implicit_gemm_routes(pkg, lib, oracle, conv_oracle, monkeypatch, name, dtype):
    """Forward (Y, Z), input gradient and weight gradient through every route: chosen by shape (the shared-memory
    patch kernel for unit-stride passes), the gathering kernels with their aligned gather where it applies, the same
    with the element-wise gather everywhere, and the column matrix in memory.  The two gathers feed the same
    arithmetic (bit-identical results), the other routes sum in another order (close), and all of them stay inside the
    bf16 / f16 bound against float64."""
    g = IMPLICIT_GEOMS[name]
    X, Wt, b, dY = conv_oracle.conv_inputs(*g[:7], seed=11, **_kw(g))
    if dtype == torch.bfloat16:
        X, Wt, dY = (oracle.bf16_round(a) for a in (X, Wt, dY))
    else:
        X, Wt, dY = (a.astype(np.float16).astype(np.float32) for a in (X, Wt, dY))
    tX, tW, tdY = dev(X, dtype), dev(Wt, dtype), dev(dY, dtype)
    Y64, Z64 = conv_oracle.forward_f64(X, Wt, b, act="tanh", **_kw(g))
    got = {}
    for route in ("auto", "gather", "general", "explicit"):
        if route == "auto":
            monkeypatch.delenv("GE2B_CONV", raising=False)
        else:
            monkeypatch.setenv("GE2B_CONV", route)
        Y, Z = pkg.ops_conv2d.forward(tX, tW, dev(b), with_bias=True, act="tanh", save_z=True, z_dtype=torch.float32,
                                      **_kw(g))
        out = pkg.ops_conv2d.backward(tX, tW, tdY, Z, with_bias=True, act="tanh", want_gB=True, **_kw(g))
        torch.cuda.synchronize()
        assert lib.ge2b_device_status(1) == 0
        got[route] = (Y, Z, out["gX"], out["gW"])
        ref = conv_oracle.backward_f64(X, Wt, dY, host(Z), act="tanh", **_kw(g))
        errs = {"Y": oracle.rel_fro(host(Y), Y64), "Z": oracle.rel_fro(host(Z), Z64),
                "gX": oracle.rel_fro(host(out["gX"]), ref["gX"]), "gW": oracle.rel_fro(host(out["gW"]), ref["gW"])}
        assert all(e <= FRO_TOL for e in errs.values()), (route, errs)
        # element-wise: fp32 accumulation of K products of 16-bit operands, then one rounding of Y
        K = g[1] * g[5] * g[6]
        eps = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -9     # 16-bit epilogues use tanh.approx
        assert float(np.abs(host(Z) - Z64).max()) <= 1e-5 * K + 1e-6, route
        assert float(np.abs(host(Y) - Y64).max()) <= eps + 1e-5 * K, route
    for a, c in zip(got["gather"], got["general"]):
        assert torch.equal(a, c)
    for other in ("auto", "gather"):
        for a, c in zip(got[other], got["explicit"]):
            assert float((a.float() - c.float()).abs().max()) <= 2e-2 * max(1.0, float(c.float().abs().max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", ["3x3_w16", "3x3_cin_160_w28", "3x3_cin_128_w14", "3x3_cin_64_w7", "5x5_cin_96_pad1",
                                  "3x3_deep_cout_300", "3x3_w32_valid"])
def test_patch_kernel_with_16bit_preactivation(pkg, lib, oracle, conv_oracle, monkeypatch, name, dtype):
    """Z saved in the tensors' own 16-bit type: on even widths the patch kernel's epilogue writes two positions per
    32-bit store (neighbouring lanes swap one value per channel pair), on odd widths one element per store.  Y and Z
    against float64 and, element for element, against the column-matrix route."""
    g = IMPLICIT_GEOMS[name]
    X, Wt, b, dY = conv_oracle.conv_inputs(*g[:7], seed=23, **_kw(g))
    rnd = oracle.bf16_round if dtype == torch.bfloat16 else (lambda a: a.astype(np.float16).astype(np.float32))
    X, Wt = rnd(X), rnd(Wt)
    tX, tW = dev(X, dtype), dev(Wt, dtype)
    Y64, Z64 = conv_oracle.forward_f64(X, Wt, b, act="leaky_relu", **_kw(g))
    eps = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    got = {}
    for route in ("auto", "explicit"):
        if route == "auto":
            monkeypatch.delenv("GE2B_CONV", raising=False)
        else:
            monkeypatch.setenv("GE2B_CONV", route)
        for with_bias in (True, False):
            Y, Z = pkg.ops_conv2d.forward(tX, tW, dev(b) if with_bias else None, with_bias=with_bias, act="leaky_relu",
                                          save_z=True, **_kw(g))
            torch.cuda.synchronize()
            assert Z.dtype == dtype
            if with_bias:
                got[route] = (Y, Z)
                scale = float(np.abs(Z64).max())
                assert float(np.abs(host(Z) - Z64).max()) <= eps * scale + 1e-5 * g[1] * g[5] * g[6], route
                assert float(np.abs(host(Y) - Y64).max()) <= eps * scale + 1e-5 * g[1] * g[5] * g[6], route
            else:
                Y0, Z0 = conv_oracle.forward_f64(X, Wt, np.zeros_like(b), act="leaky_relu", **_kw(g))
                assert oracle.rel_fro(host(Z), Z0) <= FRO_TOL and oracle.rel_fro(host(Y), Y0) <= FRO_TOL
    for a, c in zip(got["auto"], got["explicit"]):
        assert float((a.float() - c.float()).abs().max()) <= 2 * eps * max(1.0, float(c.float().abs().max()))


def test_conv_routes_on_random_geometries(pkg, lib, monkeypatch):
    """Seeded random layers (channels 16..130 -> 8..300, planes 5..36 x 5..40, kernels up to 5 x 5, strides up to 3,
    padding up to 2, dilation up to 2, bf16 / f16, Z in 16 or 32 bits): the route chosen by shape against the
    column-matrix route on Y, Z, gX, gW and gB, and Z against torch's fp32 convolution of the same 16-bit inputs."""
    import random
    rng = random.Random(7)
    done = 0
    for trial in range(60):
        N = rng.randint(1, 3)
        Cin = rng.choice([16, 17, 24, 32, 48, 64, 70, 128, 130])
        Cout = rng.choice([8, 16, 33, 64, 65, 100, 128, 200, 300])
        H, W = rng.randint(5, 36), rng.choice([5, 7, 8, 9, 12, 14, 16, 20, 24, 28, 31, 32, 40])
        Kh, Kw = rng.randint(1, 5), rng.randint(1, 5)
        st = (rng.randint(1, 3), rng.randint(1, 3)) if rng.random() < 0.4 else (1, 1)
        kw = dict(stride=st, padding=(rng.randint(0, 2), rng.randint(0, 2)), dilation=(rng.randint(1, 2), rng.randint(1, 2)))
        Ho, Wo = pkg.ops_conv2d.out_hw(H, W, Kh, Kw, **kw)
        if Ho < 1 or Wo < 1:
            continue
        dt = rng.choice([torch.bfloat16, torch.float16])
        act, zdt = rng.choice(["none", "relu", "tanh"]), rng.choice([dt, torch.float32])
        g = torch.Generator(device="cuda").manual_seed(trial)
        X = torch.randn((N, Cin, H, W), device="cuda", generator=g).to(dt)
        Wt = (torch.randn((Cout, Cin, Kh, Kw), device="cuda", generator=g) / (Cin * Kh * Kw) ** 0.5).to(dt)
        b = torch.randn(Cout, device="cuda", generator=g)
        dY = torch.randn((N, Cout, Ho, Wo), device="cuda", generator=g).to(dt)
        res = {}
        for route in ("auto", "explicit"):
            if route == "auto":
                monkeypatch.delenv("GE2B_CONV", raising=False)
            else:
                monkeypatch.setenv("GE2B_CONV", route)
            Y, Z = pkg.ops_conv2d.forward(X, Wt, b, with_bias=True, act=act, save_z=True, z_dtype=zdt, **kw)
            out = pkg.ops_conv2d.backward(X, Wt, dY, Z, with_bias=True, act=act, want_gB=True, **kw)
            torch.cuda.synchronize()
            res[route] = [t.float() for t in (Y, Z, out["gX"], out["gW"], out["gB"])]
        geom = (trial, N, Cin, H, W, Cout, Kh, Kw, kw, str(dt), act, str(zdt))
        for name, a, c in zip(("Y", "Z", "gX", "gW", "gB"), res["auto"], res["explicit"]):
            assert float((a - c).abs().max()) <= 3e-2 * max(1.0, float(c.abs().max())), (name, geom)
        ref = torch.nn.functional.conv2d(X.float(), Wt.float(), b, **kw)
        assert float((res["auto"][1] - ref).abs().max()) <= 2e-2 * max(1.0, float(ref.abs().max())), geom
        done += 1
    assert done >= 40
    assert lib.ge2b_device_status(1) == 0


def test_implicit_gemm_is_the_default_route_and_moves_no_column_matrix(pkg, lib, monkeypatch):
    """On a ResNet-sized layer the default forward is the weight re-layout plus ONE convolution launch (the
    column-matrix route allocates and fills K x N x HWo elements first)."""
    monkeypatch.delenv("GE2B_CONV", raising=False)
    g = torch.Generator(device="cuda").manual_seed(5)
    X = torch.randn((4, 64, 56, 56), device="cuda", generator=g).bfloat16()
    W = (torch.randn((64, 64, 3, 3), device="cuda", generator=g) / 24).bfloat16()
    b = torch.randn(64, device="cuda", generator=g)
    pkg.ops_conv2d.forward(X, W, b, with_bias=True, act="relu", padding=(1, 1))
    torch.cuda.synchronize()
    before = lib.ge2b_launches_total()
    Y = pkg.ops_conv2d.forward(X, W, b, with_bias=True, act="relu", padding=(1, 1))
    torch.cuda.synchronize()
    assert lib.ge2b_launches_total() - before == 2
    assert lib.ge2b_last_route() == 2
    want = torch.nn.functional.conv2d(X.float(), W.float(), b, padding=1).relu()
    assert float((Y.float() - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())


# --------------------------------------------------------------------------- against the reference's own GPU op
def _ref_conv():
    path = ROOT / "oracle" / "_ref" / "libref_conv.so"
    if not path.exists():
        pytest.skip("oracle/_ref/libref_conv.so not built (needs the reference tree at build time)")
    lib = C.CDLL(str(path))
    ints = [C.c_int] * 13
    lib.ref_conv_forward.argtypes = [C.c_void_p] * 5 + ints + [C.c_int, C.c_float, C.c_void_p]
    lib.ref_conv_forward.restype = C.c_int
    lib.ref_conv_backward.argtypes = [C.c_void_p] * 7 + ints + [C.c_int, C.c_float, C.c_void_p]
    lib.ref_conv_backward.restype = C.c_int
    return lib


@pytest.mark.parametrize("act", ["relu", "gelu"])
@pytest.mark.parametrize("name", ["3x3_same", "3x3_stride2", "5x3_dilated", "1x1_pointwise"])
def test_fp32_path_against_reference_gpu_op(pkg, lib, oracle, conv_oracle, name, act):
    ref = _ref_conv()
    g = GEOMS[name]
    N, Cin, H, W, Cout, Kh, Kw, st, pd, dl = g
    X, Wt, b, dY = conv_oracle.conv_inputs(*g[:7], seed=8, **_kw(g))
    tX, tW, tb, tdY = dev(X), dev(Wt), dev(b), dev(dY)
    Y, Z = pkg.ops_conv2d.forward(tX, tW, tb, with_bias=True, act=act, save_z=True, **_kw(g))
    rY, rZ = torch.empty_like(Y), torch.empty_like(Z)
    geom = (N, Cin, H, W, Cout, Kh, Kw, st[0], st[1], pd[0], pd[1], dl[0], dl[1])
    assert ref.ref_conv_forward(tX.data_ptr(), tW.data_ptr(), tb.data_ptr(), rY.data_ptr(), rZ.data_ptr(), *geom,
                                ACT_CODE[act], 0.01, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(Z, rZ)                      # same fmaf chain per output
    assert oracle.rel_fro(host(Y), host(rY)) <= 1e-6

    out = pkg.ops_conv2d.backward(tX, tW, tdY, Z, with_bias=True, act=act, want_gB=True, **_kw(g))
    rdW, rdX, rdB = torch.empty_like(tW), torch.empty_like(tX), torch.empty(Cout, device="cuda")
    assert ref.ref_conv_backward(tX.data_ptr(), tW.data_ptr(), tdY.data_ptr(), rZ.data_ptr(), rdW.data_ptr(),
                                 rdB.data_ptr(), rdX.data_ptr(), *geom, ACT_CODE[act], 0.01, None) == 0
    torch.cuda.synchronize()
    assert oracle.rel_fro(host(out["gX"]), host(rdX)) <= 3e-4
    # The reference's weight gradient is not comparable: its launcher lets GemmCudaBackward write gA into the very
    # buffer that holds A = im2col(X) (conv2d/launcher.cu:404-405), and the backward computes gA before gB
    # (regemm_backward.cu:270-291), so its gB = gA^T . gZ.  Check that this is indeed what it returns, and check this
    # library's dW against float64 instead.
    full = conv_oracle.backward_f64(X, Wt, dY, host(Z), act=act, **_kw(g))
    assert oracle.rel_fro(host(out["gW"]), full["gW"]) <= 1e-5
    Wm = Wt.reshape(Cout, -1).astype(np.float64)
    aliased = np.zeros_like(Wm)
    for n in range(N):
        gz = full["gZ"][n].reshape(Cout, -1)                  # [Cout, HWo]
        aliased += gz @ (gz.T @ Wm)                           # gZ . gA_rows, gA_rows = gZ^T . W
    assert oracle.rel_fro(host(rdW).reshape(Cout, -1), aliased) <= 3e-4
    # The reference's bias gradient holds the last image only (its per-image backward zeroes it each time), so the
    # comparable quantity is the last image's share of the sum.
    gz_last = conv_oracle.backward_f64(X[-1:], Wt, dY[-1:], host(Z)[-1:], act=act, **_kw(g))["gB"]
    assert oracle.rel_fro(host(rdB), gz_last) <= 3e-4
    assert oracle.rel_fro(host(out["gB"]), full["gB"]) <= 1e-5


# --------------------------------------------------------------------------- the reference's own binding, linked here
def test_reference_conv2d_binding_runs_on_this_library(pkg, lib, oracle, conv_oracle):
    dropin = ROOT / "oracle" / "_ref" / "dropin"
    if not list((dropin / "graph_executor_v2" / "ops").glob("_ops_conv2d*")):
        pytest.skip("oracle/_ref/dropin/_ops_conv2d not built (needs the reference tree at build time)")
    sys.path.insert(0, str(dropin))
    try:
        from graph_executor_v2.ops import _ops_common as c, _ops_conv2d as cv  # noqa: F401
    finally:
        sys.path.remove(str(dropin))
    g = GEOMS["3x3_same"]
    X, Wt, b, dY = conv_oracle.conv_inputs(*g[:7], seed=9, **_kw(g))
    tX, tW, tb, tdY = dev(X), dev(Wt), dev(b), dev(dY)
    N, Cin, H, W, Cout, Kh, Kw = g[:7]
    Ho, Wo = conv_oracle.out_hw(H, W, Kh, Kw, **_kw(g))
    Y = torch.empty(N, Cout, Ho, Wo, device="cuda")
    Z = torch.empty_like(Y)
    at = cv.Conv2DAttrs()
    at.pad_h = at.pad_w = 1
    at.with_bias = True
    at.act = cv.ActKind.ReLU
    at.save_z = True
    dummy = torch.zeros(64, device="cuda").data_ptr()     # the binding insists on non-null workspaces; unused here
    cv.forward(tX.data_ptr(), list(X.shape), tW.data_ptr(), list(Wt.shape), Y.data_ptr(), list(Y.shape),
               tb.data_ptr(), Z.data_ptr(), at, 0, dCol_ptr=dummy, W_KC_ptr=dummy, Y_tmp_ptr=dummy, Z_rows_ptr=dummy)
    torch.cuda.synchronize()
    Y32, Z32 = conv_oracle.forward_f32(X, Wt, b, act="relu", **_kw(g))
    assert np.array_equal(host(Z), Z32) and np.array_equal(host(Y), Y32)
    dW, dX, dB = torch.empty_like(tW), torch.empty_like(tX), torch.empty(Cout, device="cuda")
    cv.backward(tX.data_ptr(), list(X.shape), tW.data_ptr(), list(Wt.shape), tdY.data_ptr(), list(Y.shape),
                Z.data_ptr(), list(Y.shape), dW.data_ptr(), dB.data_ptr(), dX.data_ptr(), at, 0,
                dCol_ptr=dummy, dTmp_ptr=dummy, W_CK_ptr=dummy, dWpack_ptr=dummy, dY_HT_ptr=dummy, gy_rows_ptr=dummy,
                Z_rows_ptr=dummy)
    torch.cuda.synchronize()
    ref = conv_oracle.backward_f64(X, Wt, dY, Z32, act="relu", **_kw(g))
    assert oracle.rel_fro(host(dX), ref["gX"]) <= 1e-5
    assert oracle.rel_fro(host(dW), ref["gW"]) <= 1e-5
    assert oracle.rel_fro(host(dB), ref["gB"]) <= 1e-5


def test_conv2d_forward_backward_replay_from_a_cuda_graph(pkg, lib):
    """The convolution takes its Col / gZ scratch from the stream-ordered allocator, which a stream capture records as
    graph memory nodes: forward + backward captured once and replayed must give the eager results.  (The reference's
    `*_into` path gets the same property from caller workspaces sized for ONE image, python/graph_executor_v2/ops/
    conv2d.py:274-330; the batched kernels here need the whole batch's columns, so those buffers cannot serve.)"""
    cv = pkg.ops_conv2d
    g = torch.Generator(device="cuda").manual_seed(2)
    X = torch.randn((8, 32, 28, 28), device="cuda", generator=g).bfloat16()
    W = (torch.randn((64, 32, 3, 3), device="cuda", generator=g) / 17).bfloat16()
    b = torch.randn(64, device="cuda", generator=g)
    Y = torch.empty((8, 64, 28, 28), device="cuda", dtype=torch.bfloat16)
    Z, dY = torch.empty_like(Y), torch.randn((8, 64, 28, 28), device="cuda", generator=g).bfloat16()
    gX, gW, gB = torch.empty_like(X), torch.empty_like(W), torch.empty(64, device="cuda")

    def step():
        cv.forward_into(X, W, out=Y, B=b, with_bias=True, act="relu", save_z=True, Z_saved=Z, padding=(1, 1))
        cv.backward_into(X, W, dY, Z, with_bias=True, act="relu", gX_out=gX, gW_out=gW, gB_out=gB, padding=(1, 1))

    step()
    torch.cuda.synchronize()
    want = [t.clone() for t in (Y, Z, gX, gW, gB)]
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        step()                                   # the capture stream's own first run
    st.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=st, capture_error_mode="thread_local"):
        step()
    for t in (Y, Z, gX, gW, gB):
        t.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    for a, c in zip(want[:4], (Y, Z, gX, gW)):
        assert torch.equal(a, c)
    assert float((want[4] - gB).abs().max()) <= 1e-3
    assert lib.ge2b_device_status(1) == 0
