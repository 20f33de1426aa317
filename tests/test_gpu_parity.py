"""GPU parity tests of the dense-layer path: every call goes through the C ABI of libge2_b200.so and is
compared with the CPU oracle, the golden vectors made from the reference's own epilogue code, and (where it
was built) the reference's own GPU kernels.

Tolerances (from the contract of this path):
  fp32 tensors, exact path      pre-activation Z bit-identical to the oracle / golden; Y, gA, gB, gBias within
                                the reference tests' own bounds (atol 1e-5 / rtol 1e-4 forward, 3e-4 backward)
  bf16 / f16 / TF32 tensor cores  relative Frobenius error <= 2e-2 against float64 on the rounded inputs
"""
import ctypes as C
import itertools
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from cases import CASES  # noqa: E402
from parity_util import check_close  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
ROOT = Path(__file__).resolve().parent.parent
FRO_TOL = 2e-2

ACT_CODE = {"none": 0, "relu": 1, "leaky_relu": 2, "gelu": 3, "sigmoid": 4, "tanh": 5}
ABI_BIAS = {1: 0, 2: 1, 3: 2}   # oracle numbering (scalar 1, per-row 2, per-column 3) -> C-ABI numbering


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


# --------------------------------------------------------------------------- fp32 exact, legacy C ABI
def legacy_forward_ex(pkg, lib, c, by_name=False):
    L = pkg._lib
    A, B = dev(c["A"]), dev(c["B"])
    M, K = c["A"].shape
    N = c["B"].shape[1]
    D = torch.full((M, N), float("nan"), device="cuda")
    Z = torch.full((M, N), float("nan"), device="cuda")
    Cin = dev(c["C"]) if c["C"] is not None else None
    bias = dev(c["bias"].reshape(-1)) if c["bias"] is not None else None
    p = L.ParamsEx()
    p.M, p.N, p.K = M, N, K
    p.lda = p.ldb = p.ldc = p.ldd = 0
    p.alpha, p.beta = c["alpha"], c["beta"]
    p.use_C, p.has_bias = int(Cin is not None), int(bias is not None)
    p.bias_kind = ABI_BIAS.get(c["bias_kind"], 0)
    p.act_kind = ACT_CODE[c["act"]]
    p.leaky_slope = c["leaky"]
    p.save_preact, p.ldZ = 1, 0
    ptrs = [A.data_ptr(), B.data_ptr()] + ([Cin.data_ptr()] if Cin is not None else []) + [D.data_ptr()] + \
           ([bias.data_ptr()] if bias is not None else []) + [Z.data_ptr()]
    bufs = L.make_bufs(ptrs, p)
    s = torch.cuda.current_stream().cuda_stream
    rc = lib.ge2_launch(b"gemm_bias_act_f32_ex", bufs, len(bufs), s) if by_name else \
        lib.ge2_launch_gemm_bias_act_f32_ex(bufs, len(bufs), s)
    assert rc == 0
    torch.cuda.synchronize()
    return D, Z


@pytest.mark.parametrize("name", sorted(CASES))
def test_fp32_forward_matches_golden_and_oracle(pkg, lib, oracle, name):
    c = CASES[name]()
    g = np.load(GOLD / f"{name}.npz")
    D, Z = legacy_forward_ex(pkg, lib, c, by_name=(name.startswith("legacy")))
    assert lib.ge2b_last_route() == 1
    assert np.array_equal(host(Z), g["Z"]), "pre-activation must be bit-identical to the reference's"
    np.testing.assert_allclose(host(D), g["Y"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", sorted(CASES))
def test_fp32_backward_matches_oracle(pkg, lib, oracle, name):
    L = pkg._lib
    c = CASES[name]()
    g = np.load(GOLD / f"{name}.npz")
    M, K = c["A"].shape
    N = c["B"].shape[1]
    kind = c["bias_kind"] or 3
    A, B, gY, Z = dev(c["A"]), dev(c["B"]), dev(c["gY"]), dev(g["Z"])
    Cin = dev(c["C"]) if c["C"] is not None else None
    gA = torch.full((M, K), float("nan"), device="cuda")
    gB = torch.full((K, N), float("nan"), device="cuda")
    gC = torch.full((M, N), float("nan"), device="cuda") if Cin is not None else None
    nb = {1: 1, 2: M, 3: N}[kind]
    gBias = torch.full((nb,), float("nan"), device="cuda")
    p = L.ParamsBwd()
    p.M, p.N, p.K = M, N, K
    p.alpha, p.beta = c["alpha"], c["beta"]
    p.bias_kind, p.act_kind, p.leaky_slope = ABI_BIAS[kind], ACT_CODE[c["act"]], c["leaky"]
    ptr = lambda t: t.data_ptr() if t is not None else 0   # noqa: E731
    bufs = L.make_bufs([ptr(A), ptr(B), ptr(Cin), ptr(gY), ptr(Z), ptr(gA), ptr(gB), ptr(gC), ptr(gBias)], p)
    assert lib.ge2_launch(b"gemm_bias_act_bwd_f32_ex", bufs, len(bufs), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    o = oracle.backward_f32(c["A"], c["B"], c["gY"], g["Z"], act=c["act"], leaky=c["leaky"], alpha=c["alpha"],
                            beta=c["beta"], bias_kind=kind, want_gC=Cin is not None)
    np.testing.assert_allclose(host(gA), o["gA"], rtol=1e-4, atol=3e-4)
    np.testing.assert_allclose(host(gB), o["gB"], rtol=1e-4, atol=3e-4)
    np.testing.assert_allclose(host(gBias), o["gBias"], rtol=1e-4, atol=3e-4)
    if Cin is not None:
        np.testing.assert_allclose(host(gC), o["gC"], rtol=1e-5, atol=1e-5)


def test_legacy_relu_entry_and_name_table(pkg, lib, oracle):
    L = pkg._lib
    c = CASES["relu128"]()
    A, B, bias = dev(c["A"]), dev(c["B"]), dev(c["bias"])
    D = torch.empty((128, 128), device="cuda")
    p = L.ParamsLegacy(128, 128, 128, 1, 1)
    bufs = L.make_bufs([A.data_ptr(), B.data_ptr(), bias.data_ptr(), D.data_ptr()], p)
    assert lib.ge2_launch(b"gemm_bias_act_f32", bufs, len(bufs), None) == 0
    torch.cuda.synchronize()
    g = np.load(GOLD / "relu128.npz")
    np.testing.assert_array_equal(host(D), g["Y"])     # ReLU has no transcendental: exact
    # the fp16 slot: same call shape with half tensors, on tensor cores
    Ah, Bh = A.half(), B.half()
    Dh = torch.empty((128, 128), device="cuda", dtype=torch.float16)
    bufs = L.make_bufs([Ah.data_ptr(), Bh.data_ptr(), bias.data_ptr(), Dh.data_ptr()], p)
    assert lib.ge2_launch(b"gemm_bias_act_tc_f16", bufs, len(bufs), None) == 0
    torch.cuda.synchronize()
    assert lib.ge2b_last_route() == 2
    y64, _ = oracle.forward_f64(host(Ah), host(Bh), c["bias"], act="relu")
    assert oracle.rel_fro(host(Dh), y64) <= FRO_TOL


SMALL = [1, 7, 16, 33, 127, 128, 129, 255, 257]


@pytest.mark.parametrize("act", ["none", "gelu"])
def test_fp32_small_shape_sweep_bit_exact(pkg, lib, oracle, act):
    rng = np.random.default_rng(11)
    combos = list(itertools.product(SMALL, SMALL, SMALL))
    picks = [combos[i] for i in rng.choice(len(combos), 40, replace=False)] + [(1, 1, 1), (257, 257, 257)]
    for (M, N, K) in picks:
        A = rng.standard_normal((M, K), dtype=np.float32)
        B = rng.standard_normal((K, N), dtype=np.float32)
        b = rng.standard_normal(N, dtype=np.float32)
        Y, Z = pkg.ops_gemm.forward(dev(A), dev(B), dev(b), act=act, return_z=True)
        Yo, Zo = oracle.forward_f32(A, B, b, act=act)
        assert np.array_equal(host(Z), Zo), (M, N, K)
        np.testing.assert_allclose(host(Y), Yo, rtol=1e-4, atol=1e-5)


def test_padded_rows_and_canaries_fp32_and_bf16(pkg, lib, oracle):
    """ld > cols on every tensor; the padding must not be written."""
    rng = np.random.default_rng(5)
    M, K, N = 200, 136, 304
    for dtype, math in ((torch.float32, "fp32"), (torch.bfloat16, "fp32"), (torch.float32, "tf32")):
        Af = oracle.bf16_round(rng.standard_normal((M, K), dtype=np.float32))
        Bf = oracle.bf16_round(rng.standard_normal((K, N), dtype=np.float32))
        b = rng.standard_normal(N, dtype=np.float32)
        Abuf = torch.zeros((M, K + 8), device="cuda", dtype=dtype)
        Bbuf = torch.zeros((K, N + 16), device="cuda", dtype=dtype)
        Abuf[:, :K] = dev(Af, dtype)
        Bbuf[:, :N] = dev(Bf, dtype)
        out = torch.full((M, N + 24), 777.0, device="cuda", dtype=dtype)
        zout = torch.full((M, N + 8), 555.0, device="cuda", dtype=dtype)
        pkg.ops_gemm.forward_into(Abuf[:, :K], Bbuf[:, :N], out=out[:, :N], bias=dev(b), with_bias=True, act="relu",
                                  save_z=True, z_out=zout[:, :N], math=math)
        torch.cuda.synchronize()
        assert torch.all(out[:, N:] == 777.0) and torch.all(zout[:, N:] == 555.0)
        y64, z64 = oracle.forward_f64(Af, Bf, b, act="relu")
        tol = 1e-5 if (dtype == torch.float32 and math == "fp32") else FRO_TOL
        assert oracle.rel_fro(host(out[:, :N]), y64) <= tol
        assert oracle.rel_fro(host(zout[:, :N]), z64) <= tol


# --------------------------------------------------------------------------- tensor-core paths
def tc_case(pkg, lib, oracle, M, K, N, dtype, math, act, seed=0, z_dtype=None, expect_route=2):
    X, W, b, dY = oracle.dense_inputs(M, K, N, seed=seed)
    if dtype != torch.float32:
        X, W, dY = (oracle.bf16_round(a) if dtype == torch.bfloat16 else a.astype(np.float16).astype(np.float32)
                    for a in (X, W, dY))
    tX, tW, tdY, tb = dev(X, dtype), dev(W, dtype), dev(dY, dtype), dev(b)
    Y, Z = pkg.ops_gemm.forward(tX, tW, tb, act=act, return_z=True, math=math, z_dtype=z_dtype)
    if expect_route:
        assert lib.ge2b_last_route() == expect_route
    g = pkg.ops_gemm.backward(tX, tW, tdY, Z, act=act, want_gBias=True, math=math)
    torch.cuda.synchronize()
    Y64, Z64 = oracle.forward_f64(X, W, b, act=act)
    g64 = oracle.backward_f64(X, W, dY, host(Z), act=act)
    # whole-tensor bound of the contract (2e-2) and the local bound (every 128 x 128 block within 5e-3)
    errs = {"Y": check_close("Y", host(Y), Y64)[0], "Z": check_close("Z", host(Z), Z64)[0],
            "dX": check_close("dX", host(g["gA"]), g64["gA"])[0], "dW": check_close("dW", host(g["gB"]), g64["gB"])[0],
            "db": check_close("db", host(g["gBias"]).ravel(), g64["gBias"])[0]}
    return errs


@pytest.mark.parametrize("act", ["none", "relu", "gelu", "sigmoid", "tanh", "leaky_relu"])
@pytest.mark.parametrize("dtype,math", [(torch.bfloat16, "fp32"), (torch.float16, "fp32"), (torch.float32, "tf32")])
def test_tensor_core_forward_backward_vs_float64(pkg, lib, oracle, dtype, math, act):
    errs = tc_case(pkg, lib, oracle, 384, 320, 512, dtype, math, act)
    assert all(e <= FRO_TOL for e in errs.values()), errs


@pytest.mark.parametrize("shape", [(128, 64, 128), (129, 72, 136), (1, 8, 8), (333, 1000, 264), (1024, 1024, 1024),
                                   (16, 1024, 2048), (2048, 136, 24)])
def test_bf16_ragged_shapes(pkg, lib, oracle, shape):
    M, K, N = shape
    errs = tc_case(pkg, lib, oracle, M, K, N, torch.bfloat16, "fp32", "gelu", seed=3, z_dtype=torch.float32)
    assert all(e <= FRO_TOL for e in errs.values()), errs


def test_bf16_unaligned_pitch_uses_the_cuda_core_kernel(pkg, lib, oracle):
    """K and N not multiples of 8 elements: TMA cannot address the rows, the exact kernel takes over."""
    errs = tc_case(pkg, lib, oracle, 65, 37, 51, torch.bfloat16, "fp32", "gelu", expect_route=1)
    assert all(e <= FRO_TOL for e in errs.values()), errs


def test_config2_full_size_row_sampled(pkg, lib, oracle):
    """M=N=K=4096 bf16 GELU forward + backward; float64 reference on sampled rows / columns only."""
    M = N = K = 4096
    X, W, b, dY = oracle.dense_inputs(M, K, N, seed=0)
    X, W, dY = (oracle.bf16_round(a) for a in (X, W, dY))
    tX, tW, tdY, tb = dev(X, torch.bfloat16), dev(W, torch.bfloat16), dev(dY, torch.bfloat16), dev(b)
    Y, Z = pkg.ops_gemm.forward(tX, tW, tb, act="gelu", return_z=True)
    g = pkg.ops_gemm.backward(tX, tW, tdY, Z, act="gelu", want_gBias=True)
    torch.cuda.synchronize()
    rng = np.random.default_rng(1)
    rows = np.sort(rng.choice(M, 96, replace=False))
    Y64, Z64 = oracle.forward_f64(X[rows], W, b, act="gelu")
    assert oracle.rel_fro(host(Y[rows]), Y64) <= FRO_TOL
    assert oracle.rel_fro(host(Z[rows]), Z64) <= FRO_TOL
    Zh = host(Z)
    gZ = dY.astype(np.float64) * oracle.act_deriv_f64("gelu", Zh)
    assert oracle.rel_fro(host(g["gA"][rows]), gZ[rows] @ W.astype(np.float64).T) <= FRO_TOL
    cols = np.sort(rng.choice(K, 96, replace=False))
    assert oracle.rel_fro(host(g["gB"][cols]), X[:, cols].astype(np.float64).T @ gZ) <= FRO_TOL
    assert oracle.rel_fro(host(g["gBias"]).ravel(), gZ.sum(axis=0)) <= FRO_TOL


def test_linearity_at_full_size(pkg, lib):
    """act = none: f(X1 + X2) == f(X1) + f(X2) up to bf16 output rounding, at 4096^3."""
    torch.manual_seed(0)
    n = 4096
    X1 = torch.randn(n, n, device="cuda").bfloat16()
    X2 = (torch.randn(n, n, device="cuda") * 0.5).bfloat16()
    W = (torch.randn(n, n, device="cuda") / 64).bfloat16()
    Xs = (X1.float() + X2.float()).bfloat16()
    exact = (Xs.float() == X1.float() + X2.float())
    y1 = pkg.ops_gemm.forward(X1, W).float()
    y2 = pkg.ops_gemm.forward(X2, W).float()
    ys = pkg.ops_gemm.forward(Xs, W).float()
    rows = exact.all(dim=1)                       # rows where the bf16 sum is exact
    assert rows.sum() >= 0
    num = (ys - (y1 + y2))[rows].norm() if rows.any() else torch.tensor(0.0)
    den = ys[rows].norm() if rows.any() else torch.tensor(1.0)
    assert float(num / den) <= 1e-2


def test_run_to_run_determinism(pkg, lib):
    torch.manual_seed(1)
    X = torch.randn(1024, 768, device="cuda").bfloat16()
    W = torch.randn(768, 1280, device="cuda").bfloat16()
    gY = torch.randn(1024, 1280, device="cuda").bfloat16()
    b = torch.randn(1280, device="cuda")
    outs = []
    for _ in range(2):
        Y, Z = pkg.ops_gemm.forward(X, W, b, act="gelu", return_z=True)
        g = pkg.ops_gemm.backward(X, W, gY, Z, act="gelu", want_gBias=True)
        outs.append((Y.clone(), Z.clone(), g["gA"].clone(), g["gB"].clone(), g["gBias"].clone()))   # db too: no atomics
    for a, c in zip(*outs):
        assert torch.equal(a, c)


# --------------------------------------------------------------------------- strided-batched form
@pytest.mark.parametrize("dtype,math", [(torch.bfloat16, "fp32"), (torch.float32, "tf32"), (torch.float32, "fp32")])
def test_batched_attention_gemms(pkg, lib, oracle, dtype, math):
    """S = (Q.K^T)/sqrt(d) and O = P.V per (batch, head) in one launch each (reduced B, H, L of config 4)."""
    Bn, H, L, d = 2, 3, 256, 128
    rng = np.random.default_rng(0)
    Q = oracle.bf16_round(rng.standard_normal((Bn, H, L, d), dtype=np.float32))
    Kx = oracle.bf16_round(rng.standard_normal((Bn, H, L, d), dtype=np.float32))
    V = oracle.bf16_round(rng.standard_normal((Bn, H, L, d), dtype=np.float32))
    raw = rng.standard_normal((Bn, H, L, L)).astype(np.float64)
    P = np.exp(raw - raw.max(-1, keepdims=True))
    P = oracle.bf16_round((P / P.sum(-1, keepdims=True)).astype(np.float32))
    tQ, tK, tV, tP = (dev(a, dtype) for a in (Q, Kx, V, P))
    S = torch.empty((Bn, H, L, L), device="cuda", dtype=dtype)
    O = torch.empty((Bn, H, L, d), device="cuda", dtype=dtype)
    scale = 1.0 / np.sqrt(d)
    pkg.ops_gemm.forward_batched(tQ, tK, out=S, trans_b=True, alpha=scale, math=math)
    pkg.ops_gemm.forward_batched(tP, tV, out=O, math=math)
    torch.cuda.synchronize()
    S64 = scale * np.einsum("bhld,bhmd->bhlm", Q.astype(np.float64), Kx.astype(np.float64))
    O64 = np.einsum("bhlm,bhmd->bhld", P.astype(np.float64), V.astype(np.float64))
    tol = 1e-5 if (dtype == torch.float32 and math == "fp32") else FRO_TOL
    assert oracle.rel_fro(host(S), S64) <= tol
    assert oracle.rel_fro(host(O), O64) <= tol


def test_batched_shared_weight_broadcast(pkg, lib, oracle):
    """Batch stride 0 on B: every slice multiplies the same weight (the per-image conv2d / v1 executor form)."""
    rng = np.random.default_rng(2)
    A = oracle.bf16_round(rng.standard_normal((5, 96, 72), dtype=np.float32))
    W = oracle.bf16_round(rng.standard_normal((1, 72, 40), dtype=np.float32))
    b = rng.standard_normal(40, dtype=np.float32)
    out = torch.empty((5, 96, 40), device="cuda", dtype=torch.bfloat16)
    pkg.ops_gemm.forward_batched(dev(A, torch.bfloat16), dev(W, torch.bfloat16), out=out, bias=dev(b), act="relu")
    torch.cuda.synchronize()
    ref = np.maximum(A.astype(np.float64) @ W[0].astype(np.float64) + b, 0)
    assert oracle.rel_fro(host(out), ref) <= FRO_TOL


# --------------------------------------------------------------------------- Dense layer
def test_dense_layer_eager_and_into(pkg, lib, oracle):
    layer = pkg.Dense(256, activation="gelu", dtype=torch.bfloat16, seed=0)
    x = torch.randn(128, 192, device="cuda").bfloat16()
    y = layer(x)
    gy = torch.randn_like(y)
    gx = layer.backward(gy)
    y2 = torch.empty_like(y)
    z2 = torch.empty_like(y)
    layer.forward_into(x, out=y2, z_out=z2)
    gA, gW = torch.empty_like(x), torch.empty_like(layer.W)
    gb = torch.empty((1, 256), device="cuda")
    work = torch.empty((128, 256), device="cuda")
    layer.backward_into(gy, gA_out=gA, gW_out=gW, gB_out=gb, work_dZ=work)
    torch.cuda.synchronize()
    assert torch.equal(y, y2) and torch.equal(gx, gA)
    Y64, Z64 = oracle.forward_f64(host(x), host(layer.W), host(layer.b), act="gelu")
    assert oracle.rel_fro(host(y), Y64) <= FRO_TOL


# --------------------------------------------------------------------------- the reference's own GPU kernels
def _ref_gpu():
    so = ROOT / "oracle" / "_ref" / "libref_gemm.so"
    if not so.exists():
        pytest.skip("oracle/_ref/libref_gemm.so was not built (needs the reference tree at build time)")
    lib = C.CDLL(str(so))
    lib.ref_gpu_forward.restype = C.c_int
    lib.ref_gpu_forward.argtypes = [C.c_void_p] * 3 + [C.c_longlong] + [C.c_void_p] * 2 + [C.c_int] * 4 + \
                                   [C.c_float, C.c_void_p]
    lib.ref_gpu_backward.restype = C.c_int
    lib.ref_gpu_backward.argtypes = [C.c_void_p] * 7 + [C.c_longlong, C.c_void_p] + [C.c_int] * 4 + \
                                    [C.c_float, C.c_void_p]
    return lib


@pytest.mark.parametrize("act", ["relu", "gelu", "sigmoid", "tanh"])
def test_fp32_path_against_reference_gpu_kernels(pkg, lib, oracle, act):
    """Config 1 (256x512 . 512x512 + b, seed 0) through the reference's GemmCudaLaunch / GemmCudaBackward built
    for sm_100a, and through this library, on the same device buffers."""
    ref = _ref_gpu()
    X, W, b, dY = oracle.dense_inputs(256, 512, 512, seed=0)
    tX, tW, tb, tdY = dev(X), dev(W), dev(b), dev(dY)
    Yr, Zr = torch.empty((256, 512), device="cuda"), torch.empty((256, 512), device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert ref.ref_gpu_forward(tX.data_ptr(), tW.data_ptr(), tb.data_ptr(), 512, Yr.data_ptr(), Zr.data_ptr(),
                               256, 512, 512, ACT_CODE[act], 0.01, s) == 0
    Y, Z = pkg.ops_gemm.forward(tX, tW, tb, act=act, return_z=True)
    torch.cuda.synchronize()
    assert torch.equal(Z, Zr), "pre-activation differs from the reference kernel's"
    rel = ((Y - Yr).abs() / Yr.abs().clamp_min(1e-5)).max().item()
    assert rel <= 1e-5, rel
    gAr, gBr = torch.empty_like(tX), torch.empty_like(tW)
    gbr = torch.empty(512, device="cuda")
    scratch = torch.empty((256, 512), device="cuda")
    assert ref.ref_gpu_backward(tX.data_ptr(), tW.data_ptr(), tdY.data_ptr(), Zr.data_ptr(), gAr.data_ptr(),
                                gBr.data_ptr(), gbr.data_ptr(), 512, scratch.data_ptr(), 256, 512, 512,
                                ACT_CODE[act], 0.01, s) == 0
    g = pkg.ops_gemm.backward(tX, tW, tdY, Z, act=act, want_gBias=True)
    torch.cuda.synchronize()
    for got, want in ((g["gA"], gAr), (g["gB"], gBr), (g["gBias"].ravel(), gbr)):
        err = ((got - want).abs() / want.abs().clamp_min(1.0)).max().item()
        assert err <= 1e-5 * 30, err   # different summation orders over 256..512 terms of O(1) products


# --------------------------------------------------------------------------- host-buffer plan
def test_host_plan_step_and_pipelined_submit(pkg, lib, oracle):
    """ge2b_dense_plan_*: host pointers in, host pointers out; `step` and the two-in-flight submit/wait form
    must give the results of the device-resident calls."""
    L = pkg._lib
    M, K, N = 512, 256, 384
    X, W, b, dY = oracle.dense_inputs(M, K, N, seed=9)
    hX, hW, hdY = (torch.from_numpy(oracle.bf16_round(a)).bfloat16().pin_memory() for a in (X, W, dY))
    hb = torch.from_numpy(b).pin_memory()
    plan = C.c_void_p()
    assert lib.ge2b_dense_plan_create(C.byref(plan), M, K, N, L.DT_BF16, L.ACT["gelu"], 0.01, 1, L.MATH_TENSOR) == 0
    try:
        outs = [(torch.zeros((M, N), dtype=torch.bfloat16).pin_memory(), torch.zeros((M, K), dtype=torch.bfloat16).pin_memory(),
                 torch.zeros((K, N), dtype=torch.bfloat16).pin_memory(), torch.zeros((N,), dtype=torch.float32).pin_memory())
                for _ in range(3)]
        y, dx, dw, db = outs[0]
        assert lib.ge2b_dense_plan_step(plan, hX.data_ptr(), hW.data_ptr(), hb.data_ptr(), hdY.data_ptr(), y.data_ptr(),
                                        dx.data_ptr(), dw.data_ptr(), db.data_ptr()) == 0
        dX_, dW_, b_, dY_ = hX.cuda(), hW.cuda(), hb.cuda(), hdY.cuda()
        Yd, Zd = pkg.ops_gemm.forward(dX_, dW_, b_, act="gelu", return_z=True)
        gd = pkg.ops_gemm.backward(dX_, dW_, dY_, Zd, act="gelu", want_gBias=True)
        torch.cuda.synchronize()
        assert torch.equal(y, Yd.cpu()) and torch.equal(dx, gd["gA"].cpu()) and torch.equal(dw, gd["gB"].cpu())
        np.testing.assert_allclose(db.numpy(), gd["gBias"].cpu().numpy().ravel(), rtol=1e-4, atol=3e-4)
        # three submits with two buffer sets in flight, then drain
        for i in (1, 2):
            o = outs[i]
            assert lib.ge2b_dense_plan_submit(plan, hX.data_ptr(), hW.data_ptr(), hb.data_ptr(), hdY.data_ptr(),
                                              o[0].data_ptr(), o[1].data_ptr(), o[2].data_ptr(), o[3].data_ptr()) == 0
        assert lib.ge2b_dense_plan_wait(plan) == 0 and lib.ge2b_dense_plan_wait(plan) == 0
        assert lib.ge2b_dense_plan_wait(plan) == 0          # nothing outstanding: no-op
        for i in (1, 2):
            assert torch.equal(outs[i][0], y) and torch.equal(outs[i][1], dx) and torch.equal(outs[i][2], dw)
    finally:
        lib.ge2b_dense_plan_destroy(plan)


@pytest.mark.parametrize("shape", [(16, 8192, 2048), (64, 4096, 1024), (128, 8192, 8192), (300, 2048, 512),
                                   (40, 2048, 6000), (16, 8192, 8192)])
def test_split_reduction_for_small_grids(pkg, lib, oracle, shape):
    """Few output tiles, long reduction: the launch splits the reduction across SMs and adds fp32 partial sums."""
    M, K, N = shape
    errs = tc_case(pkg, lib, oracle, M, K, N, torch.bfloat16, "fp32", "gelu", seed=5)
    assert all(e <= FRO_TOL for e in errs.values()), errs
    # the same call twice gives the same bits (fixed order of the partial sums)
    X = torch.randn(M, K, device="cuda").bfloat16()
    W = (torch.randn(K, N, device="cuda") / 32).bfloat16()
    assert torch.equal(pkg.ops_gemm.forward(X, W), pkg.ops_gemm.forward(X, W))


# --------------------------------------------------------------------------- narrow tail of a partly filled last wave
@pytest.mark.parametrize("dtype,math", [(torch.bfloat16, "fp32"), (torch.float32, "tf32")])
@pytest.mark.parametrize("shape", [(2304, 2304, 2304), (2300, 2056, 2200)])
def test_narrow_tail_tiles(pkg, lib, oracle, dtype, math, shape):
    """9 x 9 = 81 tiles of 256 x 256 on 74 CTA pairs: the 7 tiles left after the first wave run as 14 halves of 128
    columns.  Forward, dX and dW each have that tile count, so all three operand orders take the path; the ragged
    shape leaves the second half of the last column block partly (N) or wholly (K) outside the matrix."""
    M, K, N = shape
    errs = tc_case(pkg, lib, oracle, M, K, N, dtype, math, "gelu", seed=11)
    assert all(e <= FRO_TOL for e in errs.values()), errs


def test_narrow_tail_batched(pkg, lib, oracle):
    """3 slices x 25 tiles = 75 tiles: one tail tile in the last slice, with K^T as a transposed operand."""
    rng = np.random.default_rng(4)
    Q = oracle.bf16_round(rng.standard_normal((3, 1280, 64), dtype=np.float32))
    Kx = oracle.bf16_round(rng.standard_normal((3, 1280, 64), dtype=np.float32))
    S = torch.empty((3, 1280, 1280), device="cuda", dtype=torch.bfloat16)
    pkg.ops_gemm.forward_batched(dev(Q, torch.bfloat16), dev(Kx, torch.bfloat16), out=S, trans_b=True, alpha=0.125)
    torch.cuda.synchronize()
    S64 = 0.125 * np.einsum("bld,bmd->blm", Q.astype(np.float64), Kx.astype(np.float64))
    assert oracle.rel_fro(host(S), S64) <= FRO_TOL


# --------------------------------------------------------------------------- dX and dW in one launch
@pytest.mark.parametrize("dtype,math", [(torch.bfloat16, "fp32"), (torch.float32, "tf32")])
@pytest.mark.parametrize("shape", [(4096, 4096, 4096, 1), (2304, 2304, 2304, 1), (2300, 2056, 2200, 1), (2048, 1536, 2560, 0),
                                   (1100, 1032, 1416, 0)])
def test_backward_pair_in_one_launch(pkg, lib, oracle, dtype, math, shape):
    """When both gradients are wanted and their combined tile list fills the machine better than the two lists do
    one after the other, dX = gZ.W^T and dW = X^T.gZ run as ONE persistent launch (two problems with different
    operand orders in one tile list).  The launch counter tells which form ran; results are checked on sampled rows
    against float64 either way."""
    M, K, N, expect_dual = shape
    rng = np.random.default_rng(21)
    X = rng.standard_normal((M, K), dtype=np.float32)
    W = (rng.standard_normal((K, N), dtype=np.float32) / np.sqrt(K)).astype(np.float32)
    dY = rng.standard_normal((M, N), dtype=np.float32)
    Zh = rng.standard_normal((M, N), dtype=np.float32)
    if dtype == torch.bfloat16:
        X, W, dY, Zh = (oracle.bf16_round(a) for a in (X, W, dY, Zh))
    tX, tW, tdY, tZ = dev(X, dtype), dev(W, dtype), dev(dY, dtype), dev(Zh, dtype)
    work = torch.empty_like(tdY)
    gA, gB, gb = torch.empty_like(tX), torch.empty_like(tW), torch.empty(N, device="cuda")
    kw = dict(act="gelu", gA_out=gA, gB_out=gB, gBias_out=gb, work_dZ=work, math=math)
    pkg.ops_gemm.backward_into(tX, tW, tdY, tZ, **kw)           # warm (first-use setup)
    l0 = lib.ge2b_launches_total()
    pkg.ops_gemm.backward_into(tX, tW, tdY, tZ, **kw)
    launches = lib.ge2b_launches_total() - l0
    torch.cuda.synchronize()
    units = lib.ge2b_sm_count() // 2
    tiles = lambda r, c: -(-r // 256) * -(-c // 256)              # noqa: E731
    waves = lambda t: -(-t // units)                              # noqa: E731
    dual = (tiles(M, K) + tiles(K, N) >= units and
            waves(tiles(M, K) + tiles(K, N)) < waves(tiles(M, K)) + waves(tiles(K, N)))
    assert dual == bool(expect_dual) or units != 74
    assert launches == (2 if dual else 3)                         # prologue + one or two GEMM launches
    gZ = dY.astype(np.float64) * oracle.act_deriv_f64("gelu", Zh.astype(np.float64))
    gZ = host(work).astype(np.float64) if dtype == torch.bfloat16 else gZ
    rows = np.sort(rng.choice(M, min(M, 64), replace=False))
    cols = np.sort(rng.choice(K, min(K, 64), replace=False))
    assert oracle.rel_fro(host(gA[rows]), gZ[rows] @ W.astype(np.float64).T) <= FRO_TOL
    assert oracle.rel_fro(host(gB[cols]), X[:, cols].astype(np.float64).T @ gZ) <= FRO_TOL
    # the same call twice gives the same bits
    gA2, gB2 = gA.clone(), gB.clone()
    pkg.ops_gemm.backward_into(tX, tW, tdY, tZ, **kw)
    torch.cuda.synchronize()
    assert torch.equal(gA, gA2) and torch.equal(gB, gB2)


# --------------------------------------------------------------------------- the bounded wait, made to run out
def test_bounded_wait_expires_and_reports(pkg, lib):
    """Every mbarrier wait in the GEMM kernels is bounded; this runs the expiry path itself: a barrier nothing arrives
    at, a budget of a million clocks.  The wait returns false, the status word gets its bit, the context lives on."""
    rep = (C.c_int * 4)()
    assert lib.ge2b_device_status(1) == 0
    assert lib.ge2b_selftest_wait_expiry(1_000_000, rep, torch.cuda.current_stream().cuda_stream) == 0
    gave_up, abort_flag, cycles, second = list(rep)
    assert gave_up == 0 and abort_flag == 1 and second == 0
    assert 1_000_000 <= cycles < 50_000_000                 # waited its budget, not forever
    assert lib.ge2b_device_status(1) == 1                   # kErrWaitTimeout, read and cleared
    assert lib.ge2b_device_status(0) == 0
    # the context is still usable: an ordinary launch works and leaves the status clean
    x = torch.randn(256, 256, device="cuda").bfloat16()
    y = pkg.ops_gemm.forward(x, x)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and lib.ge2b_device_status(0) == 0
    assert lib.ge2b_selftest_wait_expiry(0, rep, None) == -1            # budget out of range


# --------------------------------------------------------------------------- fp32 on tensor cores, error-compensated
@pytest.mark.parametrize("shape", [(256, 512, 512), (384, 320, 512), (1024, 1024, 1024), (130, 72, 264), (2304, 2304, 2304)])
def test_fp32x3_forward_matches_the_fp32_path(pkg, lib, oracle, shape):
    """math = "fp32x3": operands split into TF32-exact big parts and fp32 remainders, three tensor-core products in one
    fp32 accumulator.  Every product is exact; what remains is the tensor core's accumulator, which truncates (up to
    one unit in the last place per MMA, K/8 of them at full magnitude), so the bound grows with K: max error
    <= 3e-6 + 2^-23 * K/8 relative to max(|y|, 1) against the exact fp32 chain (about the fp32 path's 1e-5 at K = 512),
    relative Frobenius error against float64 <= 1e-8 * K."""
    M, K, N = shape
    X, W, b, _ = oracle.dense_inputs(M, K, N, seed=4)
    tX, tW, tb = dev(X), dev(W), dev(b)
    Y, Z = pkg.ops_gemm.forward(tX, tW, tb, act="gelu", return_z=True, math="fp32x3")
    assert lib.ge2b_last_route() == 2
    Ye, Ze = pkg.ops_gemm.forward(tX, tW, tb, act="gelu", return_z=True, math="fp32")       # exact chain (CUDA cores)
    assert lib.ge2b_last_route() == 1
    torch.cuda.synchronize()
    bound = 3e-6 + 2.0 ** -23 * K / 8      # a few units in the last place of the two fp32 results + the accumulator's
    for got, want in ((Z, Ze), (Y, Ye)):
        rel = ((got - want).abs() / want.abs().clamp_min(1.0)).max().item()
        print(f"fp32x3 vs exact chain, K={K}: max error {rel:.2e} (bound {bound:.2e})")
        assert rel <= bound, (rel, bound)
    Y64, Z64 = oracle.forward_f64(X, W, b, act="gelu")
    e3 = oracle.rel_fro(host(Z), Z64)
    assert e3 <= max(1e-6, 1e-8 * K), e3


@pytest.mark.parametrize("math", ["fp32", "fp32x3"])
def test_fp32_backward_runs_compensated_on_tensor_cores(pkg, lib, oracle, math):
    """fp32 backward GEMMs (the reference hands them to cuBLAS SGEMM) run error-compensated on the tensor cores by
    default; against float64 the result is fp32-grade."""
    M, K, N = 512, 384, 640
    X, W, b, dY = oracle.dense_inputs(M, K, N, seed=6)
    tX, tW, tdY = dev(X), dev(W), dev(dY)
    Y, Z = pkg.ops_gemm.forward(tX, tW, dev(b), act="tanh", return_z=True)
    g = pkg.ops_gemm.backward(tX, tW, tdY, Z, act="tanh", want_gBias=True, math=math)
    torch.cuda.synchronize()
    assert lib.ge2b_last_route() == 2
    g64 = oracle.backward_f64(X, W, dY, host(Z), act="tanh")
    assert oracle.rel_fro(host(g["gA"]), g64["gA"]) <= 1e-8 * N          # reduction over N
    assert oracle.rel_fro(host(g["gB"]), g64["gB"]) <= 1e-8 * M          # reduction over M
    assert oracle.rel_fro(host(g["gBias"]).ravel(), g64["gBias"]) <= 2e-6
