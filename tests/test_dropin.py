"""Drop-in check with the reference's OWN Python binding: oracle/Makefile compiles the reference's unmodified
src/bindings/ops_common_pybind.cpp and src/bindings/gemm_pybind.cpp and links them against libge2_b200.so in place
of the reference's GEMM sources (oracle/_ref/dropin, built where the reference tree is mounted; the built modules
travel with the repository snapshot).  The tests below are the reference's binding smoke test
(graph_executor_v2/tests/cuda_pyd_test/smoke_gemm_binding.py:130-310) restated with torch instead of CuPy, plus the
host-side error behaviour of the launcher."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
DROPIN = ROOT / "oracle" / "_ref" / "dropin"


@pytest.fixture(scope="module")
def ref_ops(lib):
    if not (DROPIN / "graph_executor_v2" / "ops").is_dir():
        pytest.skip("oracle/_ref/dropin not built (needs the reference tree at build time)")
    sys.path.insert(0, str(DROPIN))
    try:
        from graph_executor_v2.ops import _ops_common as c, _ops_gemm as g
    finally:
        sys.path.remove(str(DROPIN))
    return c, g


def test_host_side_validation_matches_reference_messages(ref_ops):
    c, g = ref_ops
    at = c.GemmAttrs()
    A = c.make_tensor_2d(1024, [4, 8], c.DType.F32, c.Device.CUDA, 0)
    Y = c.make_tensor_2d(4096, [4, 3], c.DType.F32, c.Device.CUDA, 0)
    with pytest.raises(RuntimeError, match=r"\[_ops_gemm::forward\] ShapeMismatch"):
        g.forward(A, c.make_tensor_2d(2048, [9, 3], c.DType.F32, c.Device.CUDA, 0), None, Y, at, None, None)
    with pytest.raises(RuntimeError, match="DeviceMismatch"):      # operands of different dtypes
        g.forward(A, c.make_tensor_2d(2048, [8, 3], c.DType.BF16, c.Device.CUDA, 0), None, Y, at, None, None)
    at.trans_b = True
    with pytest.raises(RuntimeError, match="TransposeNotSupported"):
        g.forward(A, c.make_tensor_2d(2048, [8, 3], c.DType.F32, c.Device.CUDA, 0), None, Y, at, None, None)
    at.trans_b = False
    with pytest.raises(RuntimeError, match="DeviceMismatch"):      # host tensor
        g.forward(c.make_tensor_2d(1024, [4, 8], c.DType.F32, c.Device.CPU, 0),
                  c.make_tensor_2d(2048, [8, 3], c.DType.F32, c.Device.CUDA, 0), None, Y, at, None, None)


@pytest.mark.gpu
@pytest.mark.parametrize("with_bias,act", [(True, "relu"), (False, "none"), (True, "gelu"), (True, "sigmoid"),
                                           (True, "tanh"), (True, "leaky_relu")])
def test_reference_binding_raw_forward_backward(ref_ops, oracle, with_bias, act):
    import torch
    c, g = ref_ops
    m, k, n = 32, 64, 16
    rng = np.random.default_rng(2025)
    A_h = rng.standard_normal((m, k), dtype=np.float32)
    B_h = rng.standard_normal((k, n), dtype=np.float32)
    gY_h = rng.standard_normal((m, n), dtype=np.float32)
    bias_h = rng.standard_normal((1, n), dtype=np.float32) if with_bias else None
    A, B, gY = (torch.from_numpy(x).cuda() for x in (A_h, B_h, gY_h))
    bias = torch.from_numpy(bias_h).cuda() if with_bias else None
    Y, Z = torch.empty((m, n), device="cuda"), torch.empty((m, n), device="cuda")
    g.forward_raw(A.data_ptr(), B.data_ptr(), bias.data_ptr() if with_bias else 0, Y.data_ptr(), m, k, n,
                  False, False, act, with_bias, 0.01, True, Z.data_ptr(), None)
    gA, gB = torch.empty((m, k), device="cuda"), torch.empty((k, n), device="cuda")
    gBias = torch.empty((1, n), device="cuda") if with_bias else None
    g.backward_raw(A.data_ptr(), B.data_ptr(), 0, gY.data_ptr(), Z.data_ptr(), gA.data_ptr(), gB.data_ptr(), 0,
                   gBias.data_ptr() if with_bias else 0, m, k, n, False, False, act, with_bias, 0.01, None)
    torch.cuda.synchronize()
    Yo, Zo = oracle.forward_f32(A_h, B_h, bias_h, act=act)
    go = oracle.backward_f32(A_h, B_h, gY_h, Zo, act=act)
    assert np.array_equal(Z.cpu().numpy(), Zo)
    atol, rtol = (5e-4, 1e-3) if act == "gelu" else (1e-5, 1e-4)       # the reference test's own bounds
    np.testing.assert_allclose(Y.cpu().numpy(), Yo, atol=atol, rtol=rtol)
    np.testing.assert_allclose(gA.cpu().numpy(), go["gA"], atol=max(atol, 1e-4), rtol=1e-3)
    np.testing.assert_allclose(gB.cpu().numpy(), go["gB"], atol=max(atol, 1e-4), rtol=1e-3)
    if with_bias:
        np.testing.assert_allclose(gBias.cpu().numpy().ravel(), go["gBias"], atol=max(atol, 1e-4), rtol=1e-3)


@pytest.mark.gpu
def test_reference_binding_tensor_api_with_bf16(ref_ops, oracle):
    """Tensor-object entry points; BF16-tagged tensors, which the reference launcher refuses, run on tcgen05."""
    import torch
    c, g = ref_ops
    M, K, N = 256, 192, 320
    X, W, b, dY = oracle.dense_inputs(M, K, N, seed=4)
    X, W, dY = (oracle.bf16_round(a) for a in (X, W, dY))
    tX, tW, tdY = (torch.from_numpy(a).cuda().bfloat16() for a in (X, W, dY))
    tb = torch.from_numpy(b).cuda()
    Y = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    Z = torch.empty((M, N), device="cuda", dtype=torch.float32)
    mk = lambda t, dt: c.make_tensor_2d(t.data_ptr(), list(t.shape), dt, c.Device.CUDA, 0)   # noqa: E731
    at = c.GemmAttrs()
    at.act, at.with_bias, at.save_z = c.ActKind.GELU, True, True
    bias_t = c.make_tensor_2d(tb.data_ptr(), [1, N], c.DType.F32, c.Device.CUDA, 0)
    g.forward(mk(tX, c.DType.BF16), mk(tW, c.DType.BF16), bias_t, mk(Y, c.DType.BF16), at, mk(Z, c.DType.F32), None)
    gA = torch.empty_like(tX)
    gB = torch.empty_like(tW)
    gb = torch.empty((1, N), device="cuda")
    g.backward(mk(tX, c.DType.BF16), mk(tW, c.DType.BF16), None, mk(tdY, c.DType.BF16), mk(Z, c.DType.F32),
               mk(gA, c.DType.BF16), mk(gB, c.DType.BF16), None,
               c.make_tensor_2d(gb.data_ptr(), [1, N], c.DType.F32, c.Device.CUDA, 0), at, None)
    torch.cuda.synchronize()
    Y64, Z64 = oracle.forward_f64(X, W, b, act="gelu")
    g64 = oracle.backward_f64(X, W, dY, Z.cpu().numpy(), act="gelu")
    for got, ref in ((Y, Y64), (Z, Z64), (gA, g64["gA"]), (gB, g64["gB"]), (gb.ravel(), g64["gBias"])):
        assert oracle.rel_fro(got.float().cpu().numpy(), ref) <= 2e-2
