"""The CPU oracle against the golden vectors produced by the reference's own host-compiled epilogue code
(tests/golden/make_golden.py).  Integer-free but deterministic fp32: the forward pre-activation Z must match
bit for bit (same fmaf chain), activations within 2 ulp-scale tolerance only where libm versions could differ
(here both ran on the same libm, so they are compared exactly as well)."""
from pathlib import Path

import numpy as np
import pytest

from cases import CASES

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_matches_reference_golden(oracle, name):
    c = CASES[name]()
    g = np.load(GOLD / f"{name}.npz")
    Y, Z = oracle.forward_f32(c["A"], c["B"], c["bias"], act=c["act"], leaky=c["leaky"], alpha=c["alpha"],
                              beta=c["beta"], Cin=c["C"])
    assert np.array_equal(Z, g["Z"]), "pre-activation must be bit-identical to the reference epilogue"
    np.testing.assert_allclose(Y, g["Y"], rtol=0, atol=0)


@pytest.mark.parametrize("name", sorted(CASES))
def test_backward_gz_matches_reference_golden(oracle, name):
    c = CASES[name]()
    g = np.load(GOLD / f"{name}.npz")
    out = oracle.backward_f32(c["A"], c["B"], c["gY"], g["Z"], act=c["act"], leaky=c["leaky"], alpha=c["alpha"],
                              beta=c["beta"], bias_kind=c["bias_kind"] or 3)
    np.testing.assert_array_equal(out["gZ"], g["gZ"])
    # gA, gB, gBias: products / sums of gZ -- against float64 at the reference tests' tolerance
    ref = oracle.backward_f64(c["A"], c["B"], c["gY"], g["Z"], act=c["act"], leaky=c["leaky"])
    np.testing.assert_allclose(out["gA"], c["alpha"] * ref["gA"], rtol=1e-4, atol=3e-4)
    np.testing.assert_allclose(out["gB"], c["alpha"] * ref["gB"], rtol=1e-4, atol=3e-4)


@pytest.mark.parametrize("name", sorted(CASES))
def test_activation_probes(oracle, name):
    c = CASES[name]()
    g = np.load(GOLD / f"{name}.npz")
    np.testing.assert_array_equal(oracle.act_f32(c["act"], g["probe"], c["leaky"]), g["act_probe"])
    np.testing.assert_array_equal(oracle.act_deriv_f32(c["act"], g["probe"], c["leaky"]), g["deriv_probe"])
    # the float64 formulas agree with the fp32 ones to fp32 rounding
    np.testing.assert_allclose(oracle.act_f64(c["act"], g["probe"], c["leaky"]), g["act_probe"], rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(oracle.act_deriv_f64(c["act"], g["probe"], c["leaky"]), g["deriv_probe"], rtol=2e-5,
                               atol=2e-6)


def test_bias_kinds_and_thread_split_invariance(oracle):
    rng = np.random.default_rng(7)
    A = rng.standard_normal((37, 19), dtype=np.float32)
    B = rng.standard_normal((19, 23), dtype=np.float32)
    for bias in (None, np.float32([0.3]), rng.standard_normal(23, dtype=np.float32),
                 rng.standard_normal((37, 1), dtype=np.float32)):
        y1, z1 = oracle.forward_f32(A, B, bias, act="gelu", threads=1)
        y8, z8 = oracle.forward_f32(A, B, bias, act="gelu", threads=8)
        assert np.array_equal(z1, z8) and np.array_equal(y1, y8)
        y64, z64 = oracle.forward_f64(A, B, bias, act="gelu")
        np.testing.assert_allclose(z1, z64, rtol=1e-5, atol=1e-5)


def test_trans_b_and_float64_agree(oracle):
    rng = np.random.default_rng(3)
    Q = rng.standard_normal((33, 16), dtype=np.float32)
    Kt = rng.standard_normal((41, 16), dtype=np.float32)
    y, _ = oracle.forward_f32(Q, Kt, None, alpha=0.25, trans_b=True)
    y64, _ = oracle.forward_f64(Q, Kt, None, alpha=0.25, trans_b=True)
    np.testing.assert_allclose(y, y64, rtol=1e-5, atol=1e-5)


def test_bf16_round_is_nearest_even(oracle):
    x = np.float32([1.0, 1.00390625, 1.005859375, -2.5, 3.140625, 1e-40])
    r = oracle.bf16_round(x)
    assert r[0] == 1.0 and r[3] == -2.5
    assert r[1] == 1.0            # exactly half way between 1.0 and 1.0078125 -> even
    assert r[2] == np.float32(1.0078125)
    assert np.all((r.view(np.uint32) & 0xFFFF) == 0)
