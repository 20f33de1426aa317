"""The attention oracle (oracle/sdpa_oracle.py) against an independent CPU implementation (torch's
scaled_dot_product_attention in float64): no mask, causal, additive float mask, integer keep/drop mask."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")


@pytest.mark.parametrize("case", ["plain", "causal", "float_mask", "int_mask", "scale"])
def test_sdpa_oracle_matches_torch_float64(case):
    so = importlib.import_module("oracle.sdpa_oracle")
    rng = np.random.default_rng(3)
    B, H, M, N, D = 2, 3, 37, 53, 16
    if case == "causal":
        N = M
    Q, K, V = rng.standard_normal((B, H, M, D)), rng.standard_normal((B, H, N, D)), rng.standard_normal((B, H, N, D))
    kw, tkw = {}, {}
    if case == "causal":
        kw["causal"] = True
        tkw["is_causal"] = True
    if case == "float_mask":
        m = rng.standard_normal((B, 1, M, N)).astype(np.float32)
        kw["mask"] = m
        tkw["attn_mask"] = torch.from_numpy(m.astype(np.float64))
    if case == "int_mask":
        m = (rng.random((B, 1, M, N)) < 0.3).astype(np.int8)
        m[..., 0] = 0                                     # never a fully masked row
        kw["mask"] = m
        tkw["attn_mask"] = torch.from_numpy(m == 0)       # torch: True = keep
    if case == "scale":
        kw["scale"] = 0.37
        tkw["scale"] = 0.37
    O, P = so.sdpa_forward_f64(Q, K, V, **kw)
    ref = torch.nn.functional.scaled_dot_product_attention(torch.from_numpy(Q), torch.from_numpy(K), torch.from_numpy(V),
                                                           **tkw).numpy()
    np.testing.assert_allclose(O, ref, rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(P.sum(-1), 1.0, rtol=1e-12)
