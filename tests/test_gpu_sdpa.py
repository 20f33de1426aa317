"""Fused attention forward (ge2b_sdpa_forward) against the float64 oracle of the reference's SDPA sequence.
bf16 tensors; tolerance of the 16-bit tensor-core paths: relative Frobenius <= 2e-2 over the output and every
128 x 128 block within 5e-3 (P is rounded to bf16 before P.V, O once at the end)."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from parity_util import check_close  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def so():
    return importlib.import_module("oracle.sdpa_oracle")


def _bf(a):
    return torch.from_numpy(a).cuda().bfloat16()


def _f64(t):
    return t.detach().double().cpu().numpy()


@pytest.mark.parametrize("shape", [(2, 3, 256, 256, 128), (1, 2, 200, 333, 128), (2, 2, 128, 640, 64), (1, 1, 1, 7, 64),
                                   (1, 4, 384, 128, 128)])
@pytest.mark.parametrize("mode", ["plain", "causal", "float_mask", "int8_mask", "int32_mask", "scale"])
def test_sdpa_forward_matches_oracle(pkg, lib, so, shape, mode):
    B, H, M, N, D = shape
    if mode == "causal":
        N = M
    rng = np.random.default_rng(sum(shape) * 7 + len(mode))
    Q, K, V = (_bf(rng.standard_normal(s, dtype=np.float32)) for s in ((B, H, M, D), (B, H, N, D), (B, H, N, D)))
    kw, okw = {}, {}
    if mode == "causal":
        kw["causal"] = okw["causal"] = True
    elif mode == "float_mask":
        m = rng.standard_normal((B, 1, M, N)).astype(np.float32) * 2
        kw["mask"], okw["mask"] = torch.from_numpy(m).cuda(), m
    elif mode in ("int8_mask", "int32_mask"):
        m = (rng.random((B, 1, M, N)) < 0.4).astype(np.int8 if mode == "int8_mask" else np.int32)
        m[..., 0] = 0                                           # no fully masked row (see the edge-case test)
        kw["mask"], okw["mask"] = torch.from_numpy(m).cuda(), m
    elif mode == "scale":
        kw["scale"] = okw["scale"] = 0.21
    lse = torch.empty((B, H, M), device="cuda")
    O = pkg.ops_sdpa.forward(Q, K, V, lse=lse, **kw)
    torch.cuda.synchronize()
    assert lib.ge2b_device_status(1) == 0
    O64, P64 = so.sdpa_forward_f64(_f64(Q), _f64(K), _f64(V), **okw)
    check_close("O", _f64(O).reshape(B * H * M, D), O64.reshape(B * H * M, D))
    # log-sum-exp of the scaled, masked scores
    sc = okw.get("scale", 0.0) or 1.0 / np.sqrt(D)
    S = sc * np.einsum("bhmd,bhnd->bhmn", _f64(Q), _f64(K))
    if mode == "causal":
        S = S + np.where(np.arange(N)[None, :] > np.arange(M)[:, None], -np.inf, 0.0)
    if "mask" in okw:
        S = S + (np.where(okw["mask"] != 0, -np.inf, 0.0) if okw["mask"].dtype.kind == "i" else okw["mask"])
    want = np.log(np.exp(S - S.max(-1, keepdims=True)).sum(-1)) + S.max(-1)
    np.testing.assert_allclose(lse.cpu().numpy(), want, rtol=2e-3, atol=2e-3)


def test_sdpa_fully_masked_row_gives_zeros(pkg, lib):
    """Every key of a row masked out: the fused kernel returns zeros for that row (the reference adds -1e9 to every
    score of the row, which cancels in the softmax and returns the unmasked attention; a row without keys has no
    meaningful answer, and zeros do not poison the next layer)."""
    B, H, M, N, D = 1, 2, 130, 140, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    Q, K, V = (torch.randn(s, device="cuda", generator=g).bfloat16() for s in ((B, H, M, D), (B, H, N, D), (B, H, N, D)))
    mask = torch.zeros((B, 1, M, N), device="cuda", dtype=torch.int8)
    mask[0, 0, 5, :] = 1
    O = pkg.ops_sdpa.forward(Q, K, V, mask=mask)
    torch.cuda.synchronize()
    assert torch.all(O[:, :, 5] == 0) and torch.isfinite(O.float()).all()
    O2 = pkg.ops_sdpa.forward(Q, K, V)
    assert torch.equal(O[:, :, 6:], O2[:, :, 6:])              # other rows untouched by the mask


def test_sdpa_unsupported_arguments_are_refused(pkg, lib):
    Q = torch.zeros((1, 1, 8, 32), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="-99"):
        pkg.ops_sdpa.forward(Q, Q, Q)                           # head dimension 32
    Q = torch.zeros((1, 1, 8, 64), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="-99"):
        pkg.ops_sdpa.forward(Q, Q, Q, dropout_p=0.1)
    with pytest.raises(ValueError):
        pkg.ops_sdpa.forward(Q.float(), Q.float(), Q.float())


def test_sdpa_full_size_config4(pkg, lib, so):
    """B = 8, H = 16, L = 2048, d = 128 in one launch; sampled (batch, head) slices against float64, and the two-GEMM
    form of the same computation (S and P through HBM) as a cross-check on one slice."""
    Bn, H, L, d = 8, 16, 2048, 128
    g = torch.Generator(device="cuda").manual_seed(44)
    Q, K, V = (torch.randn((Bn, H, L, d), device="cuda", generator=g).bfloat16() for _ in range(3))
    O = pkg.ops_sdpa.forward(Q, K, V)
    Oc = pkg.ops_sdpa.forward(Q, K, V, causal=True)
    torch.cuda.synchronize()
    assert lib.ge2b_device_status(1) == 0
    for (bi, hi) in ((0, 0), (3, 7), (7, 15)):
        q, k, v = (_f64(t[bi:bi + 1, hi:hi + 1]) for t in (Q, K, V))
        check_close(f"O[{bi},{hi}]", _f64(O[bi, hi]), so.sdpa_forward_f64(q, k, v)[0][0, 0])
        check_close(f"O causal[{bi},{hi}]", _f64(Oc[bi, hi]), so.sdpa_forward_f64(q, k, v, causal=True)[0][0, 0])
    S = torch.empty((1, 1, L, L), device="cuda", dtype=torch.bfloat16)
    pkg.ops_gemm.forward_batched(Q[7:8, 15:16], K[7:8, 15:16], out=S, trans_b=True, alpha=1.0 / d ** 0.5)
    P = torch.softmax(S.float(), dim=-1).bfloat16()
    O2 = torch.empty((1, 1, L, d), device="cuda", dtype=torch.bfloat16)
    pkg.ops_gemm.forward_batched(P, V[7:8, 15:16], out=O2)
    torch.cuda.synchronize()
    assert float((O2[0, 0].float() - O[7, 15].float()).norm() / O[7, 15].float().norm()) <= 2e-2
