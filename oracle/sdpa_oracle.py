"""TEST INFRASTRUCTURE ONLY -- CPU restatement (NumPy float64) of the reference's scaled-dot-product attention forward.

Follows backends/cuda/ops/sdpa/launcher.cu:129-270 step by step, per (batch, head) slice:
  scale = attrs.scale or 1/sqrt(D)                         (:162)
  S = scale * Q[b,h] @ K[b,h]^T                            (:185-222; the reference transposes K, multiplies, then scales)
  causal: S[m, n] += -1e9 for n > m                        (:38-48, NEG at :163)
  mask [B,1,M,N]: int8 / int32 -> S += -1e9 where non-zero; float32 -> S += mask      (:56-95, slice offsets :166-170)
  P = softmax(S, axis=-1)
  O = P @ V[b,h]                                           (:236-270)
Only tests/ may import this module.  Parity pin: the reference's SDPA op cannot be compiled outside its own build
(it needs a second tensor header that clashes with the shim's), so this restatement is pinned by construction against
torch.nn.functional.scaled_dot_product_attention on the CPU (tests/test_oracle_sdpa.py), not against the reference's
binary: "parity unpinned" with respect to the reference itself.
"""
from __future__ import annotations

import numpy as np

NEG = -1e9


def sdpa_forward_f64(Q, K, V, mask=None, causal=False, scale=0.0):
    Q, K, V = (np.asarray(a, np.float64) for a in (Q, K, V))
    B, H, M, D = Q.shape
    N = K.shape[2]
    sc = scale if scale != 0.0 else 1.0 / np.sqrt(D)
    S = sc * np.einsum("bhmd,bhnd->bhmn", Q, K)
    if causal:
        m_idx, n_idx = np.arange(M)[:, None], np.arange(N)[None, :]
        S = S + np.where(n_idx > m_idx, NEG, 0.0)
    if mask is not None:
        mask = np.asarray(mask)
        assert mask.shape == (B, 1, M, N)
        if mask.dtype.kind in "iu":
            S = S + np.where(mask != 0, NEG, 0.0)
        else:
            S = S + mask.astype(np.float64)
    S = S - S.max(axis=-1, keepdims=True)
    P = np.exp(S)
    P /= P.sum(axis=-1, keepdims=True)
    lse = None
    return np.einsum("bhmn,bhnd->bhmd", P, V), P
