"""TEST INFRASTRUCTURE ONLY -- Python face of the CPU oracle for the dense-layer path.

Two kinds of checker:
  * fp32-exact: the C restatement in dense_oracle.c (one fmaf chain per output, k ascending, the reference's
    epilogue order), called through ctypes; rows are split over host threads (rows are independent, so the
    split changes no result).
  * float64: NumPy evaluation of the same formulas in double precision, for the bf16 / TF32 tensor-core
    paths whose contract is a relative Frobenius error.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
Parity pin: tests/test_oracle.py checks it against tests/golden/*.npz (made by tests/golden/make_golden.py
from the reference's own host-compiled epilogue code).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ACT = {"none": 0, "relu": 1, "leaky_relu": 2, "gelu": 3, "sigmoid": 4, "tanh": 5}
BIAS_NONE, BIAS_SCALAR, BIAS_PER_M, BIAS_PER_N = 0, 1, 2, 3

_lib = None
_fp = C.POINTER(C.c_float)


def build() -> Path:
    """Compiles liboracle.so (gcc) if it is missing or older than its source."""
    so, src = HERE / "liboracle.so", HERE / "dense_oracle.c"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "liboracle.so"], check=True, capture_output=True)
    return so


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        _lib.oracle_act.restype = C.c_float
        _lib.oracle_act.argtypes = [C.c_int, C.c_float, C.c_float]
        _lib.oracle_act_deriv.restype = C.c_float
        _lib.oracle_act_deriv.argtypes = [C.c_int, C.c_float, C.c_float]
    return _lib


def n_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def _p(a, off=0):
    if a is None:
        return None
    return C.cast(a.ctypes.data + off * 4, _fp)


def _f32c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def bias_kind_of(bias, M, N) -> int:
    if bias is None:
        return BIAS_NONE
    n = int(np.size(bias))
    s = tuple(np.shape(bias))
    if s in ((1,), (1, 1)):
        return BIAS_SCALAR
    if s in ((N,), (1, N)):
        return BIAS_PER_N
    if s in ((M,), (M, 1)):
        return BIAS_PER_M
    return BIAS_PER_N if n == N else BIAS_PER_M if n == M else BIAS_SCALAR


def _chunks(n, parts):
    parts = max(1, min(parts, n))
    step = (n + parts - 1) // parts
    return [(i, min(n, i + step)) for i in range(0, n, step)]


# ------------------------------------------------------------------ fp32-exact
def forward_f32(A, B, bias=None, act="none", leaky=0.01, alpha=1.0, beta=0.0, Cin=None, trans_b=False,
                threads=None):
    """Returns (Y, Z) in float32, bit-for-bit what the reference's fp32 forward computes for Z."""
    A, B, Cin = _f32c(A), _f32c(B), _f32c(Cin)
    M, K = A.shape
    N = B.shape[0] if trans_b else B.shape[1]
    bias_c = _f32c(np.reshape(bias, -1)) if bias is not None else None
    kind = bias_kind_of(bias, M, N)
    Y = np.empty((M, N), np.float32)
    Z = np.empty((M, N), np.float32)
    L = lib()

    def run(rng):
        m0, m1 = rng
        L.oracle_dense_forward_f32(
            _p(A, m0 * K), K, _p(B), B.shape[1], int(trans_b), _p(Cin, m0 * N) if Cin is not None else None, N,
            _p(bias_c, m0 if kind == BIAS_PER_M else 0) if bias_c is not None else None, kind,
            _p(Y, m0 * N), N, _p(Z, m0 * N), N, m1 - m0, N, K,
            C.c_float(alpha), C.c_float(beta), ACT[act], C.c_float(leaky))

    with ThreadPoolExecutor(threads or n_threads()) as ex:
        list(ex.map(run, _chunks(M, threads or n_threads())))
    return Y, Z


def backward_f32(A, B, gY, Z, act="none", leaky=0.01, alpha=1.0, beta=0.0, bias_kind=BIAS_PER_N, want_gC=False,
                 threads=None):
    """Returns dict(gZ, gA, gB, gBias[, gC]) in float32."""
    A, B, gY, Z = map(_f32c, (A, B, gY, Z))
    M, K = A.shape
    N = B.shape[1]
    gZ = np.empty((M, N), np.float32)
    gC = np.empty((M, N), np.float32) if want_gC else None
    nb = {BIAS_SCALAR: 1, BIAS_PER_M: M, BIAS_PER_N: N}.get(bias_kind, 0)
    gBias = np.zeros(nb, np.float32) if nb else None
    L = lib()
    L.oracle_dense_bwd_prologue_f32(_p(gY), N, _p(Z), N, _p(gZ), _p(gC), N, C.c_float(beta), _p(gBias), bias_kind,
                                    M, N, ACT[act], C.c_float(leaky))
    gA = np.empty((M, K), np.float32)
    gB = np.empty((K, N), np.float32)
    nt = threads or n_threads()

    def run_ga(rng):
        m0, m1 = rng
        L.oracle_dense_bwd_gemms_f32(_p(A, m0 * K), K, _p(B), N, _p(gZ, m0 * N), _p(gA, m0 * K), K, None, N,
                                     m1 - m0, N, K, C.c_float(alpha))

    def run_gb(rng):
        k0, k1 = rng   # a block of columns of A = rows of gB
        L.oracle_dense_bwd_gemms_f32(_p(A, k0), K, _p(B), N, _p(gZ), None, K, _p(gB, k0 * N), N,
                                     M, N, k1 - k0, C.c_float(alpha))

    with ThreadPoolExecutor(nt) as ex:
        list(ex.map(run_ga, _chunks(M, nt)))
        list(ex.map(run_gb, _chunks(K, nt)))
    out = {"gZ": gZ, "gA": gA, "gB": gB, "gBias": gBias}
    if want_gC:
        out["gC"] = gC
    return out


def act_f32(kind: str, x, leaky=0.01):
    x = _f32c(x)
    y = np.empty_like(x)
    lib().oracle_act_array(ACT[kind], _p(x), _p(y), C.c_size_t(x.size), C.c_float(leaky))
    return y


def act_deriv_f32(kind: str, x, leaky=0.01):
    x = _f32c(x)
    y = np.empty_like(x)
    lib().oracle_act_deriv_array(ACT[kind], _p(x), _p(y), C.c_size_t(x.size), C.c_float(leaky))
    return y


# ------------------------------------------------------------------ float64
_C0, _K1 = 0.7978845608, 0.044715


def act_f64(kind, x, leaky=0.01):
    x = np.asarray(x, np.float64)
    if kind == "relu":
        return np.where(x > 0, x, 0.0)
    if kind == "leaky_relu":
        return np.where(x > 0, x, leaky * x)
    if kind == "gelu":
        return 0.5 * x * (1.0 + np.tanh(_C0 * (x + _K1 * x ** 3)))
    if kind == "sigmoid":
        return 1.0 / (1.0 + np.exp(-x))
    if kind == "tanh":
        return np.tanh(x)
    return x


def act_deriv_f64(kind, x, leaky=0.01):
    x = np.asarray(x, np.float64)
    if kind == "relu":
        return (x > 0).astype(np.float64)
    if kind == "leaky_relu":
        return np.where(x > 0, 1.0, leaky)
    if kind == "gelu":
        th = np.clip(np.tanh(_C0 * (x + _K1 * x ** 3)), -0.999999, 0.999999)
        return 0.5 * (1 + th) + 0.5 * x * (1 - th * th) * _C0 * (1 + 3 * _K1 * x * x)
    if kind == "sigmoid":
        s = 1.0 / (1.0 + np.exp(-x))
        return s * (1 - s)
    if kind == "tanh":
        return 1 - np.tanh(x) ** 2
    return np.ones_like(x)


def forward_f64(A, B, bias=None, act="none", leaky=0.01, alpha=1.0, trans_b=False):
    A = np.asarray(A, np.float64)
    B = np.asarray(B, np.float64)
    Zv = alpha * (A @ (B.T if trans_b else B))
    if bias is not None:
        M, N = Zv.shape
        b = np.asarray(bias, np.float64)
        kind = bias_kind_of(bias, M, N)
        Zv = Zv + (b.reshape(1, N) if kind == BIAS_PER_N else b.reshape(M, 1) if kind == BIAS_PER_M else b.reshape(()))
    return act_f64(act, Zv, leaky), Zv


def backward_f64(A, B, gY, Z, act="none", leaky=0.01):
    A, B, gY, Z = (np.asarray(t, np.float64) for t in (A, B, gY, Z))
    gZ = gY * act_deriv_f64(act, Z, leaky)
    return {"gZ": gZ, "gA": gZ @ B.T, "gB": A.T @ gZ, "gBias": gZ.sum(axis=0)}


def softmax_ce_f64(logits, labels, grad_scale=None, ignore_index=-1, denom=None):
    """Per-row loss and dlogits = (softmax - onehot) * grad_scale in float64.  Ignored rows give zeros; the mean
    divides by `denom` (default: all rows, ignored ones included, as the reference's native op does)."""
    x = np.asarray(logits, np.float64)
    M, Cn = x.shape
    denom = M if denom is None else denom
    grad_scale = 1.0 / denom if grad_scale is None else grad_scale
    m = x.max(axis=1, keepdims=True)
    e = np.exp(x - m)
    s = e.sum(axis=1, keepdims=True)
    lab = np.asarray(labels, np.int64)
    live = (lab != ignore_index) & (lab >= 0) & (lab < Cn)
    safe = np.where(live, lab, 0)
    loss_rows = np.where(live, (m[:, 0] + np.log(s[:, 0])) - x[np.arange(M), safe], 0.0)
    d = e / s
    d[np.arange(M), safe] -= 1.0
    d = d * grad_scale * live[:, None]
    return loss_rows, d


def sgd_f64(p, g, v=None, lr=1e-3, momentum=0.0, dampening=0.0, nesterov=False, weight_decay=0.0, decay="decoupled",
            grad_scale=1.0):
    p = np.asarray(p, np.float64)
    g = grad_scale * np.asarray(g, np.float64)
    if weight_decay and decay == "l2":
        g = g + weight_decay * p
    step = g
    if momentum > 0 and v is not None:
        v = momentum * np.asarray(v, np.float64) + (1 - dampening) * g
        step = g + momentum * v if nesterov else v
    dec = lr * weight_decay * p if (weight_decay and decay == "decoupled") else 0.0
    return p - lr * step - dec, v


def mlp_step_f64(W32, b, X, labels, acts, lr, global_batch=None, lowp=None):
    """One training step of Dense stack -> softmax-CE (mean) -> SGD in float64.  W32/b are lists (float64 master
    copies); the forward uses `lowp(W)` (e.g. bf16 rounding) when given.  Returns (loss, new_W32, new_b, grads)."""
    n = len(W32)
    B = X.shape[0]
    gb = B if global_batch is None else global_batch
    a, zs, ins = np.asarray(X, np.float64), [], []
    for i in range(n):
        Wf = np.asarray(lowp(W32[i].astype(np.float32)), np.float64) if lowp else W32[i]
        ins.append(a)
        z = a @ Wf + b[i]
        zs.append(z)
        a = act_f64(acts[i], z)
    loss_rows, g = softmax_ce_f64(a, labels, grad_scale=1.0 / gb)
    loss = loss_rows.sum() / gb
    newW, newb, grads = list(W32), list(b), [None] * n
    for i in reversed(range(n)):
        Wf = np.asarray(lowp(W32[i].astype(np.float32)), np.float64) if lowp else W32[i]
        gz = g * act_deriv_f64(acts[i], zs[i])
        gW, gbias = ins[i].T @ gz, gz.sum(axis=0)
        g = gz @ Wf.T
        grads[i] = (gW, gbias)
        newW[i] = W32[i] - lr * gW
        newb[i] = b[i] - lr * gbias
    return loss, newW, newb, grads


def rel_fro(x, ref) -> float:
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(x - ref) / (den if den > 0 else 1.0))


def max_rel(x, ref, floor=1e-5) -> float:
    """max |x-ref| / max(|ref|, 1) scaled so that `floor` absolute error on small values counts like the
    reference tests' atol: returns max(|x-ref| / (floor_abs + |ref|)) with floor_abs = 1."""
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(x - ref) / (1.0 + np.abs(ref)))) if x.size else 0.0


# ------------------------------------------------------------------ inputs
def bf16_round(x):
    """float32 -> nearest-even bfloat16, returned as float32 values."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def dense_inputs(M, K, N, seed=0, bias_zero=False):
    """Inputs of the benchmark configurations: X, dY ~ N(0,1); W ~ U(+-sqrt(6/K)); b ~ U(-0.1, 0.1).
    Generator: numpy.random.default_rng(seed) (PCG64), drawn in the order X, W, b, dY, as float32."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((M, K), dtype=np.float32)
    lim = np.float32(np.sqrt(6.0 / K))
    W = rng.uniform(-lim, lim, (K, N)).astype(np.float32)
    b = np.zeros(N, np.float32) if bias_zero else rng.uniform(-0.1, 0.1, N).astype(np.float32)
    dY = rng.standard_normal((M, N), dtype=np.float32)
    return X, W, b, dY
