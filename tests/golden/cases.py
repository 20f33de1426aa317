"""Input recipes of the golden cases: the seeds, shapes and draw order of the reference's own GEMM tests,
regenerated from NumPy's default_rng rather than stored.

  smoke_*   graph_executor_v2/tests/cuda_pyd_test/smoke_gemm_binding.py:130-147 (also python_glue_test/glue_gemm.py
            and layer_test/dense_gemm.py): default_rng(2025), standard_normal, draw order A, B, gY, bias(1,N);
            m,k,n = 32,64,16
  legacy_*  dev/backend/graph_executor_v2/test/ge2_check_backward_debug.py:44-60,104,197-210 and ge2_verify_preact.py:
            default_rng(0), standard_normal, draw order A, B, C, then gY; constant bias 0.1; alpha 1.1, beta 0.9,
            leaky 0.02
  relu128   dev/backend/graph_executor_v2/test/test_gemm_bias_relu.py:6-12: default_rng(123).uniform(-1,1), 128^3,
            bias 0.10 per column
  config1   the 256x512x512 ReLU plumbing case (dev/smoke_compiler.py:13-21 shape), seed 0
"""
import numpy as np

BIAS_NONE, BIAS_SCALAR, BIAS_PER_M, BIAS_PER_N = 0, 1, 2, 3


def smoke_case(act, with_bias, m=32, k=64, n=16, leaky=0.01):
    rng = np.random.default_rng(2025)
    A = rng.standard_normal((m, k), dtype=np.float32)
    B = rng.standard_normal((k, n), dtype=np.float32)
    gY = rng.standard_normal((m, n), dtype=np.float32)
    bias = rng.standard_normal((1, n), dtype=np.float32) if with_bias else None
    return dict(A=A, B=B, C=None, gY=gY, bias=bias, bias_kind=BIAS_PER_N if with_bias else BIAS_NONE, act=act,
                leaky=leaky, alpha=1.0, beta=0.0)


def legacy_case(M, N, K, act, bias_kind, use_C, leaky=0.02, seed=0, alpha=1.1, beta=0.9):
    rng = np.random.default_rng(seed)
    A = rng.standard_normal((M, K), np.float32)
    B = rng.standard_normal((K, N), np.float32)
    C = rng.standard_normal((M, N), np.float32)
    bias = {BIAS_SCALAR: np.array([0.1], np.float32), BIAS_PER_M: np.full((M,), 0.1, np.float32),
            BIAS_PER_N: np.full((N,), 0.1, np.float32)}[bias_kind]
    gY = rng.standard_normal((M, N), np.float32)
    return dict(A=A, B=B, C=C if use_C else None, gY=gY, bias=bias, bias_kind=bias_kind, act=act, leaky=leaky,
                alpha=alpha, beta=beta if use_C else 0.0)


def relu128_case():
    rng = np.random.default_rng(123)
    A = rng.uniform(-1, 1, size=(128, 128)).astype(np.float32)
    B = rng.uniform(-1, 1, size=(128, 128)).astype(np.float32)
    gY = rng.standard_normal((128, 128), dtype=np.float32)
    return dict(A=A, B=B, C=None, gY=gY, bias=np.full((128,), 0.10, np.float32), bias_kind=BIAS_PER_N, act="relu",
                leaky=0.01, alpha=1.0, beta=0.0)


def config1_case():
    rng = np.random.default_rng(0)
    X = rng.standard_normal((256, 512), dtype=np.float32)
    lim = np.float32(np.sqrt(6.0 / 512))
    W = rng.uniform(-lim, lim, (512, 512)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 512).astype(np.float32)
    dY = rng.standard_normal((256, 512), dtype=np.float32)
    return dict(A=X, B=W, C=None, gY=dY, bias=b, bias_kind=BIAS_PER_N, act="relu", leaky=0.01, alpha=1.0, beta=0.0)


CASES = {
    "smoke_bias_relu": lambda: smoke_case("relu", True),
    "smoke_nobias_none": lambda: smoke_case("none", False),
    "smoke_bias_gelu": lambda: smoke_case("gelu", True),
    "smoke_bias_sigmoid": lambda: smoke_case("sigmoid", True),
    "smoke_bias_tanh": lambda: smoke_case("tanh", True),
    "smoke_bias_leaky": lambda: smoke_case("leaky_relu", True, leaky=0.02),
    "legacy_gelu_pern_c": lambda: legacy_case(64, 48, 32, "gelu", BIAS_PER_N, True),
    "legacy_relu_scalar": lambda: legacy_case(64, 64, 32, "relu", BIAS_SCALAR, False),
    "legacy_leaky_perm_c": lambda: legacy_case(96, 80, 40, "leaky_relu", BIAS_PER_M, True),
    "legacy_gelu_pern_c_seed1": lambda: legacy_case(64, 48, 32, "gelu", BIAS_PER_N, True, seed=1),
    "relu128": relu128_case,
    "config1": config1_case,
}
