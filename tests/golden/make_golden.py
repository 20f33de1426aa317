"""Generates tests/golden/*.npz by running the reference's own host-compilable epilogue code
(oracle/_ref/libref_host.so, built by `make -C oracle ref` from the mounted reference tree) on the inputs of
cases.py.  Run it where the reference tree is mounted; the .npz files are committed, the library is not.

Stored per case: Y, Z (forward through the reference's apply_epilogue_scalar over an ascending-k fmaf GEMM),
gZ (gY times the reference's template activation derivative) and 64 probe points of the activation and its
derivative.  gA / gB / gBias are products and sums of gZ that the reference delegates to cuBLAS and atomics;
they are checked against float64 in the tests, not stored.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from cases import CASES  # noqa: E402

ACT = {"none": 0, "relu": 1, "leaky_relu": 2, "gelu": 3, "sigmoid": 4, "tanh": 5}
fp = C.POINTER(C.c_float)


def p(a):
    return None if a is None else a.ctypes.data_as(fp)


def main():
    so = HERE.parent.parent / "oracle" / "_ref" / "libref_host.so"
    lib = C.CDLL(str(so))
    lib.ref_act_runtime.restype = C.c_float
    lib.ref_act_runtime.argtypes = [C.c_int, C.c_float, C.c_float]
    lib.ref_act_deriv.restype = C.c_float
    lib.ref_act_deriv.argtypes = [C.c_int, C.c_float, C.c_float]
    for name, make in CASES.items():
        c = make()
        A, B, Cin, gY = c["A"], c["B"], c["C"], c["gY"]
        M, K = A.shape
        N = B.shape[1]
        bias = None if c["bias"] is None else np.ascontiguousarray(c["bias"].reshape(-1))
        Y = np.empty((M, N), np.float32)
        Z = np.empty((M, N), np.float32)
        lib.ref_dense_forward_f32(p(A), K, p(B), N, p(Cin), N, p(bias), c["bias_kind"], p(Y), N, p(Z), N, M, N, K,
                                  C.c_float(c["alpha"]), C.c_float(c["beta"]), ACT[c["act"]], C.c_float(c["leaky"]))
        gZ = np.empty((M, N), np.float32)
        lib.ref_dense_bwd_gz_f32(p(gY), N, p(Z), N, p(gZ), M, N, ACT[c["act"]], C.c_float(c["leaky"]))
        probe = np.linspace(-6, 6, 64, dtype=np.float32)
        a = np.array([lib.ref_act_runtime(ACT[c["act"]], float(x), c["leaky"]) for x in probe], np.float32)
        d = np.array([lib.ref_act_deriv(ACT[c["act"]], float(x), c["leaky"]) for x in probe], np.float32)
        np.savez_compressed(HERE / f"{name}.npz", Y=Y, Z=Z, gZ=gZ, probe=probe, act_probe=a, deriv_probe=d)
        print(name, Y.shape, float(np.abs(Y).mean()))


if __name__ == "__main__":
    main()
