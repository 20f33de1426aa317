"""Error measures shared by the GPU parity tests.

The contract of the bf16 / f16 / TF32 paths is a relative Frobenius error <= 2e-2 over a whole tensor.  That number
is blind to a localised fault (one wrong row of 4096 moves it by 1.6e-2), so every comparison also applies a LOCAL
bound: the tensor is cut into 128 x 128 blocks (the finest unit any kernel here stores by itself is coarser than
32 x 32, so a misplaced or stale fragment is a large part of a block) and each block's relative Frobenius error must
stay below 5e-3 -- a few times what rounding alone gives (one bf16 rounding of the output: 2^-9 / sqrt(3) = 1.1e-3;
TF32 truncation of both operands: about 1.2e-3; bf16 gZ feeding the backward GEMMs: another 1.1e-3).
"""
import numpy as np

FRO_TOL = 2e-2      # whole tensor, the contract
LOCAL_TOL = 5e-3    # every 128 x 128 block
BLOCK = 128


def rel_fro(got, ref) -> float:
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(got - ref) / (den if den > 0 else 1.0))


def block_rel_fro(got, ref, block=BLOCK):
    """Worst relative Frobenius error over the block x block tiles of a 2-D (or flattened-to-2-D) pair, and where.
    A block whose reference is (nearly) all zero -- ReLU of a negative region -- is measured against the tensor's
    RMS instead, so that it neither divides by zero nor hides a fault."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    if got.ndim == 1:
        got, ref = got[None, :], ref[None, :]
    if got.ndim > 2:
        got, ref = got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1])
    assert got.shape == ref.shape, (got.shape, ref.shape)
    R, C = ref.shape
    rms = np.sqrt(np.mean(ref * ref)) if ref.size else 0.0
    pr, pc = -(-R // block) * block, -(-C // block) * block
    e2 = np.zeros((pr, pc)); r2 = np.zeros((pr, pc)); cnt = np.zeros((pr, pc))
    e2[:R, :C] = (got - ref) ** 2; r2[:R, :C] = ref * ref; cnt[:R, :C] = 1.0
    fold = lambda a: a.reshape(pr // block, block, pc // block, block).sum(axis=(1, 3))   # noqa: E731
    E, N2, n = fold(e2), fold(r2), fold(cnt)
    floor = (0.05 * rms) ** 2 * n                     # blocks quieter than 5 % of the tensor's RMS use this instead
    err = np.sqrt(E / np.maximum(np.maximum(N2, floor), 1e-300))
    i = np.unravel_index(int(np.argmax(err)), err.shape)
    return float(err[i]), (int(i[0]), int(i[1]))


def check_close(name, got, ref, fro_tol=FRO_TOL, local_tol=LOCAL_TOL, block=BLOCK):
    """Asserts the contract bound and the local bound; returns (fro, worst_block_error)."""
    f = rel_fro(got, ref)
    assert f <= fro_tol, f"{name}: relative Frobenius error {f:.3e} > {fro_tol}"
    w, at = block_rel_fro(got, ref, block)
    assert w <= local_tol, f"{name}: block {at} of {block}x{block} has relative Frobenius error {w:.3e} > {local_tol}"
    return f, w
