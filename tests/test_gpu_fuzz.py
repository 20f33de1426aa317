"""Seeded sweep of awkward shapes through every store path of the tensor-core GEMM (32- and 64-column bulk stores, fp32
outputs, the row-wise fall-back for unaligned pitches, split-K, batched, transposed operands, the backward pair) against
float64 products of the same rounded inputs (torch.float64 matmul on the device).  Tolerance: relative Frobenius
error <= 2e-2, the bound of the bf16 / TF32 paths."""
import random

import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu
TOL = 2e-2
MS = [1, 7, 31, 32, 33, 127, 128, 129, 255, 256, 257, 300, 511, 640, 1000, 1500]
NS = [8, 16, 24, 40, 64, 72, 120, 128, 136, 200, 256, 264, 320, 392, 520, 1000, 1416]
KS = [8, 16, 40, 64, 72, 128, 200, 264, 520, 1032]


LOCAL_TOL, BLOCK = 5e-3, 128     # every 128 x 128 block of every output (see tests/parity_util.py)


def block_err(a, b):
    """worst relative Frobenius error over 128 x 128 blocks, on the device (blocks much quieter than the tensor's RMS
    are measured against 5 % of that RMS)"""
    a, b = a.double().reshape(-1, a.shape[-1]), b.double().reshape(-1, b.shape[-1])
    R, C = b.shape
    pr, pc = -(-R // BLOCK) * BLOCK, -(-C // BLOCK) * BLOCK
    pad = lambda t: torch.nn.functional.pad(t, (0, pc - C, 0, pr - R))                          # noqa: E731
    fold = lambda t: pad(t).reshape(pr // BLOCK, BLOCK, pc // BLOCK, BLOCK).sum(dim=(1, 3))     # noqa: E731
    E, N2, n = fold((a - b) ** 2), fold(b * b), fold(torch.ones_like(b))
    floor = (0.05 ** 2) * (b * b).mean() * n
    return float(torch.sqrt(E / torch.maximum(torch.maximum(N2, floor), torch.tensor(1e-300, device=b.device))).max())


def rel(a, b):
    """relative Frobenius error; a block that breaks the local bound is reported as a failure of the whole tensor"""
    e = float((a.double() - b).norm() / (b.norm() + 1e-30))
    if a.dim() >= 2 and block_err(a, b) > LOCAL_TOL:
        return max(e, 1.0)
    return e


@pytest.mark.parametrize("mode", ["plain", "full", "full_z32", "batched", "trans_b", "backward"])
def test_random_shapes(pkg, lib, mode):
    g = pkg.ops_gemm
    rnd = random.Random(7 + ["plain", "full", "full_z32", "batched", "trans_b", "backward"].index(mode))
    torch.manual_seed(11)
    worst = []
    for _ in range(24):
        M, N, K = rnd.choice(MS), rnd.choice(NS), rnd.choice(KS)
        dt = rnd.choice([torch.bfloat16, torch.bfloat16, torch.float32])
        math = "tf32" if dt == torch.float32 else "fp32"
        A = torch.randn(M, K, device="cuda").to(dt)
        B = (torch.randn(K, N, device="cuda") / K ** 0.5).to(dt)
        bias = torch.randn(N, device="cuda")
        if mode == "plain":
            out = torch.empty(M, N, device="cuda", dtype=dt)
            g.forward_into(A, B, out=out, math=math)
            e = rel(out, A.double() @ B.double())
        elif mode in ("full", "full_z32"):
            out = torch.empty(M, N, device="cuda", dtype=dt)
            z = torch.empty(M, N, device="cuda", dtype=torch.float32 if mode == "full_z32" else dt)
            g.forward_into(A, B, out=out, bias=bias, with_bias=True, act="gelu", save_z=True, z_out=z, math=math)
            zr = A.double() @ B.double() + bias.double()
            e = max(rel(out, torch.nn.functional.gelu(zr, approximate="tanh")), rel(z, zr))
        elif mode == "batched":
            bn = rnd.choice([2, 3, 5])
            A3 = torch.randn(bn, M, K, device="cuda").to(dt)
            B3 = (torch.randn(bn, K, N, device="cuda") / K ** 0.5).to(dt)
            out = torch.empty(bn, M, N, device="cuda", dtype=dt)
            g.forward_batched(A3, B3, out=out, alpha=0.5, math=math)
            e = rel(out, 0.5 * (A3.double() @ B3.double()))
        elif mode == "trans_b":
            Bt = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dt)
            out = torch.empty(M, N, device="cuda", dtype=dt)
            g.forward_into(A, Bt, out=out, trans_b=True, math=math)
            e = rel(out, A.double() @ Bt.double().T)
        else:
            dY = torch.randn(M, N, device="cuda").to(dt)
            Z = torch.randn(M, N, device="cuda").to(dt)
            gA, gB = torch.empty_like(A), torch.empty_like(B)
            gb, work = torch.empty(N, device="cuda"), torch.empty_like(dY)
            g.backward_into(A, B, dY, Z, act="relu", with_bias=True, gA_out=gA, gB_out=gB, gBias_out=gb, work_dZ=work,
                            math=math)
            gz = dY.double() * (Z.double() > 0)
            gzr = work.double() if dt != torch.float32 else gz      # the GEMMs read the rounded gZ
            e = max(rel(gA, gzr @ B.double().T), rel(gB, A.double().T @ gzr), rel(gb, gz.sum(0)))
        torch.cuda.synchronize()
        if not e <= TOL:
            worst.append((M, N, K, str(dt), e))
    assert not worst, worst
    assert lib.ge2b_device_status(1) == 0
