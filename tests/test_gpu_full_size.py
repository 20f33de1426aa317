"""Parity at the full sizes of the benchmark configurations: the shapes that are timed are also checked.

  * squares 8192^3 and 16384^3 (bf16, GELU, forward + backward): float64 references on sampled rows and columns, at
    least one row and one column through EVERY 256 x 256 tile of every output, each tile's segment held to the local
    bound (5e-3) as well as the whole sample to the contract's 2e-2.  16384^3 runs 64 x 64 tile grids with the
    rasterisation in groups of 8 row-blocks, which nothing smaller reaches.
  * the attention GEMMs at B*H = 128, L = 2048, d = 128: sampled (batch, head) slices including the first and the last.
  * the 3-layer MLP step at batch 8192, 1024-4096-4096-1024: loss, sampled rows of every dW, every db.
Inputs are seeded and drawn on the device (a 16384^2 matrix is 1 GiB in fp32); references are float64 on the host.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from parity_util import FRO_TOL, LOCAL_TOL, check_close, rel_fro  # noqa: E402

pytestmark = pytest.mark.gpu
TILE = 256


def _f64(t):
    return t.detach().double().cpu().numpy()


def _one_per_block(n, rng):
    """one index in every block of TILE, plus the very first and last"""
    idx = [b * TILE + int(rng.integers(0, min(TILE, n - b * TILE))) for b in range(-(-n // TILE))]
    return np.unique(np.array(idx + [0, n - 1]))


def _segments_ok(name, got, ref, axis):
    """`got`/`ref` are sampled rows (axis=1: segments along columns) or sampled columns (axis=0: along rows): every
    TILE-long segment of every sample is one tile's share and must meet the local bound on its own."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    if axis == 0:
        got, ref = got.T, ref.T
    assert rel_fro(got, ref) <= FRO_TOL, (name, rel_fro(got, ref))
    n = ref.shape[1]
    pad = -(-n // TILE) * TILE - n
    e = np.pad((got - ref) ** 2, ((0, 0), (0, pad))).reshape(ref.shape[0], -1, TILE).sum(-1)
    r = np.pad(ref ** 2, ((0, 0), (0, pad))).reshape(ref.shape[0], -1, TILE).sum(-1)
    floor = (0.05 ** 2) * np.mean(ref ** 2) * TILE
    err = np.sqrt(e / np.maximum(r, floor))
    i = np.unravel_index(int(np.argmax(err)), err.shape)
    assert err[i] <= LOCAL_TOL, f"{name}: sample {i[0]}, tile segment {i[1]}: relative error {err[i]:.3e} > {LOCAL_TOL}"


@pytest.mark.parametrize("n", [8192, 16384])
def test_square_full_size_every_tile_sampled(pkg, lib, oracle, n):
    g = torch.Generator(device="cuda").manual_seed(n)
    lim = (6.0 / n) ** 0.5
    X = torch.randn((n, n), device="cuda", generator=g).bfloat16()
    W = ((torch.rand((n, n), device="cuda", generator=g) * 2 - 1) * lim).bfloat16()
    dY = torch.randn((n, n), device="cuda", generator=g).bfloat16()
    b = torch.rand((n,), device="cuda", generator=g) * 0.2 - 0.1
    Y, Z, work, dX, dW = (torch.empty((n, n), device="cuda", dtype=torch.bfloat16) for _ in range(5))
    db = torch.empty((1, n), device="cuda")
    og = pkg.ops_gemm
    og.forward_into(X, W, out=Y, bias=b, with_bias=True, act="gelu", save_z=True, z_out=Z)
    og.backward_into(X, W, dY, Z, act="gelu", with_bias=True, gA_out=dX, gB_out=dW, gBias_out=db, work_dZ=work)
    torch.cuda.synchronize()
    assert lib.ge2b_last_route() == 2 and lib.ge2b_device_status(1) == 0
    rng = np.random.default_rng(n)
    rows, cols = _one_per_block(n, rng), _one_per_block(n, rng)
    rt, ct = torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()
    b64 = _f64(b)
    Xh, Wh = _f64(X), _f64(W)                         # one device-to-host conversion each (2 GiB at n = 16384)
    # forward: sampled rows (all column tiles of every row block) and sampled columns (all row tiles)
    Zr = Xh[rows] @ Wh + b64
    _segments_ok("Z rows", _f64(Z[rt]), Zr, 1)
    _segments_ok("Y rows", _f64(Y[rt]), oracle.act_f64("gelu", Zr), 1)
    Zc = Xh @ Wh[:, cols] + b64[cols]
    _segments_ok("Z cols", _f64(Z[:, ct]), Zc, 0)
    _segments_ok("Y cols", _f64(Y[:, ct]), oracle.act_f64("gelu", Zc), 0)
    # the prologue: gZ = dY * gelu'(Z) (device Z), stored bf16, and db from the unrounded products
    gZr = _f64(dY[rt]) * oracle.act_deriv_f64("gelu", _f64(Z[rt]))
    _segments_ok("gZ rows", _f64(work[rt]), gZr, 1)
    gZc = _f64(dY[:, ct]) * oracle.act_deriv_f64("gelu", _f64(Z[:, ct]))
    assert rel_fro(_f64(db)[0, cols], gZc.sum(0)) <= 1e-3
    # backward GEMMs read the rounded gZ
    gZh = _f64(work)
    _segments_ok("dX rows", _f64(dX[rt]), gZh[rows] @ Wh.T, 1)
    _segments_ok("dX cols", _f64(dX[:, ct]), gZh @ Wh[cols].T, 0)
    _segments_ok("dW rows", _f64(dW[rt]), Xh[:, rows].T @ gZh, 1)
    _segments_ok("dW cols", _f64(dW[:, ct]), Xh.T @ gZh[:, cols], 0)


def test_attention_gemms_full_size(pkg, lib):
    """config 4: S = (Q.K^T)/sqrt(128) and O = P.V for B = 8, H = 16, L = 2048, d = 128 in bf16, one launch each."""
    Bn, H, L, d = 8, 16, 2048, 128
    g = torch.Generator(device="cuda").manual_seed(4)
    Q, Kt, V = (torch.randn((Bn, H, L, d), device="cuda", generator=g).bfloat16() for _ in range(3))
    S = torch.empty((Bn, H, L, L), device="cuda", dtype=torch.bfloat16)
    O = torch.empty((Bn, H, L, d), device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / d ** 0.5
    pkg.ops_gemm.forward_batched(Q, Kt, out=S, trans_b=True, alpha=scale)
    P = torch.softmax(torch.randn((Bn, H, L, L), device="cuda", generator=g), dim=-1).bfloat16()
    pkg.ops_gemm.forward_batched(P, V, out=O)
    torch.cuda.synchronize()
    assert lib.ge2b_device_status(1) == 0
    for (bi, hi) in ((0, 0), (2, 5), (4, 15), (7, 0), (7, 15)):
        check_close(f"S[{bi},{hi}]", _f64(S[bi, hi]), scale * (_f64(Q[bi, hi]) @ _f64(Kt[bi, hi]).T))
        check_close(f"O[{bi},{hi}]", _f64(O[bi, hi]), _f64(P[bi, hi]) @ _f64(V[bi, hi]))
    # every slice was written: no element of S / O keeps the fill value of a fresh poison pass
    S2 = torch.full_like(S, float("nan"))
    pkg.ops_gemm.forward_batched(Q, Kt, out=S2, trans_b=True, alpha=scale)
    torch.cuda.synchronize()
    assert torch.equal(S2, S)


@pytest.mark.parametrize("driver", ["plan", "trainer"])
def test_mlp_step_full_size(pkg, lib, oracle, driver):
    """config 3: batch 8192, 1024 -> 4096 -> 4096 -> 1024, ReLU / GELU / none, softmax-CE (mean), SGD lr = 1e-3, one
    captured step through the C++ plan (ge2b_mlp_plan_*) and through the torch-tensor trainer."""
    dims, acts, B, lr = [1024, 4096, 4096, 1024], ["relu", "gelu", "none"], 8192, 1e-3
    rng = np.random.default_rng(3)
    X = oracle.bf16_round(rng.standard_normal((B, dims[0]), dtype=np.float32))
    y = rng.integers(0, dims[-1], B).astype(np.int32)
    if driver == "plan":
        plan = pkg.MlpPlan(dims, acts, B, lr=lr, seed=0)
        W0 = [plan.params(i)[0].numpy().astype(np.float64) for i in range(3)]
        b0 = [plan.params(i)[1].numpy().astype(np.float64) for i in range(3)]
        plan.compile(capture=True)
        loss = plan.step_host(torch.from_numpy(X).bfloat16().pin_memory(), torch.from_numpy(y).pin_memory())
        gWs = [plan.grads(i)[0].double().numpy() for i in range(3)]
        gBs = [plan.grads(i)[1].double().numpy() for i in range(3)]
        W32 = [plan.params(i)[0].double().numpy() for i in range(3)]
        low_ok = all(torch.equal(plan.params(i)[2], plan.params(i)[0].bfloat16()) for i in range(3))
        plan.close()
    else:
        tr = pkg.DenseStackTrainer(dims, acts, B, lr=lr, seed=0)
        W0 = [w.cpu().numpy().astype(np.float64) for w in tr.W32]
        b0 = [x.cpu().numpy().astype(np.float64) for x in tr.b]
        tr.compile(capture=True)
        loss = tr.one_step(torch.from_numpy(X).cuda().bfloat16(), torch.from_numpy(y).cuda())
        torch.cuda.synchronize()
        gWs = [t.double().cpu().numpy() for t in tr.gW]
        gBs = [t.double().cpu().numpy().ravel() for t in tr.gB]
        W32 = [t.double().cpu().numpy() for t in tr.W32]
        low_ok = all(torch.equal(tr.W[i], tr.W32[i].bfloat16()) for i in range(3))
    assert lib.ge2b_device_status(1) == 0
    ref_loss, W1, b1, grads = oracle.mlp_step_f64(W0, b0, X, y, acts, lr, lowp=oracle.bf16_round)
    assert abs(loss - ref_loss) <= 5e-3 * abs(ref_loss), (loss, ref_loss)
    for i in range(3):
        rows = _one_per_block(dims[i], rng)
        # gradients as the step left them (bf16 dW, fp32 db): intermediate activations and gradients are rounded to
        # bf16 between layers on the device and not in the float64 reference, hence the contract's 2e-2 here
        assert rel_fro(gWs[i][rows], grads[i][0][rows]) <= FRO_TOL, i
        assert rel_fro(gBs[i], grads[i][1]) <= FRO_TOL, i
        # the update itself: W1 - W0 = -lr * dW in fp32 on the rounded dW
        assert rel_fro(W32[i][rows] - W0[i][rows], W1[i][rows] - W0[i][rows]) <= 2.5e-2, i
    assert low_ok
