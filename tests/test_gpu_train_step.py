"""Softmax cross-entropy, SGD and the captured Dense-stack training step against the float64 oracle."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("C", [10, 1024, 1500, 3000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_ce_fused(pkg, lib, oracle, C, dtype):
    rng = np.random.default_rng(C)
    M = 257
    x = (rng.standard_normal((M, C)) * 3).astype(np.float32)
    if dtype == torch.bfloat16:
        x = oracle.bf16_round(x)
    lab = rng.integers(0, C, M).astype(np.int32)
    lab[5] = -1                                           # ignored row
    tx, tl = torch.from_numpy(x).cuda().to(dtype), torch.from_numpy(lab).cuda()
    d = torch.empty_like(tx)
    for red in ("mean", "sum", "none"):
        loss = torch.full((M if red == "none" else 1,), 7.0, device="cuda")
        pkg.softmax_ce_fused(tx, tl, dlogits=d, loss=loss, reduction=red, ignore_index=-1)
        torch.cuda.synchronize()
        rows, dref = oracle.softmax_ce_f64(x, lab, grad_scale=(1.0 / M if red == "mean" else 1.0))
        want = {"mean": rows.sum() / M, "sum": rows.sum(), "none": rows}[red]
        np.testing.assert_allclose(loss.cpu().numpy().squeeze(), want, rtol=2e-5, atol=2e-5)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert oracle.rel_fro(d.float().cpu().numpy(), dref) <= tol
        assert torch.all(d[5] == 0)


def test_softmax_ce_data_parallel_scaling(pkg, lib, oracle):
    """A shard of a global batch: loss and gradient are scaled by the global row count."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 100)).astype(np.float32)
    lab = rng.integers(0, 100, 64).astype(np.int32)
    tx, tl = torch.from_numpy(x).cuda(), torch.from_numpy(lab).cuda()
    d, loss = torch.empty_like(tx), torch.zeros(1, device="cuda")
    pkg.softmax_ce_fused(tx, tl, dlogits=d, loss=loss, reduction="mean", grad_scale=1 / 512, mean_denominator=512)
    rows, dref = oracle.softmax_ce_f64(x, lab, grad_scale=1 / 512)
    np.testing.assert_allclose(loss.item(), rows.sum() / 512, rtol=2e-5)
    assert oracle.rel_fro(d.cpu().numpy(), dref) <= 1e-5


@pytest.mark.parametrize("momentum,nesterov,wd,decay", [(0.0, False, 0.0, "decoupled"), (0.9, True, 0.0, "decoupled"),
                                                        (0.9, False, 0.01, "l2"), (0.0, False, 0.01, "decoupled")])
def test_sgd_update(pkg, lib, oracle, momentum, nesterov, wd, decay):
    rng = np.random.default_rng(1)
    n = 100003
    p0 = rng.standard_normal(n).astype(np.float32)
    g = oracle.bf16_round(rng.standard_normal(n).astype(np.float32))
    v0 = rng.standard_normal(n).astype(np.float32)
    p, v = torch.from_numpy(p0.copy()).cuda(), torch.from_numpy(v0.copy()).cuda()
    low = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pkg.sgd_update(p, torch.from_numpy(g).cuda().bfloat16(), lr=0.05, velocity=v if momentum else None,
                   momentum=momentum, nesterov=nesterov, weight_decay=wd, decay=decay, low=low)
    torch.cuda.synchronize()
    pref, vref = oracle.sgd_f64(p0, g, v0 if momentum else None, lr=0.05, momentum=momentum, nesterov=nesterov,
                                weight_decay=wd, decay=decay)
    np.testing.assert_allclose(p.cpu().numpy(), pref, rtol=1e-6, atol=1e-6)
    if momentum:
        np.testing.assert_allclose(v.cpu().numpy(), vref, rtol=1e-6, atol=1e-6)
    assert torch.equal(low, p.bfloat16())


@pytest.mark.parametrize("capture", [False, True])
def test_dense_stack_training_steps_match_float64(pkg, lib, oracle, capture):
    dims, acts, B, lr = [96, 256, 192, 64], ["relu", "gelu", "none"], 128, 0.05
    tr = pkg.DenseStackTrainer(dims, acts, B, lr=lr, seed=3)
    W = [w.cpu().numpy().astype(np.float64) for w in tr.W32]
    b = [x.cpu().numpy().astype(np.float64) for x in tr.b]
    tr.compile(capture=capture)
    # compile() warms the step up and must leave the parameters as they were initialised
    for w0, w in zip(W, tr.W32):
        assert np.array_equal(w0, w.cpu().numpy().astype(np.float64)), "compile() changed the weights"
    for b0, x in zip(b, tr.b):
        assert np.array_equal(b0, x.cpu().numpy().astype(np.float64)), "compile() changed the biases"
    W_start = [w.copy() for w in W]
    rng = np.random.default_rng(0)
    for step in range(3):
        X = oracle.bf16_round(rng.standard_normal((B, dims[0]), dtype=np.float32))
        y = rng.integers(0, dims[-1], B).astype(np.int32)
        loss = tr.one_step(torch.from_numpy(X).cuda().bfloat16(), torch.from_numpy(y).cuda())
        ref_loss, W, b, _ = oracle.mlp_step_f64(W, b, X, y, acts, lr, lowp=oracle.bf16_round)
        assert abs(loss - ref_loss) <= 2e-2 * abs(ref_loss), (step, loss, ref_loss)
    for i in range(3):
        got = tr.W32[i].cpu().numpy().astype(np.float64) - W_start[i]
        want = W[i] - W_start[i]
        assert oracle.rel_fro(got, want) <= 5e-2, i
        assert torch.equal(tr.W[i], tr.W32[i].bfloat16())
