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


# --------------------------------------------------------------------------- the reference's own ops as the oracle
def _ref_train():
    import ctypes as C
    from pathlib import Path
    so = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_train.so"
    if not so.exists():
        pytest.skip("oracle/_ref/libref_train.so was not built (needs the reference tree at build time)")
    r = C.CDLL(str(so))
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    r.ref_ce_fused.argtypes = [vp, vp, vp, vp, i, i, i, vp]
    r.ref_ce_forward.argtypes = [vp, vp, vp, i, i, i, i, f, vp]
    r.ref_ce_backward.argtypes = [vp, vp, vp, i, i, i, i, f, vp]
    r.ref_sgd.argtypes = [vp, vp, vp, C.c_longlong, f, f, f, i, f, vp]
    for fn in (r.ref_ce_fused, r.ref_ce_forward, r.ref_ce_backward, r.ref_sgd):
        fn.restype = i
    return r


@pytest.mark.parametrize("C", [10, 1024, 1500, 3000])
@pytest.mark.parametrize("red", ["none", "mean", "sum"])
def test_softmax_ce_against_reference_fused_op(pkg, lib, C, red):
    """SoftmaxCEFusedForwardBackwardCudaLaunch (cross_entropy/launcher.cu:238-306) compiled for sm_100a, on the same
    device buffers.  Its gradient is softmax - onehot WITHOUT the 1/M of a mean loss (kernels.cu:365-369), which is
    grad_scale = 1 here; its mean loss divides by every row (kernels.cu:356-358)."""
    ref = _ref_train()
    g = torch.Generator(device="cuda").manual_seed(C)
    M = 300
    x = torch.randn((M, C), device="cuda", generator=g) * 3
    lab = torch.randint(0, C, (M,), device="cuda", generator=g, dtype=torch.int32)
    code = {"none": 0, "mean": 1, "sum": 2}[red]
    n_loss = M if red == "none" else 1
    d_ref, l_ref = torch.empty_like(x), torch.full((n_loss,), 5.0, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert ref.ref_ce_fused(x.data_ptr(), lab.data_ptr(), d_ref.data_ptr(), l_ref.data_ptr(), M, C, code, s) == 0
    d, loss = torch.empty_like(x), torch.full((n_loss,), 7.0, device="cuda")
    pkg.softmax_ce_fused(x, lab, dlogits=d, loss=loss, reduction=red, grad_scale=1.0)
    torch.cuda.synchronize()
    assert float((d - d_ref).abs().max()) <= 1e-6
    # scalar losses are atomic sums of M terms in both libraries: order differs
    np.testing.assert_allclose(loss.cpu().numpy(), l_ref.cpu().numpy(), rtol=1e-6 if red == "none" else 2e-5, atol=1e-6)


@pytest.mark.parametrize("ls", [0.0, 0.1])
@pytest.mark.parametrize("red", ["none", "mean", "sum"])
def test_softmax_ce_against_reference_separate_ops(pkg, lib, red, ls):
    """CrossEntropyCudaLaunch / CrossEntropyCudaBackwardLaunch (from logits): ignore_index rows give zero loss and zero
    gradient but still count in the mean's denominator (launcher.cu:114-115), label smoothing as kernels.cu:96-101."""
    ref = _ref_train()
    g = torch.Generator(device="cuda").manual_seed(7)
    M, C, ign = 513, 777, 5
    x = torch.randn((M, C), device="cuda", generator=g) * 2
    lab = torch.randint(0, C, (M,), device="cuda", generator=g, dtype=torch.int32)
    lab[::9] = ign                                         # about 11 % ignored rows
    code = {"none": 0, "mean": 1, "sum": 2}[red]
    n_loss = M if red == "none" else 1
    d_ref, l_ref = torch.empty_like(x), torch.full((n_loss,), 5.0, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert ref.ref_ce_forward(x.data_ptr(), lab.data_ptr(), l_ref.data_ptr(), M, C, code, ign, ls, s) == 0
    assert ref.ref_ce_backward(x.data_ptr(), lab.data_ptr(), d_ref.data_ptr(), M, C, code, ign, ls, s) == 0
    d, loss = torch.empty_like(x), torch.full((n_loss,), 7.0, device="cuda")
    pkg.softmax_ce_fused(x, lab, dlogits=d, loss=loss, reduction=red, ignore_index=ign, label_smoothing=ls)
    torch.cuda.synchronize()
    assert float((d - d_ref).abs().max()) <= 1e-6
    assert torch.all(d[::9] == 0)
    np.testing.assert_allclose(loss.cpu().numpy(), l_ref.cpu().numpy(), rtol=2e-6 if red == "none" else 2e-5, atol=2e-6)


@pytest.mark.parametrize("momentum,dampening,nesterov,wd", [(0.0, 0.0, False, 0.0), (0.9, 0.0, True, 0.0),
                                                             (0.9, 0.1, False, 0.01), (0.0, 0.0, False, 0.01)])
def test_sgd_against_reference_op(pkg, lib, momentum, dampening, nesterov, wd):
    """SGDCudaUpdateLaunch (optimizer/kernels.cu:33-66): L2 decay added to the gradient, momentum / Nesterov."""
    ref = _ref_train()
    g = torch.Generator(device="cuda").manual_seed(2)
    n = 100003
    p0 = torch.randn(n, device="cuda", generator=g)
    grad = torch.randn(n, device="cuda", generator=g)
    v0 = torch.randn(n, device="cuda", generator=g)
    p_ref, v_ref = p0.clone(), v0.clone()
    s = torch.cuda.current_stream().cuda_stream
    assert ref.ref_sgd(p_ref.data_ptr(), grad.data_ptr(), v_ref.data_ptr() if momentum else None, n, 0.05, momentum,
                       dampening, int(nesterov), wd, s) == 0
    p, v = p0.clone(), v0.clone()
    pkg.sgd_update(p, grad, lr=0.05, velocity=v if momentum else None, momentum=momentum, dampening=dampening,
                   nesterov=nesterov, weight_decay=wd, decay="l2")
    torch.cuda.synchronize()
    # the same fp32 operations, possibly contracted differently into FMAs by the two compilations
    assert float(((p - p_ref).abs() / p_ref.abs().clamp_min(1.0)).max()) <= 1e-6
    if momentum:
        assert float(((v - v_ref).abs() / v_ref.abs().clamp_min(1.0)).max()) <= 1e-6


# --------------------------------------------------------------------------- the C++ step driver (ge2b_mlp_plan_*)
@pytest.mark.parametrize("capture", [False, True])
def test_mlp_plan_training_steps_match_float64(pkg, lib, oracle, capture):
    """The library-owned plan (buffers, warm-up, capture, replay in C++) through its C ABI, host batches in."""
    dims, acts, B, lr = [96, 256, 192, 64], ["relu", "gelu", "none"], 128, 0.05
    plan = pkg.MlpPlan(dims, acts, B, lr=lr, seed=3)
    W = [plan.params(i)[0].numpy().astype(np.float64) for i in range(3)]
    b = [plan.params(i)[1].numpy().astype(np.float64) for i in range(3)]
    plan.compile(capture=capture)
    for i in range(3):                                       # the warm-up left the parameters alone
        w1, b1, wl = plan.params(i)
        assert np.array_equal(w1.numpy().astype(np.float64), W[i]) and np.array_equal(b1.numpy().astype(np.float64), b[i])
        assert torch.equal(wl, w1.bfloat16())
    W_start = [w.copy() for w in W]
    rng = np.random.default_rng(0)
    for step in range(3):
        X = oracle.bf16_round(rng.standard_normal((B, dims[0]), dtype=np.float32))
        y = rng.integers(0, dims[-1], B).astype(np.int32)
        loss = plan.step_host(torch.from_numpy(X).bfloat16().pin_memory(), torch.from_numpy(y).pin_memory())
        ref_loss, W, b, _ = oracle.mlp_step_f64(W, b, X, y, acts, lr, lowp=oracle.bf16_round)
        assert abs(loss - ref_loss) <= 2e-2 * abs(ref_loss), (step, loss, ref_loss)
    for i in range(3):
        w1, b1, wl = plan.params(i)
        assert oracle.rel_fro(w1.numpy().astype(np.float64) - W_start[i], W[i] - W_start[i]) <= 5e-2, i
        assert torch.equal(wl, w1.bfloat16())
    assert abs(plan.global_loss() - loss) <= 1e-6
    assert lib.ge2b_device_status(1) == 0
    plan.close()


def test_mlp_plan_agrees_with_the_python_trainer(pkg, lib):
    """Same seed, same batches: the C++ plan and the torch-tensor trainer launch the same kernels in the same order."""
    dims, acts, B = [128, 320, 64], ["gelu", "none"], 256
    tr = pkg.DenseStackTrainer(dims, acts, B, lr=0.02, seed=11)
    plan = pkg.MlpPlan(dims, acts, B, lr=0.02, seed=11)
    tr.compile(capture=True)
    plan.compile(capture=True)
    g = torch.Generator().manual_seed(1)
    for _ in range(2):
        X = torch.randn((B, dims[0]), generator=g).bfloat16()
        y = torch.randint(0, dims[-1], (B,), generator=g, dtype=torch.int32)
        l1 = tr.one_step(X.cuda(), y.cuda())
        l2 = plan.step_host(X, y)
        assert abs(l1 - l2) <= 1e-5 * max(1.0, abs(l1))
    for i in range(2):
        w, bb, _ = plan.params(i)
        assert torch.allclose(w, tr.W32[i].cpu(), rtol=0, atol=1e-6) and torch.allclose(bb, tr.b[i].cpu(), rtol=0, atol=1e-6)
    plan.close()
