"""The gradient exchange across GPUs (needs at least two; skipped on a single-GPU box).

Child processes, one per GPU, NCCL process group.  `GradBucket.all_reduce` (this library's multimem kernel when the
group has a multicast mapping, the collective library otherwise) must give the sum of the ranks' gradients: exactly for
values whose sums are representable, within bf16 rounding for a real dW; the same launch replayed from a CUDA graph
must keep working (the signal pads return to zero after every call); and an all-reduced dW / db of the sharded dense
backward must equal the full-batch gradient.
"""
import os
import sys
from pathlib import Path

import pytest

torch = pytest.importorskip("torch")
ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, force_nccl, out):
    import importlib
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pkg = importlib.import_module("ai_framework-dev_b200")
    lib = pkg.load_library()
    dev = torch.device("cuda", rank)
    K, N = 1024, 1536
    bucket = pkg.data_parallel.GradBucket([((K, N), torch.bfloat16), ((1, N), torch.float32)], dist.group.WORLD, dev,
                                          force_nccl=force_nccl)
    dW, db = bucket.views
    # 1. exact sums: small integers, different on every rank
    g = torch.Generator(device="cpu").manual_seed(5)
    base_w = torch.randint(-8, 9, (K, N), generator=g).float()
    base_b = torch.randint(-100, 101, (1, N), generator=g).float()
    for rep in range(3):                                   # repeated calls reuse the signal pads
        dW.copy_((base_w * (rank + 1 + rep)).bfloat16())
        db.copy_(base_b * (rank + 1 + rep))
        torch.cuda.synchronize()
        dist.barrier()
        bucket.all_reduce()
        torch.cuda.synchronize()
        f = sum(r + 1 + rep for r in range(world))
        assert torch.equal(dW.float().cpu(), (base_w * f).bfloat16().float()), ("dW", rank, rep)
        assert torch.equal(db.cpu(), base_b * f), ("db", rank, rep)
    # 2. the same exchange captured into a CUDA graph and replayed
    st = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    dist.barrier()
    with torch.cuda.graph(graph, stream=st, capture_error_mode="thread_local"):
        bucket.all_reduce()
    for rep in range(3):
        dW.copy_((base_w * (rank + 2)).bfloat16())
        db.copy_(base_b * (rank + 2))
        torch.cuda.synchronize()
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        f = sum(r + 2 for r in range(world))
        assert torch.equal(dW.float().cpu(), (base_w * f).bfloat16().float()), ("graph dW", rank, rep)
        assert torch.equal(db.cpu(), base_b * f), ("graph db", rank, rep)
    # 3. sharded dense backward: rows of the batch split over the ranks, dW / db combined
    M = 512 * world
    g.manual_seed(9)
    X = torch.randn((M, K), generator=g).bfloat16()
    W = (torch.randn((K, N), generator=g) / 32).bfloat16()
    dY = torch.randn((M, N), generator=g).bfloat16()
    Z = torch.randn((M, N), generator=g).bfloat16()
    lo, hi = pkg.train.shard_rows(M, world, rank)
    Xs, dYs, Zs, Wd = X[lo:hi].to(dev), dY[lo:hi].to(dev), Z[lo:hi].to(dev), W.to(dev)
    dX = torch.empty_like(Xs)
    work = torch.empty_like(dYs)
    pkg.ops_gemm.backward_into(Xs, Wd, dYs, Zs, act="gelu", with_bias=True, gA_out=dX, gB_out=dW, gBias_out=db,
                               work_dZ=work)
    bucket.all_reduce()
    torch.cuda.synchronize()
    gz = dY.double() * torch.from_numpy(
        importlib.import_module("oracle.dense_oracle").act_deriv_f64("gelu", Z.double().numpy()))
    want_w, want_b = X.double().T @ gz, gz.sum(0, keepdim=True)
    err_w = float((dW.double().cpu() - want_w).norm() / want_w.norm())
    err_b = float((db.double().cpu() - want_b).norm() / want_b.norm())
    assert err_w <= 2e-2 and err_b <= 2e-2, (err_w, err_b)
    assert lib.ge2b_device_status(1) == 0
    if rank == 0:
        Path(out).write_text(f"{bucket.impl}|{bucket.why}")
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)        # the communicator may live in an instantiated graph: leave without tearing it down


@pytest.mark.parametrize("force_nccl", [False, True])
def test_gradient_bucket_all_reduce(tmp_path, force_nccl):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    world = min(4, torch.cuda.device_count())
    port = 29700 + os.getpid() % 200 + (50 if force_nccl else 0)
    out = tmp_path / "impl.txt"
    mp.spawn(_worker, args=(world, port, force_nccl, str(out)), nprocs=world, join=True)
    impl = out.read_text()
    print("all-reduce implementation:", impl)
    assert impl.startswith("nccl") if force_nccl else True


def _mlp_worker(rank, world, port, exchange, out):
    import importlib
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pkg = importlib.import_module("ai_framework-dev_b200")
    oracle = importlib.import_module("oracle.dense_oracle")
    lib = pkg.load_library()
    dims, acts, B, lr = [256, 512, 384, 128], ["relu", "gelu", "none"], 512, 0.05
    rows = B // world
    plan = pkg.MlpPlan(dims, acts, rows, lr=lr, seed=5, device=torch.device("cuda", rank), group=dist.group.WORLD,
                       global_batch=B, exchange=exchange, comm_blocks=8)
    W = [plan.params(i)[0].numpy().astype(np.float64) for i in range(3)]
    b = [plan.params(i)[1].numpy().astype(np.float64) for i in range(3)]
    plan.compile(capture=True)
    rng = np.random.default_rng(1)                         # every rank draws the same global batch
    for step in range(3):
        X = oracle.bf16_round(rng.standard_normal((B, dims[0]), dtype=np.float32))
        y = rng.integers(0, dims[-1], B).astype(np.int32)
        lo, hi = pkg.train.shard_rows(B, world, rank)
        plan.step_host(torch.from_numpy(X[lo:hi]).bfloat16().pin_memory(), torch.from_numpy(y[lo:hi]).pin_memory())
        loss = plan.global_loss()
        ref_loss, W, b, _ = oracle.mlp_step_f64(W, b, X, y, acts, lr, lowp=oracle.bf16_round)   # the FULL batch
        assert abs(loss - ref_loss) <= 2e-2 * abs(ref_loss), (rank, step, loss, ref_loss)
    got = [plan.params(i)[0] for i in range(3)]
    for i in range(3):
        # every replica holds the same parameters, and they follow the full-batch reference
        t = got[i].cuda()
        ref = t.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(t, ref), ("replicas diverged", i)
    assert lib.ge2b_device_status(1) == 0
    if rank == 0:
        Path(out).write_text(plan.exchange)
    plan.close()
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


@pytest.mark.parametrize("exchange", ["auto", "nccl"])
def test_mlp_plan_data_parallel(tmp_path, exchange):
    """The C++ step driver on two replicas: each gets half of the rows, every layer's dW / db are summed over the
    replicas inside the captured step, and the result follows the float64 reference of the FULL batch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    port = 29900 + os.getpid() % 90 + (5 if exchange == "nccl" else 0)
    out = tmp_path / "x.txt"
    mp.spawn(_mlp_worker, args=(2, port, exchange, str(out)), nprocs=2, join=True)
    print("exchange:", out.read_text())
    if exchange == "nccl":
        assert out.read_text() == "nccl"
