"""The data-parallel rule of the path on CPU ranks (gloo, world size 2): rows of the batch are sharded along M, the
loss gradient is scaled by 1/global_batch on every replica, and the SUM all-reduce of the replicas' dW and db equals
the full-batch gradient.  Device kernels are not involved: each rank evaluates its shard with the float64 oracle."""
import importlib
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = importlib.import_module("ai_framework-dev_b200")
    oracle = importlib.import_module("oracle.dense_oracle")
    rng = np.random.default_rng(0)                       # every rank draws the same global batch
    B, dims, acts = 37, [12, 20, 9], ["gelu", "none"]    # 37 rows: uneven shards
    X = rng.standard_normal((B, dims[0]))
    y = rng.integers(0, dims[-1], B)
    W = [rng.standard_normal((dims[i], dims[i + 1])) * 0.3 for i in range(2)]
    b = [rng.standard_normal(dims[i + 1]) * 0.1 for i in range(2)]
    lo, hi = pkg.train.shard_rows(B, world, rank)
    _, _, _, grads = oracle.mlp_step_f64(W, b, X[lo:hi], y[lo:hi], acts, lr=0.1, global_batch=B)
    flat = torch.from_numpy(np.concatenate([np.concatenate([gw.ravel(), gb.ravel()]) for gw, gb in grads]))
    dist.all_reduce(flat)                                # SUM, as the trainer does
    np.save(Path(out_dir) / f"rank{rank}.npy", flat.numpy())
    if rank == 0:
        _, _, _, full = oracle.mlp_step_f64(W, b, X, y, acts, lr=0.1)
        np.save(Path(out_dir) / "full.npy", np.concatenate([np.concatenate([gw.ravel(), gb.ravel()]) for gw, gb in full]))
    dist.destroy_process_group()


def test_sharded_gradients_sum_to_full_batch(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    full = np.load(tmp_path / "full.npy")
    for r in range(2):
        np.testing.assert_allclose(np.load(tmp_path / f"rank{r}.npy"), full, rtol=1e-10, atol=1e-12)


def test_shard_rows_cover_the_batch(pkg):
    for B, world in ((8192, 8), (37, 2), (5, 4), (3, 8)):
        edges = [pkg.train.shard_rows(B, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == B
        assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
        assert max(e - s for s, e in edges) - min(e - s for s, e in edges) <= 1
    with pytest.raises(ValueError):
        pkg.train.shard_rows(8, 2, 2)
    assert pkg.train.loss_grad_scale(8192) == 1.0 / 8192


def test_reference_arm_under_torchrun_prints_one_line():
    """Under torchrun only rank 0 runs the CPU arm; the other rank exits 0 without work."""
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(29900 + os.getpid() % 90),
                        str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-800:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    import json
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["e2e"]["h2d_bytes_per_step"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["value"] > 0


def _bucket_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = importlib.import_module("ai_framework-dev_b200")
    # the gradient bucket on host ranks: same layout and exchange protocol, collective library instead of the NVLink kernel
    b = pkg.data_parallel.GradBucket([((5, 7), torch.float32), ((3, 7), torch.float32), ((1, 7), torch.float32)],
                                     dist.group.WORLD, "cpu")
    assert b.impl == "nccl" and [o % 256 for o in b.offsets] == [0, 0, 0] and b.offsets[1] >= 5 * 7 * 4
    for i, v in enumerate(b.views):
        v.fill_(float((rank + 1) * (i + 1)))
    b.all_reduce(1, 2)                                    # a sub-range: the first region must stay untouched
    ok = bool((b.views[0] == rank + 1).all() and (b.views[1] == 2 * 3).all() and (b.views[2] == 3 * 3).all())
    b.all_reduce()
    ok = ok and bool((b.views[0] == 3).all() and (b.views[1] == 12).all())
    (Path(out_dir) / f"bucket{rank}.txt").write_text("ok" if ok else "bad")
    dist.destroy_process_group()


def test_gradient_bucket_layout_and_exchange_on_host_ranks(tmp_path):
    import torch.multiprocessing as mp
    port = 29650 + os.getpid() % 300
    mp.spawn(_bucket_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all((tmp_path / f"bucket{r}.txt").read_text() == "ok" for r in range(2))


def test_gradient_bucket_segments_merge_runs_of_one_dtype(pkg):
    import torch
    gb = pkg.data_parallel.GradBucket.__new__(pkg.data_parallel.GradBucket)
    gb.regions = [((4, 64), torch.bfloat16), ((4, 64), torch.bfloat16), ((1, 64), torch.float32)]
    gb.offsets, gb.data_bytes = [0, 512, 1024], 1280
    assert gb._segments(0, 2) == [(0, 1024, pkg._lib.DT_BF16), (1024, 256, pkg._lib.DT_F32)]
    assert gb._segments(1, 1) == [(512, 512, pkg._lib.DT_BF16)]
    gb.regions.append(((4, 64), torch.bfloat16))
    gb.offsets.append(1280)
    gb.data_bytes = 1792
    with pytest.raises(ValueError):
        gb._segments(0, 3)                                # bf16, fp32, bf16: three runs


def test_mlp_plan_configuration_is_validated_without_a_gpu(pkg, lib):
    import ctypes as C
    L = pkg._lib
    cfg = L.MlpConfig()
    plan = C.c_void_p()
    assert lib.ge2b_mlp_plan_create(C.byref(plan), C.byref(cfg)) == -1           # no layers
    cfg.n_layers, cfg.batch, cfg.dtype, cfg.lr, cfg.world = 2, 8, L.DT_BF16, 0.1, 1
    cfg.dims[0], cfg.dims[1], cfg.dims[2] = 16, 32, 8
    assert lib.ge2b_mlp_plan_grad_bytes(C.byref(cfg)) == (16 * 32 * 2 + 256 + 32 * 8 * 2 + 256) + lib.ge2b_allreduce_nvls_pad_bytes()
    cfg.world, cfg.exchange = 2, 0
    assert lib.ge2b_mlp_plan_create(C.byref(plan), C.byref(cfg)) == -1           # replicas without an exchange
    cfg.exchange = 1
    assert lib.ge2b_mlp_plan_create(C.byref(plan), C.byref(cfg)) == -1           # ... or without symmetric memory
    cfg.world, cfg.lr = 1, 0.0
    assert lib.ge2b_mlp_plan_create(C.byref(plan), C.byref(cfg)) == -1           # learning rate must be positive
    a = L.AllreduceNvls()
    assert lib.ge2b_allreduce_nvls(C.byref(a), None) == -1                       # no buffer, no ranks
