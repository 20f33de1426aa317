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
