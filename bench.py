#!/usr/bin/env python
"""Benchmark of the dense-layer hot path on B200.

Workload: dense layer forward + backward, M = N = K = 4096, bf16 tensors with fp32
accumulation, fp32 bias, tanh-GELU epilogue; outputs Y, Z (pre-activation), dX, dW, db.  One step = one forward
and one backward over one batch.  Work counted per step: 6*M*N*K flop (2 forward + 4 backward); epilogue,
bias and reduction arithmetic is not counted.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 (under torch.distributed.run): every rank runs its own M = 4096 rows against the same W (batch sharded
along M, weak scaling); dW and db are combined by NCCL all-reduce (sum), issued per row block of dW as soon as
that block is written so that the exchange overlaps the remaining dW blocks and the dX GEMM.  `value` counts the flop of all ranks over the slowest rank's device time.

Prints ONE JSON line on rank 0.  `--impl reference` times the CPU restatement of the reference's path (the
oracle) on this host's cores on a bounded row-slab of the same workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N = K = 4096
ACT = "gelu"
FLOP_PER_STEP = 6.0 * M * N * K
FLOP_FWD_LAUNCH = 2.0 * M * N * K
METRIC = "dense_gemm_bias_gelu_fwd_bwd_throughput"
UNIT = "TFLOP/s"
CONFIG = {
    "workload": "dense layer fwd+bwd, M=N=K=4096, bf16 in / fp32 accumulate, fp32 bias, GELU(tanh), outputs Y,Z,dX,dW,db",
    "l2": "no flush: a step touches 8 tensors x 32 MiB = 256 MiB, twice the 126 MB L2",
    "cpu_arm": "the CPU legs time a row slab of this workload and extrapolate (the loop nest is linear in rows)",
}
FALLBACK_PEAK_TFLOPS = 1590.0
FALLBACK_SUSTAINED_TFLOPS = 1400.0
NOMINAL_PEAK_TFLOPS = 2250.0
TRAFFIC_PROFILE = "profiles/gemm_tc_fwd_4096_bf16_pair.md"
MIN_WINDOW_S = 1.0       # the timed region replays the step until it is at least this long


def measured_peak(key="bf16_tflops"):
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())[key]), "measured"
        except Exception:
            pass
    return (FALLBACK_PEAK_TFLOPS if key == "bf16_tflops" else FALLBACK_SUSTAINED_TFLOPS), "fallback"


def launch_traffic(key="dram_bytes_per_launch"):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload, as recorded in the tracked ncu
    summary (a line `<key> = <bytes>`: `dram_bytes_per_launch` for the forward launch, `dram_bytes_per_launch_dual` for
    the dX + dW launch); None when the summary has no such line."""
    try:
        for line in (ROOT / TRAFFIC_PROFILE).read_text().splitlines():
            if line.split("=")[0].strip() == key:
                return float(line.split("=")[1].split()[0])
    except Exception:
        pass
    return None


def fwd_launch_traffic():
    return launch_traffic("dram_bytes_per_launch")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=1.0)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "sm_mhz_min": min(self.samples) if self.samples else None,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------ CPU legs
def cpu_fwd_bwd(oracle, rows, X, W, b, dY):
    """One forward + backward of the oracle on a slab of `rows` rows; returns seconds."""
    t0 = time.perf_counter()
    Y, Z = oracle.forward_f32(X[:rows], W, b, act=ACT)
    oracle.backward_f32(X[:rows], W, dY[:rows], Z, act=ACT)
    return time.perf_counter() - t0


def cpu_inputs(oracle):
    X, W, b, dY = oracle.dense_inputs(512, K, N, seed=0)        # at most 512 rows are ever sampled
    return tuple(oracle.bf16_round(a) for a in (X, W)) + (b, oracle.bf16_round(dY))


def cpu_rows_for(oracle, data, seconds_per_step):
    t = cpu_fwd_bwd(oracle, 4, *data)
    rows = int(max(1, min(512, 4 * seconds_per_step / max(t, 1e-6))))
    return rows


def run_cpu_baseline(target_seconds=12.0):
    oracle = importlib.import_module("oracle.dense_oracle")
    data = cpu_inputs(oracle)
    rows = cpu_rows_for(oracle, data, target_seconds)
    t = cpu_fwd_bwd(oracle, rows, *data)
    return {"value": 6.0 * rows * N * K / t / 1e12, "unit": UNIT, "cores": oracle.n_threads(), "kind": "port",
            "sample": f"rows 0..{rows - 1} of the M=4096 batch (all of N and K), forward + backward once, {t:.1f} s; "
                      "fp32 fmaf chains of oracle/dense_oracle.c over bf16-rounded inputs, rows split over host threads"}


def run_cpu_tuned():
    """The same forward + backward on all host cores through a tuned library (torch CPU fp32 matmul on the bf16-rounded
    inputs: oneDNN / MKL SGEMM), beside the loop-nest port: what a CPU user of the layer would really get."""
    import torch
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    X = torch.randn((M, K), generator=g).bfloat16().float()
    W = ((torch.rand((K, N), generator=g) * 2 - 1) * (6.0 / K) ** 0.5).bfloat16().float()
    b = torch.rand((N,), generator=g) * 0.2 - 0.1
    dY = torch.randn((M, N), generator=g).bfloat16().float()
    c0, c1 = 0.7978845608, 0.044715

    def fwd_bwd():
        Z = torch.addmm(b, X, W)
        th = torch.tanh(c0 * (Z + c1 * Z * Z * Z))
        Y = 0.5 * Z * (1 + th)
        gZ = dY * (0.5 * (1 + th) + 0.5 * Z * (1 - th * th) * c0 * (1 + 3 * c1 * Z * Z))
        return Y, gZ @ W.t(), X.t() @ gZ, gZ.sum(0)

    fwd_bwd()
    best = min(_timed(fwd_bwd) for _ in range(3))
    return {"value": FLOP_PER_STEP / best / 1e12, "unit": UNIT, "cores": cores,
            "kind": "tuned library (torch CPU fp32 matmul + vectorised epilogue; not the reference's code)",
            "sample": f"the whole M=N=K=4096 forward + backward, best of 3, {best:.2f} s"}


def _timed(fn):
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle = importlib.import_module("oracle.dense_oracle")
    data = cpu_inputs(oracle)
    budget = 150.0 / max(1, args.steps + args.warmup)
    rows = cpu_rows_for(oracle, data, min(budget, 10.0))
    for _ in range(args.warmup):
        cpu_fwd_bwd(oracle, rows, *data)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_fwd_bwd(oracle, rows, *data)
    dt = time.perf_counter() - t0
    value = 6.0 * rows * N * K * args.steps / dt / 1e12
    sample = (f"each step = forward + backward of rows 0..{rows - 1} of the M=4096 batch (all of N and K) through "
              "oracle/dense_oracle.c, the CPU restatement of the reference path (the reference has no CPU GEMM of its "
              "own), rows split over all host threads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": CONFIG,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.n_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the dense-layer path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = importlib.import_module("ai_framework-dev_b200")
    lib = pkg.load_library()
    og = pkg.ops_gemm
    dev = torch.device("cuda", local)

    # seeded synthetic inputs: X, dY ~ N(0,1); W ~ U(+-sqrt(6/K)); b ~ U(-0.1, 0.1); each rank its own rows
    gen = torch.Generator(device="cpu").manual_seed(0)
    lim = (6.0 / K) ** 0.5
    W_h = ((torch.rand((K, N), generator=gen) * 2 - 1) * lim).bfloat16().pin_memory()
    b_h = (torch.rand((N,), generator=gen) * 0.2 - 0.1).pin_memory()
    gen.manual_seed(1 + rank)
    X_h = torch.randn((M, K), generator=gen).bfloat16().pin_memory()
    dY_h = torch.randn((M, N), generator=gen).bfloat16().pin_memory()
    X, W, b, dY = X_h.to(dev), W_h.to(dev), b_h.to(dev), dY_h.to(dev)
    Y = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
    Z = torch.empty_like(Y)
    work = torch.empty_like(Y)
    dX = torch.empty((M, K), device=dev, dtype=torch.bfloat16)
    sm_total = lib.ge2b_sm_count()
    comm_sms = int(os.environ.get("GE2B_BENCH_COMM_SMS", "16"))   # SMs of the exchange kernel; GEMMs beside it leave them free
    # Row blocks of dW whose exchange starts as each finishes (0: the backward runs as on one GPU, dX and dW in one
    # launch, and the exchange follows it).
    dw_chunks = max(0, int(os.environ.get("GE2B_BENCH_DW_CHUNKS", "1" if world == 1 else "2")))
    rows_per_chunk = K // max(1, dw_chunks)
    n_reg = max(1, dw_chunks)
    chunk_rows = [(c * rows_per_chunk, K if c == n_reg - 1 else (c + 1) * rows_per_chunk) for c in range(n_reg)]
    # dW (in row blocks) and db share ONE gradient bucket: symmetric memory mapped into a multicast object, summed over
    # the ranks by this library's NVLink kernel (multimem.ld_reduce / multimem.st), one launch per exchange; where the
    # process group has no such mapping the bucket uses the collective library instead (reported in the JSON line)
    bucket = None
    if world > 1:
        bucket = pkg.data_parallel.GradBucket([((r1 - r0, N), torch.bfloat16) for r0, r1 in chunk_rows] +
                                              [((1, N), torch.float32)], dist.group.WORLD, dev, blocks=comm_sms,
                                              force_nccl=os.environ.get("GE2B_BENCH_EXCHANGE", "") == "nccl")
        flat = bucket.buffer[:K * N * 2].view(torch.bfloat16).view(K, N)     # the row blocks are contiguous: one dW
        assert flat.data_ptr() == bucket.views[0].data_ptr() and (K * N * 2) % 256 == 0
        dW, db = flat, bucket.views[-1]
    else:
        dW = torch.empty((K, N), device=dev, dtype=torch.bfloat16)
        db = torch.empty((1, N), device=dev, dtype=torch.float32)
    comm = torch.cuda.Stream(device=dev) if world > 1 else None
    fwd_events = []

    def step(timed):
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        og.forward_into(X, W, out=Y, bias=b, with_bias=True, act=ACT, save_z=True, z_out=Z)
        if timed:
            e1.record()
            fwd_events.append((e0, e1))
        cur = torch.cuda.current_stream()
        if world == 1 or dw_chunks == 0:
            # the whole backward in one call: gZ = dY * gelu'(Z) with db, then dX and dW (one launch for both: their
            # tiles form one list, so only the combined list's last wave is partly filled)
            og.backward_into(X, W, dY, Z, act=ACT, with_bias=True, gA_out=dX, gB_out=dW, gBias_out=db, work_dZ=work)
            if world > 1:
                bucket.all_reduce()                     # dW and db in one exchange
            return
        # gZ = dY * gelu'(Z) and db in one pass; gZ stays in `work` for the two GEMMs
        og.backward_into(X, W, dY, Z, act=ACT, with_bias=True, gBias_out=db, work_dZ=work)
        # dW = X^T . gZ first, in row blocks; each block's exchange starts on the side stream as soon as it is written
        # and runs under the remaining dW blocks and the dX GEMM, which leave the exchange kernel its SMs
        for c, (r0, r1) in enumerate(chunk_rows):
            if c > 0 and comm_sms > 0:
                lib.ge2b_set_sm_limit(sm_total - comm_sms)
            og.forward_into(X[:, r0:r1], work, out=dW[r0:r1], trans_a=True)
            comm.wait_stream(cur)
            last = c == len(chunk_rows) - 1
            bucket.all_reduce(c, c + 1 if last else c, stream=comm)      # the last exchange takes db along
        if comm_sms > 0:
            lib.ge2b_set_sm_limit(sm_total - comm_sms)
        og.backward_into(X, W, dY, Z, act=ACT, gA_out=dX, work_dZ=work, reuse_dZ=True)
        lib.ge2b_set_sm_limit(0)
        cur.wait_stream(comm)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile == "conv":
        # conv2d forward + backward of one ResNet-like layer (bf16, N=32, 64 -> 64 channels, 56 x 56, 3 x 3), twice
        cv = pkg.ops_conv2d
        cX = torch.randn(32, 64, 56, 56, device=dev).bfloat16()
        cW = (torch.randn(64, 64, 3, 3, device=dev) / 24).bfloat16()
        cb = torch.randn(64, device=dev)
        cY = torch.empty(32, 64, 56, 56, device=dev, dtype=torch.bfloat16)
        cZ, cdY = torch.empty_like(cY), torch.randn(32, 64, 56, 56, device=dev).bfloat16()
        cgX, cgW, cgB = torch.empty_like(cX), torch.empty_like(cW), torch.empty(64, device=dev)
        for _ in range(2):
            cv.forward_into(cX, cW, out=cY, B=cb, with_bias=True, act="relu", save_z=True, Z_saved=cZ, padding=(1, 1))
            cv.backward_into(cX, cW, cdY, cZ, with_bias=True, act="relu", gX_out=cgX, gW_out=cgW, gB_out=cgB,
                             padding=(1, 1))
        barrier()
        print(json.dumps({"profile": "conv", "status": lib.ge2b_device_status(0)}), flush=True)
        return
    if args.profile == "qk":
        # the batched attention GEMM S = (Q.K^T)/sqrt(d) at L = 2048, d = 128 on 16 of the 128 (batch, head) slices
        # (134 MB of output: larger than L2, small enough for a profiler's save / restore), four launches
        Q, Kt = (torch.randn((2, 8, 2048, 128), device=dev).bfloat16() for _ in range(2))
        S = torch.empty((2, 8, 2048, 2048), device=dev, dtype=torch.bfloat16)
        for _ in range(4):
            og.forward_batched(Q, Kt, out=S, trans_b=True, alpha=1.0 / 128 ** 0.5)
        barrier()
        print(json.dumps({"profile": "qk", "status": lib.ge2b_device_status(0)}), flush=True)
        return
    if args.profile == "sdpa":
        # the fused attention forward at config 4's shape (B = 8, H = 16, L = 2048, d = 128, bf16), three launches
        Q, Kt, V = (torch.randn((8, 16, 2048, 128), device=dev).bfloat16() for _ in range(3))
        O = torch.empty_like(Q)
        for _ in range(3):
            pkg.ops_sdpa.forward(Q, Kt, V, out=O)
        barrier()
        print(json.dumps({"profile": "sdpa", "status": lib.ge2b_device_status(0)}), flush=True)
        return
    if args.profile:
        # a short, fixed launch sequence for a profiler capture: 2 warm-up steps, then 2 more
        for _ in range(4):
            if args.profile == "fwd":
                og.forward_into(X, W, out=Y, bias=b, with_bias=True, act=ACT, save_z=True, z_out=Z)
            else:
                step(False)
        barrier()
        print(json.dumps({"profile": args.profile, "status": lib.ge2b_device_status(0)}), flush=True)
        return

    for _ in range(max(3, args.warmup)):
        step(False)
    barrier()
    # One step = a fixed sequence of kernels (+ collectives): it is captured once into a CUDA graph and the timed
    # region replays it, so host launch cost (which exceeds the device time once NCCL calls are added) is off the path.
    nccl_graph = os.environ.get("GE2B_NCCL_GRAPH", "1") == "1"      # also capture multi-rank steps (with their NCCL calls)
    use_graph = os.environ.get("GE2B_BENCH_GRAPH", "1") == "1" and (world == 1 or nccl_graph)
    launches_per_step = None
    graph = None
    split_unavailable0 = lib.ge2b_split_unavailable_total()
    if use_graph:
        cap = torch.cuda.Stream(device=dev)
        cap.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cap):
            step(False)           # first use of this stream outside capture: per-stream scratch exists before capture
        cap.synchronize()
        l0 = lib.ge2b_launches_total()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=cap, capture_error_mode="thread_local"):
            step(False)
        launches_per_step = lib.ge2b_launches_total() - l0
        torch.cuda.current_stream().wait_stream(cap)
        for _ in range(3):
            graph.replay()
        barrier()

    def run_steps(n):
        for _ in range(n):
            if graph is not None:
                graph.replay()
            else:
                step(False)

    def timed_window(n, sampler):
        """n steps between two events; the ranks enter together: one untimed step and a barrier come right before the
        first event, and the clock sampler is already running."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with sampler:
            run_steps(1)
            barrier()
            a.record()
            run_steps(n)
            b.record()
            barrier()
        t = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # burst: exactly --steps steps.  sustained: the step replayed until the region is at least MIN_WINDOW_S long (the
    # count is agreed between the ranks from the burst window), so that the clock settles and is sampled many times.
    def graph_of(fn):
        g_ = torch.cuda.CUDAGraph()
        st = torch.cuda.Stream(device=dev)
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            fn()
        st.synchronize()
        with torch.cuda.graph(g_, stream=st, capture_error_mode="thread_local"):
            fn()
        torch.cuda.current_stream().wait_stream(st)
        return g_

    def replay_ms(g_, reps):
        for _ in range(3):
            g_.replay()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        f0.record()
        for _ in range(reps):
            g_.replay()
        f1.record()
        torch.cuda.synchronize()
        return f0.elapsed_time(f1) / reps

    clk_burst = ClockSampler(local)
    clk = ClockSampler(local, period_s=0.01)
    burst_ms = timed_window(args.steps, clk_burst)
    # per-launch duration of the forward kernel for the roofline, burst form: the forward launch alone captured into a
    # graph and replayed back to back (no host in the loop), CUDA events around a run of a few milliseconds, taken
    # while the GPU is still at its burst clock (before the long windows below pull it down to the power cap)
    fwd_graph = graph_of(lambda: og.forward_into(X, W, out=Y, bias=b, with_bias=True, act=ACT, save_z=True, z_out=Z))
    torch.cuda.synchronize()
    time.sleep(0.5)
    with ClockSampler(local, period_s=0.002) as clk_fwd_burst:
        fwd_ms = replay_ms(fwd_graph, max(10, min(args.steps, 50)))
    # the same for the launch that computes dX and dW together (the larger share of the step): gZ is taken as already
    # in `work` (reuse_dZ), so the graph holds that one launch
    og.backward_into(X, W, dY, Z, act=ACT, with_bias=True, gA_out=dX, gB_out=dW, gBias_out=db, work_dZ=work)
    l_b0 = lib.ge2b_launches_total()
    bwd_graph = graph_of(lambda: og.backward_into(X, W, dY, Z, act=ACT, gA_out=dX, gB_out=dW, work_dZ=work, reuse_dZ=True))
    bwd_gemm_launches = (lib.ge2b_launches_total() - l_b0) // 2          # graph_of runs the call twice
    torch.cuda.synchronize()
    time.sleep(0.3)
    with ClockSampler(local, period_s=0.002) as clk_bwd_burst:
        bwd_ms = replay_ms(bwd_graph, max(10, min(args.steps, 50)))
    replays = max(args.steps, int(MIN_WINDOW_S * 1e3 / max(burst_ms / args.steps, 1e-3)) + 1)
    launches0 = lib.ge2b_launches_total()
    total_ms = timed_window(replays, clk)
    launches = (launches_per_step * replays) if graph is not None else lib.ge2b_launches_total() - launches0

    # the same launch replayed for at least half a second (the clock the power cap settles at)
    with ClockSampler(local, period_s=0.01) as clk_fwd:
        fwd_sustained_ms = replay_ms(fwd_graph, int(500.0 / max(fwd_ms, 1e-3)) + 1)
    with ClockSampler(local, period_s=0.01) as clk_bwd:
        bwd_sustained_ms = replay_ms(bwd_graph, int(500.0 / max(bwd_ms, 1e-3)) + 1)
    for _ in range(min(args.steps, 30)):
        step(True)
    barrier()
    fwd_eager_ms = statistics.median(a.elapsed_time(c) for a, c in fwd_events)

    # the target shape of the path: M = N = K = 8192 (single GPU only; windows of at least 0.7 s each)
    target = None
    if world == 1 and not args.skip_target:
        n8 = 8192
        g8 = torch.Generator(device="cpu").manual_seed(8)
        X8 = torch.randn((n8, n8), generator=g8).bfloat16().to(dev)
        W8 = ((torch.rand((n8, n8), generator=g8) * 2 - 1) * (6.0 / n8) ** 0.5).bfloat16().to(dev)
        dY8 = torch.randn((n8, n8), generator=g8).bfloat16().to(dev)
        b8 = (torch.rand((n8,), generator=g8) * 0.2 - 0.1).to(dev)
        Y8, Z8, work8, dX8, dW8 = (torch.empty((n8, n8), device=dev, dtype=torch.bfloat16) for _ in range(5))
        db8 = torch.empty((1, n8), device=dev, dtype=torch.float32)
        f8 = lambda: og.forward_into(X8, W8, out=Y8, bias=b8, with_bias=True, act=ACT, save_z=True, z_out=Z8)  # noqa: E731
        r8 = lambda: og.backward_into(X8, W8, dY8, Z8, act=ACT, with_bias=True, gA_out=dX8, gB_out=dW8,  # noqa: E731
                                      gBias_out=db8, work_dZ=work8)
        flop8 = 2.0 * n8 ** 3
        target = {"workload": "M=N=K=8192 bf16, fp32 bias, GELU(tanh), outputs Y,Z / dX,dW,db; CUDA-graph replays, "
                              "each window at least 0.7 s"}
        peak_b, _ = measured_peak("bf16_tflops")
        peak_s, _ = measured_peak("bf16_tflops_sustained")
        for name, fn, flop in (("fwd", f8, flop8), ("bwd", r8, 2 * flop8), ("fwd_bwd", lambda: (f8(), r8()), 3 * flop8)):
            g_ = graph_of(fn)
            short = replay_ms(g_, 5)
            with ClockSampler(local, period_s=0.01) as ck:
                ms_ = replay_ms(g_, int(700.0 / max(short, 1e-3)) + 1)
            tf = flop / (ms_ * 1e-3) / 1e12
            cs = ck.summary()
            target[name] = {"tflops": tf, "ms": ms_, "burst_tflops": flop / (short * 1e-3) / 1e12,
                            "frac_of_nominal_2250": tf / NOMINAL_PEAK_TFLOPS, "frac_of_measured_burst": tf / peak_b,
                            "frac_of_measured_sustained": tf / peak_s, "sm_mhz": cs["sm_mhz"],
                            "ms_x_ghz": (ms_ * cs["sm_mhz"] / 1e3) if cs["sm_mhz"] else None, "reasons": cs["reasons"]}
            del g_
        target["peaks"] = {"nominal": NOMINAL_PEAK_TFLOPS, "measured_burst": peak_b, "measured_sustained": peak_s}
        del X8, W8, dY8, Y8, Z8, work8, dX8, dW8
        torch.cuda.empty_cache()

    # multi-GPU: the combined gradients are checked after the timed region.  One eager step; dW / db must equal the
    # fp32 sum of every rank's own dW / db (gathered) on sampled rows.
    allreduce_check = None
    if world > 1:
        allreduce_check = "ok"
        for form in ("step",):
            # this rank's own gradients (no exchange) ...
            og.backward_into(X, W, dY, Z, act=ACT, with_bias=True, gA_out=dX, gB_out=dW, gBias_out=db, work_dZ=work)
            rows_chk = torch.arange(0, K, 61, device=dev)
            own = torch.cat([dW[rows_chk].float().reshape(-1), db.reshape(-1)])
            gathered = [torch.empty_like(own) for _ in range(world)]
            dist.all_gather(gathered, own)
            want = torch.stack(gathered).sum(0)
            # ... and the step's combined ones
            step(False)
            barrier()
            got = torch.cat([dW[rows_chk].float().reshape(-1), db.reshape(-1)])
            err_t = ((got - want).norm() / want.norm()).reshape(1)
            dist.all_reduce(err_t, op=dist.ReduceOp.MAX)              # the worst rank decides
            err = float(err_t.item())
            if not err <= 1e-2:          # bf16 storage of the sum: 2^-9 relative per element
                allreduce_check = f"MISMATCH rel_fro={err:.3e}"
    value = world * FLOP_PER_STEP * replays / (total_ms * 1e-3) / 1e12
    burst_value = world * FLOP_PER_STEP * args.steps / (burst_ms * 1e-3) / 1e12
    assert lib.ge2b_device_status(0) == 0, "a bounded wait inside a kernel timed out"

    # ---- end to end through the host-buffer plan of the C ABI: pinned host inputs up, results down, every step
    import ctypes as C
    plan = C.c_void_p()
    L = pkg._lib
    rc = lib.ge2b_dense_plan_create(C.byref(plan), M, K, N, L.DT_BF16, L.ACT[ACT], 0.01, 1, L.MATH_TENSOR)
    assert rc == 0, rc
    # two sets of pinned result buffers: two steps are kept in flight (submit i+1, then wait for i)
    outs = [(torch.empty((M, N), dtype=torch.bfloat16).pin_memory(), torch.empty((M, K), dtype=torch.bfloat16).pin_memory(),
             torch.empty((K, N), dtype=torch.bfloat16).pin_memory(), torch.empty((N,), dtype=torch.float32).pin_memory())
            for _ in range(2)]
    Y_o, dX_o, dW_o, db_o = outs[0]

    def e2e_submit(i):
        y, dx, dw, dbo = outs[i % 2]
        r = lib.ge2b_dense_plan_submit(plan, X_h.data_ptr(), W_h.data_ptr(), b_h.data_ptr(), dY_h.data_ptr(),
                                       y.data_ptr(), dx.data_ptr(), dw.data_ptr(), dbo.data_ptr())
        assert r == 0, r

    def e2e_run(n):
        e2e_submit(0)
        for i in range(1, n):
            e2e_submit(i)
            assert lib.ge2b_dense_plan_wait(plan) == 0       # step i-1 complete: its results are in host memory
        assert lib.ge2b_dense_plan_wait(plan) == 0

    e2e_steps = max(2, min(args.steps, 50))
    e2e_run(3)
    barrier()
    with ClockSampler(local) as clk2:
        w0 = time.perf_counter()
        e2e_run(e2e_steps)
        torch.cuda.synchronize()
        w1 = time.perf_counter()
    e2e_ms = torch.tensor([(w1 - w0) * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    lib.ge2b_dense_plan_destroy(plan)
    h2d = X_h.numel() * 2 + W_h.numel() * 2 + dY_h.numel() * 2 + b_h.numel() * 4
    d2h = Y_o.numel() * 2 + dX_o.numel() * 2 + dW_o.numel() * 2 + db_o.numel() * 4
    e2e_value = world * FLOP_PER_STEP * e2e_steps / (float(e2e_ms.item()) * 1e-3) / 1e12
    # plausibility of the plan's results against the device-resident run
    assert torch.equal(Y_o, Y.cpu()), "host-plan Y differs from the device-resident forward"

    # ---- the 3-layer MLP training step: global batch 8192 sharded along M (strong scaling), driven by the C++ plan
    # (ge2b_mlp_plan_*: buffers, warm-up, capture and replay inside the library; each layer's dW / db summed over the
    # ranks under the rest of the backward pass)
    mlp = None
    if not args.skip_mlp and 8192 % world == 0:
        rows = 8192 // world
        mp_ = pkg.MlpPlan([1024, 4096, 4096, 1024], ["relu", "gelu", "none"], rows, lr=1e-3, seed=0, device=dev,
                          group=dist.group.WORLD if world > 1 else None, global_batch=8192, comm_blocks=comm_sms,
                          exchange="nccl" if os.environ.get("GE2B_BENCH_EXCHANGE", "") == "nccl" else "auto")
        mp_.compile(capture=True)
        gen.manual_seed(100 + rank)
        Xm_h = torch.randn((rows, 1024), generator=gen).bfloat16().pin_memory()
        ym_h = torch.randint(0, 1024, (rows,), generator=gen, dtype=torch.int32).pin_memory()
        mp_.step_host(Xm_h, ym_h)                       # the batch is now in the plan's device buffers
        mst = mp_.stream()
        for _ in range(3):
            mp_.launch()
        barrier()

        def mlp_window(n):
            m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            mp_.launch()
            barrier()                  # the ranks enter the window together
            m0.record(mst)
            for _ in range(n):
                mp_.launch()
            m1.record(mst)
            barrier()
            mms = torch.tensor([m0.elapsed_time(m1)], device=dev)
            if world > 1:
                dist.all_reduce(mms, op=dist.ReduceOp.MAX)
            return float(mms.item())

        probe_n = max(5, min(args.steps, 20))
        probe = mlp_window(probe_n) / probe_n
        mlp_steps = max(20, int(500.0 / max(probe, 1e-3)) + 1)          # a window of at least half a second
        per = mlp_window(mlp_steps) / mlp_steps
        # end to end: every step copies its batch up from pinned host memory and reads the loss back
        e_n = max(5, min(args.steps, 30))
        mp_.step_host(Xm_h, ym_h)
        barrier()
        w0 = time.perf_counter()
        for _ in range(e_n):
            mloss = mp_.step_host(Xm_h, ym_h)
        w1 = time.perf_counter()
        e_t = torch.tensor([(w1 - w0) / e_n], device=dev)
        if world > 1:
            dist.all_reduce(e_t, op=dist.ReduceOp.MAX)
        mlp = {"workload": "3-layer MLP training step, global batch 8192, 1024-4096-4096-1024, ReLU/GELU/none, bf16 weights "
                           "with fp32 master, softmax cross-entropy, SGD lr=1e-3; batch rows sharded over the GPUs",
               "steps_per_s": 1e3 / per, "ms_per_step": per, "burst_steps_per_s": 1e3 / probe, "scaling": "strong",
               "steps_timed": mlp_steps, "tflops": world * mp_.flop_per_step() / (per * 1e-3) / 1e12,
               "driver": "ge2b_mlp_plan_* (C ABI): CUDA graph replay", "exchange": mp_.exchange,
               "gpu_launches_per_step": mp_.launches_per_step(),
               "e2e": {"steps_per_s": 1.0 / float(e_t.item()), "h2d_bytes_per_step": Xm_h.numel() * 2 + ym_h.numel() * 4,
                       "d2h_bytes_per_step": 4, "api": "ge2b_mlp_plan_step (pinned host batch up, loss back, every step)"},
               "loss": mp_.global_loss()}
        assert lib.ge2b_device_status(0) == 0
        mp_.close()

    if rank == 0:
        peak, peak_kind = measured_peak("bf16_tflops")
        peak_sus, _ = measured_peak("bf16_tflops_sustained")
        cs = clk.summary()

        def roof_block(name, flop, ms, ms_sus, ck, ck_sus, traffic, what):
            a_, a_s = flop / (ms * 1e-3) / 1e12, flop / (ms_sus * 1e-3) / 1e12
            return {"bound": "tensor", "achieved": a_, "peak": peak, "unit": "TFLOP/s", "frac": a_ / peak,
                    "traffic": traffic,
                    "traffic_source": f"{TRAFFIC_PROFILE} (ncu capture of `bench.py --profile fwd` / `--profile step`, "
                                      "not re-measured by this run)",
                    "kernel": f"gemm_tc_kernel, {name}: {what}; duration = CUDA events around a run of back-to-back graph "
                              "replays of that launch, between the burst window and the long window",
                    "launch_ms": ms, "share_of_step": ms / (burst_ms / args.steps), "clocks": ck.summary(),
                    "peak_source": f"MEASURED_PEAKS.json bf16_tflops (burst: the launch is timed alone, a few ms), {peak_kind}",
                    "frac_of_nominal_2250": a_ / NOMINAL_PEAK_TFLOPS,
                    "sustained": {"achieved": a_s, "launch_ms": ms_sus, "peak": peak_sus, "frac": a_s / peak_sus,
                                  "clocks": ck_sus.summary(),
                                  "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained (the same launch replayed for "
                                                 "half a second)"}}

        roof_fwd = roof_block("forward launch", FLOP_FWD_LAUNCH, fwd_ms, fwd_sustained_ms, clk_fwd_burst, clk_fwd,
                              launch_traffic("dram_bytes_per_launch"), "Y, Z = GELU(X.W + b), 2*M*N*K flop")
        roof_fwd["launch_ms_eager_events"] = fwd_eager_ms
        roof_bwd = roof_block("dX + dW launch", 2 * FLOP_FWD_LAUNCH, bwd_ms, bwd_sustained_ms, clk_bwd_burst, clk_bwd,
                              launch_traffic("dram_bytes_per_launch_dual") if bwd_gemm_launches == 1 else None,
                              "dX = gZ.W^T and dW = X^T.gZ as one tile list, 4*M*N*K flop")
        # the dominant kernel of the step is the one with the larger measured share; the other sits beside it
        if bwd_gemm_launches == 1 and bwd_ms >= fwd_ms:
            roofline = dict(roof_bwd, other_kernel=roof_fwd)
        else:
            roofline = dict(roof_fwd, other_kernel=roof_bwd if bwd_gemm_launches == 1 else None)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": total_ms / replays, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(CONFIG, parallelism=(f"dp{world} (rows of the batch; dW in {dw_chunks} row block(s), each summed over the "
                                                f"ranks under the rest of the backward; exchange: {bucket.impl})"
                                                if dw_chunks > 0 else
                                                f"dp{world} (rows of the batch; dX and dW in one launch, dW + db summed over the "
                                                f"ranks after it; exchange: {bucket.impl})")
                           if world > 1 else "single GPU"),
            "replays_timed": replays, "timed_region_s": total_ms * 1e-3,
            "window": f"value: the step replayed {replays} times (a region of at least {MIN_WINDOW_S} s, the clock the "
                      "power cap settles at); burst: exactly --steps steps",
            "burst": {"value": burst_value, "ms_per_step": burst_ms / args.steps, "steps": args.steps,
                      "clocks": clk_burst.summary()},
            "clocks": cs,
            "ms_x_ghz": (total_ms / replays * cs["sm_mhz"] / 1e3) if cs["sm_mhz"] else None,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "timer": "host clock from the first submit to the last wait, max over ranks",
                    "api": "ge2b_dense_plan_submit / _wait (C ABI, pinned host buffers, two steps in flight)", "clocks": clk2.summary()},
            "gpu_launches": int(launches), "launch_mode": "cuda graph replay" if graph is not None else "eager",
            "split_k_unavailable_in_capture": int(lib.ge2b_split_unavailable_total() - split_unavailable0),
            "roofline": roofline,
        }
        if target is not None:
            line["target_8192"] = target
        if allreduce_check is not None:
            line["allreduce_check"] = allreduce_check
            line["exchange"] = {"impl": bucket.impl, "fallback_reason": bucket.why or None, "sms": comm_sms,
                                "dw_row_blocks": dw_chunks}
        if mlp is not None:
            line["mlp_step"] = mlp
        if world == 1 and not args.skip_cpu_baseline:
            line["cpu_baseline"] = run_cpu_baseline()
            line["cpu_baseline_tuned"] = run_cpu_tuned()
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: destroying a process group whose collectives live in
        # instantiated CUDA graphs was seen to block at exit.  Everything has been synchronised and printed.
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# ------------------------------------------------------------------------------------------------ shape sweep
def run_sweep(args):
    """Shape sweep (squares and decode-like skinny M, four activations, bf16 and fp32
    via TF32 / exact) and the batched attention GEMMs (B*H = 128, L = 2048, d = 128).  One JSON line per point; not the contract line."""
    import ctypes as C
    import torch
    pkg = importlib.import_module("ai_framework-dev_b200")
    lib = pkg.load_library()
    og = pkg.ops_gemm
    torch.cuda.set_device(0)
    ref = None
    so = ROOT / "oracle" / "_ref" / "libref_gemm.so"
    if so.exists():
        ref = C.CDLL(str(so))
        ref.ref_gpu_forward.restype = C.c_int
        ref.ref_gpu_forward.argtypes = [C.c_void_p] * 3 + [C.c_longlong] + [C.c_void_p] * 2 + [C.c_int] * 4 + [C.c_float, C.c_void_p]
        ref.ref_gpu_backward.restype = C.c_int
        ref.ref_gpu_backward.argtypes = [C.c_void_p] * 7 + [C.c_longlong, C.c_void_p] + [C.c_int] * 4 + [C.c_float, C.c_void_p]
    act_code = {"none": 0, "relu": 1, "gelu": 3, "sigmoid": 4}

    def timeit(fn, iters, reps=8):
        """median over `iters` samples of the mean time of `reps` back-to-back launches (host launch cost amortised)"""
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / reps)
        return statistics.median(ts)

    def timeit_graph(fn, iters, reps=16):
        """the same launches captured once into a CUDA graph and replayed: no host work between the kernels"""
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            fn()                                   # the capture stream's own first (un-captured) run
        st.synchronize()
        g_ = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_, stream=st, capture_error_mode="thread_local"):
            for _ in range(reps):
                fn()
        torch.cuda.current_stream().wait_stream(st)
        g_.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g_.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / reps)
        return statistics.median(ts)

    hbm_peak = 6547.2
    try:
        hbm_peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"])
    except Exception:
        pass

    def dense_point(Mx, Nx, Kx, dtype, math, act, iters, with_ref=False):
        tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
        X = torch.randn((Mx, Kx), device="cuda").to(tdt)
        W = ((torch.rand((Kx, Nx), device="cuda") * 2 - 1) * (6.0 / Kx) ** 0.5).to(tdt)
        b = torch.rand((Nx,), device="cuda") * 0.2 - 0.1
        dY = torch.randn((Mx, Nx), device="cuda").to(tdt)
        Y, Z, work = (torch.empty((Mx, Nx), device="cuda", dtype=tdt) for _ in range(3))
        dX = torch.empty_like(X)
        dW = torch.empty_like(W)
        db = torch.empty((1, Nx), device="cuda")
        f = lambda: og.forward_into(X, W, out=Y, bias=b, with_bias=True, act=act, save_z=True, z_out=Z, math=math)  # noqa: E731
        g = lambda: og.backward_into(X, W, dY, Z, act=act, with_bias=True, gA_out=dX, gB_out=dW, gBias_out=db,  # noqa: E731
                                     work_dZ=work, math=math)
        tf, tb = timeit(f, iters), timeit(g, iters)
        small = Mx * Nx * Kx <= 4096 ** 3
        tfg, tbg = (timeit_graph(f, iters), timeit_graph(g, iters)) if small else (tf, tb)
        esz = 2 if dtype == "bf16" else 4
        fwd_bytes = esz * (Mx * Kx + Kx * Nx + 2 * Mx * Nx) + 4 * Nx          # X, W, bias in; Y, Z out
        line = {"sweep": "dense", "M": Mx, "N": Nx, "K": Kx, "dtype": dtype, "math": math, "act": act,
                "fwd_ms": round(tf, 4), "fwd_tflops": round(2.0 * Mx * Nx * Kx / tf / 1e9, 1),
                "bwd_ms": round(tb, 4), "bwd_tflops": round(4.0 * Mx * Nx * Kx / tb / 1e9, 1),
                "fwd_bwd_tflops": round(6.0 * Mx * Nx * Kx / (tf + tb) / 1e9, 1),
                "graph": {"fwd_ms": round(tfg, 4), "bwd_ms": round(tbg, 4),
                          "fwd_tflops": round(2.0 * Mx * Nx * Kx / tfg / 1e9, 1),
                          "bwd_tflops": round(4.0 * Mx * Nx * Kx / tbg / 1e9, 1),
                          "fwd_GBs": round(fwd_bytes / tfg / 1e6, 1),
                          "fwd_frac_of_hbm": round(fwd_bytes / tfg / 1e6 / hbm_peak, 3)} if small else None,
                "route": {1: "exact fp32 (CUDA cores)", 2: "tcgen05"}.get(lib.ge2b_last_route())}
        if with_ref and ref is not None and dtype == "fp32":
            scratch = torch.empty((Mx, Nx), device="cuda")
            rf = lambda: ref.ref_gpu_forward(X.data_ptr(), W.data_ptr(), b.data_ptr(), Nx, Y.data_ptr(), Z.data_ptr(),  # noqa: E731
                                             Mx, Kx, Nx, act_code[act], 0.01, None)
            rb = lambda: ref.ref_gpu_backward(X.data_ptr(), W.data_ptr(), dY.data_ptr(), Z.data_ptr(), dX.data_ptr(),  # noqa: E731
                                              dW.data_ptr(), db.data_ptr(), Nx, scratch.data_ptr(), Mx, Kx, Nx,
                                              act_code[act], 0.01, None)
            trf, trb = timeit(rf, max(2, iters // 2)), timeit(rb, max(2, iters // 2))
            line["reference_gpu_kernels"] = {"fwd_ms": round(trf, 4), "fwd_tflops": round(2.0 * Mx * Nx * Kx / trf / 1e9, 2),
                                             "bwd_ms": round(trb, 4), "bwd_tflops": round(4.0 * Mx * Nx * Kx / trb / 1e9, 2)}
        print(json.dumps(line), flush=True)

    quick = args.sweep_quick
    only = args.sweep_only

    def small_points():
        """small / skinny / MLP-layer shapes from a graph replay: full epilogue, plain epilogue, backward"""
        for (Mx, Nx, Kx) in [(1024, 1024, 1024), (2048, 2048, 2048), (16, 8192, 8192), (32, 8192, 8192), (128, 8192, 8192),
                             (1024, 4096, 1024), (1024, 4096, 4096), (1024, 1024, 4096)]:
            X = torch.randn(Mx, Kx, device="cuda").bfloat16()
            W = (torch.randn(Kx, Nx, device="cuda") / Kx ** 0.5).bfloat16()
            b = torch.randn(Nx, device="cuda")
            Y = torch.empty(Mx, Nx, device="cuda", dtype=torch.bfloat16)
            Z, dY, work = torch.empty_like(Y), torch.randn(Mx, Nx, device="cuda").bfloat16(), torch.empty_like(Y)
            dX, dW, db = torch.empty_like(X), torch.empty_like(W), torch.empty(1, Nx, device="cuda")
            tf = timeit_graph(lambda: og.forward_into(X, W, out=Y, bias=b, with_bias=True, act="gelu", save_z=True, z_out=Z), 7)
            tp = timeit_graph(lambda: og.forward_into(X, W, out=Y), 7)
            tb = timeit_graph(lambda: og.backward_into(X, W, dY, Z, act="gelu", with_bias=True, gA_out=dX, gB_out=dW,
                                                       gBias_out=db, work_dZ=work), 7)
            print(json.dumps({"sweep": "small", "M": Mx, "N": Nx, "K": Kx, "dtype": "bf16", "fwd_us": round(tf * 1e3, 1),
                              "fwd_plain_us": round(tp * 1e3, 1), "bwd_us": round(tb * 1e3, 1),
                              "fwd_tflops": round(2.0 * Mx * Nx * Kx / tf / 1e9, 1)}), flush=True)

    def fp32_mode_points():
        """fp32 tensors under the three math modes (eager): exact chain, compensated tensor cores, TF32"""
        for (Mx, Nx, Kx) in [(256, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096)]:
            X = torch.randn(Mx, Kx, device="cuda")
            W = torch.randn(Kx, Nx, device="cuda") / Kx ** 0.5
            b = torch.randn(Nx, device="cuda")
            Y = torch.empty(Mx, Nx, device="cuda")
            Z, dY, work = torch.empty_like(Y), torch.randn(Mx, Nx, device="cuda"), torch.empty_like(Y)
            dX, dW, db = torch.empty_like(X), torch.empty_like(W), torch.empty(1, Nx, device="cuda")
            rec = {"sweep": "fp32_modes", "M": Mx, "N": Nx, "K": Kx}
            for m in ("fp32", "fp32x3", "tf32"):
                rec["fwd_ms_" + m] = round(timeit(lambda: og.forward_into(X, W, out=Y, bias=b, with_bias=True, act="relu",
                                                                          save_z=True, z_out=Z, math=m), 5, reps=4), 4)
                rec["bwd_ms_" + m] = round(timeit(lambda: og.backward_into(X, W, dY, Z, act="relu", with_bias=True, gA_out=dX,
                                                                           gB_out=dW, gBias_out=db, work_dZ=work, math=m),
                                                  5, reps=4), 4)
            print(json.dumps(rec), flush=True)

    if only == "small":
        small_points()
        assert lib.ge2b_device_status(0) == 0
        return
    if only == "fp32":
        fp32_mode_points()
        assert lib.ge2b_device_status(0) == 0
        return
    for n in (() if only == "attention" else (1024, 2048, 4096, 8192, 16384)):
        for dtype, math in (("bf16", "fp32"), ("fp32", "tf32")):
            for act in (("gelu",) if quick else ("none", "relu", "gelu", "sigmoid")):
                dense_point(n, n, n, dtype, math, act, 5 if n <= 8192 else 2)
    if only != "attention":
        for m in (16, 32, 64, 128):
            for dtype, math in (("bf16", "fp32"), ("fp32", "tf32")):
                dense_point(m, 8192, 8192, dtype, math, "gelu", 7)
        for n in (256, 1024, 2048, 4096):          # the parity path and the reference's own kernels on the same box
            dense_point(n, n if n > 256 else 512, n if n > 256 else 512, "fp32", "fp32", "relu", 3, with_ref=True)
        if quick:
            assert lib.ge2b_device_status(0) == 0
            return
        small_points()
        fp32_mode_points()

    # batched attention GEMMs: B*H = 128 slices, L = 2048, d = 128, bf16, fp32 accumulate
    Bn, H, L, d = 8, 16, 2048, 128
    Q, Kt, V = (torch.randn((Bn, H, L, d), device="cuda").bfloat16() for _ in range(3))
    P = torch.softmax(torch.randn((Bn, H, L, L), device="cuda"), dim=-1).bfloat16()
    S = torch.empty((Bn, H, L, L), device="cuda", dtype=torch.bfloat16)
    O = torch.empty((Bn, H, L, d), device="cuda", dtype=torch.bfloat16)
    t_qk = timeit(lambda: og.forward_batched(Q, Kt, out=S, trans_b=True, alpha=1.0 / d ** 0.5), 7)
    t_pv = timeit(lambda: og.forward_batched(P, V, out=O), 7)
    flop = 2.0 * Bn * H * L * L * d
    for (b_, h_, l_, d_) in ((Bn, H, L, d), (Bn, H, L, 64), (2, 8, 4096, 128)):
        q_, k_, v_ = (torch.randn((b_, h_, l_, d_), device="cuda").bfloat16() for _ in range(3))
        o_ = torch.empty_like(q_)
        t_fa = timeit(lambda: pkg.ops_sdpa.forward(q_, k_, v_, out=o_), 7)
        t_fac = timeit(lambda: pkg.ops_sdpa.forward(q_, k_, v_, out=o_, causal=True), 7)
        fl = 4.0 * b_ * h_ * l_ * l_ * d_
        rec = {"sweep": "fused_attention", "B": b_, "H": h_, "L": l_, "d": d_, "dtype": "bf16",
               "fwd_ms": round(t_fa, 4), "fwd_tflops": round(fl / t_fa / 1e9, 1),
               "causal_fwd_ms": round(t_fac, 4), "causal_fwd_tflops": round(fl / 2 / t_fac / 1e9, 1),
               "note": "S = scale.Q.K^T, softmax and P.V in one launch: no S / P traffic"}
        try:       # the vendor's fused attention through torch, for context
            rec["torch_sdpa_ms"] = round(timeit(lambda: torch.nn.functional.scaled_dot_product_attention(q_, k_, v_), 7), 4)
        except Exception as e:  # noqa: BLE001
            rec["torch_sdpa_ms"] = None
        if (b_, h_, l_, d_) == (Bn, H, L, d):
            s_ = torch.empty((b_, h_, l_, l_), device="cuda", dtype=torch.bfloat16)
            p_ = torch.empty_like(s_)

            def unfused():
                og.forward_batched(q_, k_, out=s_, trans_b=True, alpha=1.0 / d_ ** 0.5)
                torch.softmax(s_, dim=-1, out=p_)
                og.forward_batched(p_, v_, out=o_)
            rec["two_gemms_and_softmax_through_hbm_ms"] = round(timeit(unfused, 3, reps=2), 4)
            del s_, p_
        print(json.dumps(rec), flush=True)
    print(json.dumps({"sweep": "batched_attention", "B": Bn, "H": H, "L": L, "d": d, "dtype": "bf16",
                      "qk_ms": round(t_qk, 4), "qk_tflops": round(flop / t_qk / 1e9, 1),
                      "qk_GBs": round((2 * Q.numel() * 2 + S.numel() * 2) / t_qk / 1e6, 1),
                      "pv_ms": round(t_pv, 4), "pv_tflops": round(flop / t_pv / 1e9, 1),
                      "pv_GBs": round((P.numel() * 2 + 2 * V.numel() * 2) / t_pv / 1e6, 1)}), flush=True)
    assert lib.ge2b_device_status(0) == 0
    if only == "attention":
        return
    run_conv_points(pkg, lib, timeit, timeit_graph)


CONV_POINTS = [  # name, N, Cin, H, W, Cout, k, stride, pad  (ResNet-50-like layer shapes, batch 32)
    ("3x3 64->64 56x56", 32, 64, 56, 56, 64, 3, 1, 1), ("3x3 128->128 28x28", 32, 128, 28, 28, 128, 3, 1, 1),
    ("3x3 128->128 28x28 s2", 32, 128, 56, 56, 128, 3, 2, 1),
    ("3x3 256->256 14x14", 32, 256, 14, 14, 256, 3, 1, 1), ("1x1 256->1024 14x14", 32, 256, 14, 14, 1024, 1, 1, 0),
    ("7x7 3->64 224x224 s2", 32, 3, 224, 224, 64, 7, 2, 3)]


def run_conv_points(pkg, lib, timeit, timeit_graph):
    """conv2d (+bias+ReLU, pre-activation saved) forward and backward through this library (replayed from a CUDA graph:
    no host launch cost in the timed region), the reference's own conv2d op (fp32, per-image loop) where its library
    was built, and torch's convolution of the same bf16 layer for context.  One JSON line per point."""
    import ctypes as C
    import torch
    cv = pkg.ops_conv2d
    ref = None
    so = ROOT / "oracle" / "_ref" / "libref_conv.so"
    if so.exists():
        ref = C.CDLL(str(so))
        ref.ref_conv_forward.argtypes = [C.c_void_p] * 5 + [C.c_int] * 14 + [C.c_float, C.c_void_p]
        ref.ref_conv_backward.argtypes = [C.c_void_p] * 7 + [C.c_int] * 14 + [C.c_float, C.c_void_p]
    for name, N, Cin, H, W, Cout, k, st, pd in CONV_POINTS:
        kw = dict(stride=(st, st), padding=(pd, pd))
        Ho, Wo = cv.out_hw(H, W, k, k, **kw)
        flop = 2.0 * N * Cout * Ho * Wo * Cin * k * k
        for dt, math in ((torch.bfloat16, "fp32"), (torch.float32, "tf32"), (torch.float32, "fp32")):
            X = torch.randn(N, Cin, H, W, device="cuda").to(dt)
            Wt = (torch.randn(Cout, Cin, k, k, device="cuda") / (Cin * k * k) ** 0.5).to(dt)
            b = torch.randn(Cout, device="cuda")
            Y = torch.empty(N, Cout, Ho, Wo, device="cuda", dtype=dt)
            Z, dY = torch.empty_like(Y), torch.randn(N, Cout, Ho, Wo, device="cuda").to(dt)
            gX, gW, gB = torch.empty_like(X), torch.empty_like(Wt), torch.empty(Cout, device="cuda")
            fwd = lambda: cv.forward_into(X, Wt, out=Y, B=b, with_bias=True, act="relu", save_z=True, Z_saved=Z,  # noqa: E731
                                          math=math, **kw)
            bwd = lambda: cv.backward_into(X, Wt, dY, Z, with_bias=True, act="relu", gX_out=gX, gW_out=gW,  # noqa: E731
                                           gB_out=gB, math=math, **kw)
            t_f, t_b = timeit_graph(fwd, 5), timeit_graph(bwd, 5)
            rec = {"sweep": "conv2d", "layer": name, "N": N, "dtype": str(dt)[6:], "math": math,
                   "fwd_ms": round(t_f, 4), "fwd_tflops": round(flop / t_f / 1e9, 1),
                   "bwd_ms": round(t_b, 4), "bwd_tflops": round(2 * flop / t_b / 1e9, 1)}
            if ref is not None and dt == torch.float32 and math == "fp32" and X.numel() < 5e7:
                geom = (N, Cin, H, W, Cout, k, k, st, st, pd, pd, 1, 1)
                rf = lambda: ref.ref_conv_forward(X.data_ptr(), Wt.data_ptr(), b.data_ptr(), Y.data_ptr(), Z.data_ptr(),  # noqa: E731
                                                  *geom, 1, 0.01, None)
                rb = lambda: ref.ref_conv_backward(X.data_ptr(), Wt.data_ptr(), dY.data_ptr(), Z.data_ptr(), gW.data_ptr(),  # noqa: E731
                                                   gB.data_ptr(), gX.data_ptr(), *geom, 1, 0.01, None)
                rec["reference_fwd_ms"] = round(timeit(rf, 1, reps=3), 3)
                rec["reference_bwd_ms"] = round(timeit(rb, 1, reps=3), 3)
            if dt == torch.bfloat16:
                bt = b.to(dt)
                try:
                    rec["torch_fwd_ms"] = round(timeit_graph(
                        lambda: torch.relu(torch.nn.functional.conv2d(X, Wt, bt, **kw)), 5), 4)
                except Exception:
                    rec["torch_fwd_ms"] = None
            print(json.dumps(rec), flush=True)
    assert lib.ge2b_device_status(0) == 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile", default="", choices=["", "fwd", "step", "conv", "qk", "sdpa"],
                    help="run a short fixed launch sequence (for ncu) instead of the benchmark")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="omit the CPU-oracle leg (profiling runs)")
    ap.add_argument("--skip-mlp", action="store_true", help="omit the MLP training-step leg")
    ap.add_argument("--skip-target", action="store_true", help="omit the M=N=K=8192 block")
    ap.add_argument("--sweep", action="store_true", help="print the shape sweep (one JSON line per point) and exit")
    ap.add_argument("--sweep-quick", action="store_true", help="with --sweep: GELU only, dense points only")
    ap.add_argument("--sweep-only", default="", choices=["", "small", "fp32", "attention"],
                    help="with --sweep: one section (small / skinny shapes from a graph replay; fp32 math modes; attention)")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
