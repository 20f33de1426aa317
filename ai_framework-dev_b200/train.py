"""The training step around the dense layers: fused softmax cross-entropy, the SGD update, and a static,
graph-captured step driver for a stack of Dense layers.

Mirrors, for this path only, what the reference assembles in Python:
  * losses/softmax_ce.py + ops/cross_entropy.py  -> `softmax_ce_fused`
  * optim/sgd.py (fp32 master parameters)        -> `sgd_update`
  * layers/sequential.py:416-497 (compile / one_step), graph/capture_plan.py:250-287 (pre-allocated y, z, gA, gW, gB
    and work buffers per Dense layer), graph/runtime.py:24-148 (forward -> loss -> backward -> optimizer on one
    stream) and graph/graph_exec.py:51-152 (warm-up, capture, instantiate, replay) -> `DenseStackTrainer`
Device arrays are torch tensors; every kernel is launched through the C ABI of libge2_b200.so.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from . import _lib, ops_gemm
from ._lib import DT_BF16, DT_F16, DT_F32

_DT = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}
_RED = {"none": 0, "mean": 1, "sum": 2}


_stream_ptr = ops_gemm._stream_ptr
_one_device = ops_gemm._one_device


def softmax_ce_fused(logits: torch.Tensor, labels: torch.Tensor, *, dlogits: torch.Tensor,
                     loss: Optional[torch.Tensor] = None, reduction: str = "mean", ignore_index: int = -1,
                     grad_scale: Optional[float] = None, mean_denominator: int = 0, label_smoothing: float = 0.0,
                     stream=None) -> None:
    """loss = CE(softmax(logits), labels) and dlogits = (softmax - onehot) * grad_scale in one pass.
    labels are int32.  grad_scale defaults to 1/rows for "mean" and 1 otherwise; pass 1/global_batch (and
    mean_denominator = global_batch) when the rows are one shard of a data-parallel batch."""
    M, C = logits.shape
    if labels.dtype != torch.int32 or labels.numel() != M:
        raise ValueError("labels must be int32 of length M")
    if tuple(dlogits.shape) != (M, C):
        raise ValueError("dlogits must have the shape of logits")
    if loss is not None and (loss.dtype != torch.float32 or loss.numel() != (M if reduction == "none" else 1)):
        raise ValueError("loss must be float32 with M elements (reduction none) or 1 element")
    p = _lib.ParamsSoftmaxCE()
    p.M, p.C = M, C
    p.ld_logits, p.ld_dlogits = logits.stride(0), dlogits.stride(0)
    p.dtype, p.grad_dtype = _DT[logits.dtype], _DT[dlogits.dtype]
    p.reduction = _RED[reduction]
    p.ignore_index = ignore_index
    denom = mean_denominator if mean_denominator > 0 else M
    p.grad_scale = float(grad_scale) if grad_scale is not None else (1.0 / denom if reduction == "mean" else 1.0)
    p.mean_denominator = mean_denominator
    p.label_smoothing = float(label_smoothing)
    bufs = _lib.make_bufs([logits.data_ptr(), labels.data_ptr(), dlogits.data_ptr(),
                           loss.data_ptr() if loss is not None else 0], p)
    device = _one_device(logits, labels, dlogits, loss)
    with torch.cuda.device(device):
        _lib.check(_lib.load_library().ge2_launch_softmax_ce_fused(bufs, len(bufs), _stream_ptr(stream, device)),
                   "softmax_ce")


def sgd_update(param: torch.Tensor, grad: torch.Tensor, *, lr: float, velocity: Optional[torch.Tensor] = None,
               momentum: float = 0.0, dampening: float = 0.0, nesterov: bool = False, weight_decay: float = 0.0,
               decay: str = "decoupled", grad_scale: float = 1.0, low: Optional[torch.Tensor] = None,
               stream=None) -> None:
    """In-place SGD on fp32 `param`; `low` (bf16 / f16, same element count) receives the rounded result."""
    if param.dtype != torch.float32 or not param.is_contiguous() or not grad.is_contiguous():
        raise ValueError("param must be contiguous float32 and grad contiguous")
    if grad.numel() != param.numel() or (low is not None and low.numel() != param.numel()):
        raise ValueError("size mismatch")
    p = _lib.ParamsSGD()
    p.n = param.numel()
    p.grad_dtype = _DT[grad.dtype]
    p.low_dtype = _DT[low.dtype] if low is not None else DT_BF16
    p.lr, p.momentum, p.dampening = float(lr), float(momentum), float(dampening)
    p.nesterov = 1 if nesterov else 0
    p.weight_decay = float(weight_decay)
    p.decay_mode = 0 if weight_decay == 0.0 else {"l2": 1, "decoupled": 2}[decay]
    p.grad_scale = float(grad_scale)
    bufs = _lib.make_bufs([param.data_ptr(), grad.data_ptr(), velocity.data_ptr() if velocity is not None else 0,
                           low.data_ptr() if low is not None else 0], p)
    device = _one_device(param, grad, velocity, low)
    with torch.cuda.device(device):
        _lib.check(_lib.load_library().ge2_launch_sgd_update(bufs, len(bufs), _stream_ptr(stream, device)), "sgd_update")


def shard_rows(global_batch: int, world: int, rank: int):
    """Row range [begin, end) of `rank`'s shard of a batch split along M over `world` replicas (contiguous blocks,
    the first `global_batch % world` ranks get one extra row)."""
    if world < 1 or not (0 <= rank < world) or global_batch < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(global_batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def loss_grad_scale(global_batch: int) -> float:
    """Scale of the loss gradient on every replica for a mean loss over the GLOBAL batch: summing the replicas'
    dW / db then gives the full-batch gradient, whatever the shard sizes."""
    return 1.0 / float(global_batch)


class DenseStackTrainer:
    """Dense(d0->d1, act0) ... Dense(d_{n-1}->d_n, act_{n-1}) -> softmax cross-entropy (mean) -> SGD.

    All buffers are allocated in `compile`; `one_step` copies a batch into the static input buffers and runs the
    step: eagerly, or (single process) by replaying a CUDA graph captured once.  With a process group the batch
    rows are one shard of the global batch: each layer's dW and db are all-reduced (sum) on a side stream as soon
    as they are written, under the dX GEMM and the deeper layers' backward; the loss gradient is scaled by
    1/global_batch so every replica applies the same update.
    """

    def __init__(self, dims: Sequence[int], acts: Sequence[str], batch: int, *, dtype=torch.bfloat16, lr=1e-3,
                 seed=0, device="cuda", group=None, global_batch: Optional[int] = None, bias_init_zero=True):
        assert len(acts) == len(dims) - 1
        self.dims, self.acts, self.batch = list(dims), [a.lower() for a in acts], int(batch)
        self.dtype, self.lr, self.device = dtype, float(lr), device
        self.group = group
        self.world = torch.distributed.get_world_size(group) if group is not None else 1
        self.global_batch = int(global_batch) if global_batch else self.batch * self.world
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.W32: List[torch.Tensor] = []
        self.W: List[torch.Tensor] = []
        self.b: List[torch.Tensor] = []
        for i in range(len(dims) - 1):
            lim = math.sqrt(6.0 / dims[i])                       # Kaiming-uniform, as the benchmark config states
            w = ((torch.rand((dims[i], dims[i + 1]), generator=gen) * 2 - 1) * lim).to(device)
            self.W32.append(w.float().contiguous())
            self.W.append(w.to(dtype).contiguous())
            bias = torch.zeros(dims[i + 1]) if bias_init_zero else (torch.rand(dims[i + 1], generator=gen) * 0.2 - 0.1)
            self.b.append(bias.float().to(device))
        self.graph = None
        self.compiled = False

    # ---- plan (pre-allocated, pointer-stable buffers) ----
    def compile(self, capture=True) -> None:
        """capture: False = eager steps; True = CUDA graph when there is no process group; "with_collectives" =
        capture the step including its all-reduces."""
        B, dev, dt = self.batch, self.device, self.dtype
        n = len(self.W)
        self.X = torch.zeros((B, self.dims[0]), device=dev, dtype=dt)
        self.labels = torch.zeros((B,), device=dev, dtype=torch.int32)
        self.y = [torch.empty((B, self.dims[i + 1]), device=dev, dtype=dt) for i in range(n)]
        self.z = [torch.empty((B, self.dims[i + 1]), device=dev, dtype=dt) for i in range(n)]
        self.work = [torch.empty((B, self.dims[i + 1]), device=dev, dtype=dt) for i in range(n)]
        self.gA = [torch.empty((B, self.dims[i]), device=dev, dtype=dt) for i in range(n)]
        self.gW = [torch.empty_like(w) for w in self.W]
        self.gB = [torch.empty((1, self.dims[i + 1]), device=dev, dtype=torch.float32) for i in range(n)]
        self.dlogits = torch.empty((B, self.dims[-1]), device=dev, dtype=dt)
        self.loss = torch.zeros((1,), device=dev, dtype=torch.float32)
        self.comm = torch.cuda.Stream(device=dev) if self.world > 1 else None
        self.compiled = True
        # Warm-up outside capture (function attributes, per-stream split-K scratch, NCCL channels).  A step updates
        # the parameters, so they are saved and put back: training starts from the initial weights.
        saved = [t.clone() for t in (*self.W32, *self.W, *self.b)]
        want_graph = bool(capture) and (self.world == 1 or capture == "with_collectives")
        cap = torch.cuda.Stream(device=dev) if want_graph else None
        self.run_step()
        if cap is not None:           # the stream that will be captured must have run the step once itself
            cap.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cap):
                self.run_step()
            torch.cuda.current_stream().wait_stream(cap)
        else:
            self.run_step()
        torch.cuda.synchronize()
        for t, s0 in zip((*self.W32, *self.W, *self.b), saved):
            t.copy_(s0)
        torch.cuda.synchronize()
        if want_graph:
            cap.wait_stream(torch.cuda.current_stream())
            self.graph = torch.cuda.CUDAGraph()
            # thread-local capture mode: the collective library's watchdog thread may touch the CUDA API meanwhile
            with torch.cuda.graph(self.graph, stream=cap, capture_error_mode="thread_local"):
                self.run_step()
            torch.cuda.current_stream().wait_stream(cap)

    # ---- one step on the current stream ----
    def run_step(self) -> None:
        n = len(self.W)
        cur = self.X
        for i in range(n):
            ops_gemm.forward_into(cur, self.W[i], out=self.y[i], bias=self.b[i], with_bias=True, act=self.acts[i],
                                  save_z=True, z_out=self.z[i])
            cur = self.y[i]
        softmax_ce_fused(self.y[-1], self.labels, dlogits=self.dlogits, loss=self.loss, reduction="mean",
                         grad_scale=loss_grad_scale(self.global_batch), mean_denominator=self.global_batch)
        g = self.dlogits
        stream = torch.cuda.current_stream()
        for i in reversed(range(n)):
            x_in = self.X if i == 0 else self.y[i - 1]
            # gZ (into work) + db + dW first, so their all-reduce can start before dX is computed
            ops_gemm.backward_into(x_in, self.W[i], g, self.z[i], act=self.acts[i], with_bias=True,
                                   gB_out=self.gW[i], gBias_out=self.gB[i], work_dZ=self.work[i])
            if self.world > 1:
                self.comm.wait_stream(stream)
                with torch.cuda.stream(self.comm):
                    torch.distributed.all_reduce(self.gW[i], group=self.group)
                    torch.distributed.all_reduce(self.gB[i], group=self.group)
            ops_gemm.backward_into(x_in, self.W[i], g, self.z[i], act=self.acts[i], gA_out=self.gA[i],
                                   work_dZ=self.work[i], reuse_dZ=True)
            g = self.gA[i]
        if self.world > 1:
            stream.wait_stream(self.comm)
        for i in range(n):
            sgd_update(self.W32[i], self.gW[i], lr=self.lr, low=self.W[i])
            sgd_update(self.b[i], self.gB[i], lr=self.lr)

    def launch(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        else:
            self.run_step()

    def one_step(self, X: torch.Tensor, labels: torch.Tensor) -> float:
        """Copies the batch into the static buffers, runs one step and returns this replica's share of the mean loss
        (see global_loss)."""
        if not self.compiled:
            self.compile()
        self.X.copy_(X, non_blocking=True)
        self.labels.copy_(labels, non_blocking=True)
        self.launch()
        return float(self.loss.item())

    def global_loss(self) -> float:
        """Mean loss over the GLOBAL batch: every replica holds its rows' sum over the global denominator, so the
        replicas' values add up to the loss (the same number whatever the number of replicas)."""
        t = self.loss.clone()
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)
        return float(t.item())

    def flop_per_step(self) -> float:
        """2*B*sum(d_i*d_{i+1}) forward, twice that backward (dX is computed for the first layer too)."""
        return 6.0 * self.batch * sum(self.dims[i] * self.dims[i + 1] for i in range(len(self.W)))


class MlpPlan:
    """The C++ step driver (csrc/mlp_plan.cu) behind its C ABI: Dense stack -> softmax cross-entropy -> SGD, buffers and
    CUDA graph owned by the library.  This class only builds the configuration, draws the initial weights the way
    `DenseStackTrainer` does (Kaiming-uniform from a seeded CPU generator) and, under data parallelism, obtains the
    symmetric gradient buffer (or the collective library's unique id) from torch.distributed."""

    def __init__(self, dims: Sequence[int], acts: Sequence[str], batch: int, *, dtype=torch.bfloat16, lr=1e-3, seed=0,
                 device="cuda", group=None, global_batch: Optional[int] = None, bias_init_zero=True,
                 exchange: str = "auto", comm_blocks: int = 16):
        import ctypes as C
        self._C = C
        self.lib = _lib.load_library()
        self.dims, self.acts, self.batch = [int(d) for d in dims], [a.lower() for a in acts], int(batch)
        self.dtype, self.device = dtype, torch.device(device)
        self.group = group
        self.world = torch.distributed.get_world_size(group) if group is not None else 1
        self.rank = torch.distributed.get_rank(group) if group is not None else 0
        self.global_batch = int(global_batch) if global_batch else self.batch * self.world
        cfg = _lib.MlpConfig()
        cfg.n_layers = len(self.acts)
        for i, d in enumerate(self.dims):
            cfg.dims[i] = d
        for i, a in enumerate(self.acts):
            cfg.acts[i] = _lib.ACT[a]
        cfg.batch, cfg.global_batch, cfg.dtype, cfg.lr = self.batch, self.global_batch, _DT[dtype], float(lr)
        cfg.world, cfg.rank, cfg.comm_blocks = self.world, self.rank, int(comm_blocks)
        self.exchange, self._keep = "none", []
        with torch.cuda.device(self.device):
            if self.world > 1:
                nbytes = int(self.lib.ge2b_mlp_plan_grad_bytes(C.byref(cfg)))
                handle = None
                if exchange in ("auto", "nvls") and dtype in (torch.bfloat16, torch.float32):
                    try:
                        import torch.distributed._symmetric_memory as symm_mem
                        buf = symm_mem.empty((nbytes,), dtype=torch.uint8, device=self.device)
                        buf.zero_()
                        torch.cuda.synchronize(self.device)
                        handle = symm_mem.rendezvous(buf, group)
                        if int(handle.multicast_ptr) == 0:
                            handle = None
                    except Exception:  # noqa: BLE001
                        handle = None
                    if handle is None and exchange == "nvls":
                        raise RuntimeError("no symmetric memory with a multicast mapping for this process group")
                if handle is not None:
                    peers = (C.c_void_p * self.world)(*[int(p) for p in handle.buffer_ptrs])
                    cfg.exchange, cfg.grad_base, cfg.grad_multicast = 1, buf.data_ptr(), int(handle.multicast_ptr)
                    cfg.peer_grad_bases = C.cast(peers, C.POINTER(C.c_void_p))
                    self._keep += [buf, handle, peers]
                    self.exchange = "nvls kernel"
                else:
                    uid = torch.zeros(128, dtype=torch.uint8)
                    if self.rank == 0:
                        _lib.check(self.lib.ge2b_nccl_unique_id(uid.data_ptr()), "nccl_unique_id")
                    dev_uid = uid.to(self.device)
                    torch.distributed.broadcast(dev_uid, src=torch.distributed.get_global_rank(group, 0), group=group)
                    uid = dev_uid.cpu()
                    cfg.exchange, cfg.nccl_unique_id = 2, uid.data_ptr()
                    self._keep.append(uid)
                    self.exchange = "nccl"
            self._plan = C.c_void_p()
            _lib.check(self.lib.ge2b_mlp_plan_create(C.byref(self._plan), C.byref(cfg)), "mlp_plan_create")
            gen = torch.Generator(device="cpu").manual_seed(seed)
            for i in range(len(self.acts)):
                lim = math.sqrt(6.0 / self.dims[i])
                w = ((torch.rand((self.dims[i], self.dims[i + 1]), generator=gen) * 2 - 1) * lim).float().contiguous()
                b = (torch.zeros(self.dims[i + 1]) if bias_init_zero
                     else (torch.rand(self.dims[i + 1], generator=gen) * 0.2 - 0.1)).float().contiguous()
                _lib.check(self.lib.ge2b_mlp_plan_set_params(self._plan, i, w.data_ptr(), b.data_ptr()), "mlp_set_params")
        self.captured = False

    def compile(self, capture: bool = True) -> None:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.ge2b_mlp_plan_compile(self._plan, 1 if capture else 0), "mlp_plan_compile")
        self.captured = bool(capture)

    def stream(self) -> "torch.cuda.ExternalStream":
        return torch.cuda.ExternalStream(int(self.lib.ge2b_mlp_plan_buffer(self._plan, 3)), device=self.device)

    def launch(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.ge2b_mlp_plan_launch(self._plan), "mlp_plan_launch")

    def step_host(self, X: Optional[torch.Tensor], labels: Optional[torch.Tensor], want_loss=True) -> Optional[float]:
        """One step from host tensors (X in the compute dtype, int32 labels; pinned memory copies asynchronously).
        Returns this replica's share of the mean loss when asked to (that waits for the step)."""
        C = self._C
        loss = C.c_float(0.0)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.ge2b_mlp_plan_step(self._plan, X.data_ptr() if X is not None else None,
                                                   labels.data_ptr() if labels is not None else None,
                                                   C.byref(loss) if want_loss else None), "mlp_plan_step")
        return float(loss.value) if want_loss else None

    def sync(self) -> None:
        _lib.check(self.lib.ge2b_mlp_plan_sync(self._plan), "mlp_plan_sync")

    def params(self, layer: int):
        """(W fp32 master, b, W in the compute dtype) of one layer as CPU tensors."""
        W = torch.empty((self.dims[layer], self.dims[layer + 1]), dtype=torch.float32)
        b = torch.empty((self.dims[layer + 1],), dtype=torch.float32)
        Wl = torch.empty((self.dims[layer], self.dims[layer + 1]), dtype=self.dtype)
        _lib.check(self.lib.ge2b_mlp_plan_get_params(self._plan, layer, W.data_ptr(), b.data_ptr(), Wl.data_ptr()), "get_params")
        return W, b, Wl

    def grads(self, layer: int):
        gW = torch.empty((self.dims[layer], self.dims[layer + 1]), dtype=self.dtype)
        gb = torch.empty((self.dims[layer + 1],), dtype=torch.float32)
        _lib.check(self.lib.ge2b_mlp_plan_get_grads(self._plan, layer, gW.data_ptr(), gb.data_ptr()), "get_grads")
        return gW, gb

    def launches_per_step(self) -> int:
        return int(self.lib.ge2b_mlp_plan_launches_per_step(self._plan))

    def flop_per_step(self) -> float:
        return 6.0 * self.batch * sum(self.dims[i] * self.dims[i + 1] for i in range(len(self.acts)))

    def global_loss(self) -> float:
        """Mean loss over the global batch of the last step (the replicas' shares add up to it)."""
        self.sync()
        out = torch.zeros(1, device=self.device)
        loss = self.step_loss_tensor()
        out.copy_(loss)
        if self.world > 1:
            torch.distributed.all_reduce(out, group=self.group)
        return float(out.item())

    def step_loss_tensor(self) -> torch.Tensor:
        """The plan's loss scalar as a 1-element CUDA tensor aliasing the library's buffer."""
        ptr = int(self.lib.ge2b_mlp_plan_buffer(self._plan, 2))
        return _alias_cuda(ptr, (1,), torch.float32, self.device)

    def input_tensors(self):
        """(X, labels) aliasing the plan's static device buffers, for filling a batch on the device."""
        X = _alias_cuda(int(self.lib.ge2b_mlp_plan_buffer(self._plan, 0)), (self.batch, self.dims[0]), self.dtype, self.device)
        y = _alias_cuda(int(self.lib.ge2b_mlp_plan_buffer(self._plan, 1)), (self.batch,), torch.int32, self.device)
        return X, y

    def close(self) -> None:
        if getattr(self, "_plan", None) is not None and self._plan:
            self.lib.ge2b_mlp_plan_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


class _CudaArray:
    """Minimal __cuda_array_interface__ carrier so that torch can alias memory the library owns."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3,
                                         "strides": None}


def _alias_cuda(ptr: int, shape, dtype, device) -> torch.Tensor:
    if dtype == torch.bfloat16:                     # no typestr for bf16: alias as int16 and reinterpret
        with torch.cuda.device(device):
            return torch.as_tensor(_CudaArray(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.float16: "<f2"}[dtype]
    with torch.cuda.device(device):
        return torch.as_tensor(_CudaArray(ptr, shape, typestr), device=device)
