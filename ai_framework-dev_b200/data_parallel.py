"""Data-parallel plumbing of the dense-layer path: gradient buckets in symmetric memory and their all-reduce.

The path shards the batch along M; dW and db are partial sums that have to be added across the GPUs once per step.
`GradBucket` puts the gradient tensors of one exchange (bf16 / f16 / fp32 weight gradients and fp32 bias gradients) into
ONE allocation that every rank maps into a multicast object, and `all_reduce` launches this library's own kernel
(csrc/allreduce_nvls.cu: in-switch reduction with multimem.ld_reduce, results broadcast with multimem.st) through the
C ABI.  torch.distributed only provides what a C caller would get from its own runtime: the process group, the
symmetric allocation and the exchange of its handles.  Where that allocation or the multicast mapping is not available
the bucket falls back to ordinary tensors and the collective library's all-reduce, and says so in `impl`.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import DT_BF16, DT_F32

_ALIGN = 256


def _round_up(n: int, a: int) -> int:
    return -(-n // a) * a


class GradBucket:
    """regions: [(shape, dtype), ...] laid out one after the other (256-byte aligned) in one symmetric buffer.
    `views[i]` is the tensor of region i.  `all_reduce(first, last)` sums regions first..last (inclusive) over the
    group: they must form at most two runs of one dtype each (e.g. a bf16 dW followed by an fp32 db)."""

    def __init__(self, regions: Sequence[Tuple[Tuple[int, ...], torch.dtype]], group, device, blocks: int = 32,
                 force_nccl: bool = False):
        self.group, self.device, self.blocks = group, torch.device(device), int(blocks)
        self.world = torch.distributed.get_world_size(group)
        self.rank = torch.distributed.get_rank(group)
        self.offsets: List[int] = []
        off = 0
        for shape, dtype in regions:
            if dtype not in (torch.bfloat16, torch.float32):
                raise ValueError("gradient regions must be bfloat16 or float32")
            self.offsets.append(off)
            n = 1
            for d in shape:
                n *= int(d)
            off = _round_up(off + n * torch.empty((), dtype=dtype).element_size(), _ALIGN)
        self.regions = [(tuple(int(d) for d in s), dt) for s, dt in regions]
        self.data_bytes = off
        lib = _lib.load_library()
        self.pad_bytes = int(lib.ge2b_allreduce_nvls_pad_bytes())
        total = self.data_bytes + self.pad_bytes
        self.impl, self.why = "nccl", "forced" if force_nccl else ""
        self._handle = None
        buf = None
        if not force_nccl and self.world >= 2 and self.device.type == "cuda":
            try:
                import torch.distributed._symmetric_memory as symm_mem
                buf = symm_mem.empty((total,), dtype=torch.uint8, device=self.device)
                buf.zero_()                                    # the signal pad must start at zero
                torch.cuda.synchronize(self.device)
                self._handle = symm_mem.rendezvous(buf, group)
                if int(self._handle.multicast_ptr) == 0:
                    self.why = "no multicast mapping for this group"
                    self._handle = None
                else:
                    self.impl = "nvls kernel"
            except Exception as e:  # noqa: BLE001 - anything the allocator or the rendezvous raises means "not here"
                self.why = f"symmetric memory unavailable: {type(e).__name__}: {e}"[:300]
                self._handle, buf = None, None
        if buf is None:
            buf = torch.zeros((total,), dtype=torch.uint8, device=self.device)
        self.buffer = buf
        self.views: List[torch.Tensor] = []
        for (shape, dtype), o in zip(self.regions, self.offsets):
            n = 1
            for d in shape:
                n *= d
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            self.views.append(buf[o:o + nbytes].view(dtype).view(shape))
        if self._handle is not None:
            ptrs = [int(p) + self.data_bytes for p in self._handle.buffer_ptrs]
            self._pads = (C.c_void_p * self.world)(*ptrs)
            self._mc = int(self._handle.multicast_ptr)

    def _segments(self, first: int, last: int):
        segs = []
        for i in range(first, last + 1):
            (shape, dtype), o = self.regions[i], self.offsets[i]
            end = self.offsets[i + 1] if i + 1 < len(self.offsets) else self.data_bytes   # aligned end (padding is zero)
            code = DT_BF16 if dtype == torch.bfloat16 else DT_F32
            if segs and segs[-1][2] == code and segs[-1][0] + segs[-1][1] == o:
                segs[-1] = (segs[-1][0], end - segs[-1][0], code)
            else:
                segs.append((o, end - o, code))
        if len(segs) > 2:
            raise ValueError("an exchange covers at most two runs of one dtype each")
        return segs

    def all_reduce(self, first: int = 0, last: Optional[int] = None, stream=None) -> None:
        """Sum over the group, in place, asynchronous on `stream` (default: the current stream)."""
        last = len(self.regions) - 1 if last is None else last
        if self._handle is None:
            if self.device.type != "cuda":                    # host ranks (tests of the bucket logic on CPU process groups)
                for i in range(first, last + 1):
                    torch.distributed.all_reduce(self.views[i], group=self.group)
                return
            s = stream if isinstance(stream, torch.cuda.Stream) else None
            ctx = torch.cuda.stream(s) if s is not None else torch.cuda.stream(torch.cuda.current_stream(self.device))
            with ctx:
                for i in range(first, last + 1):
                    torch.distributed.all_reduce(self.views[i], group=self.group)
            return
        a = _lib.AllreduceNvls()
        a.multicast_base = self._mc
        a.signal_pads = C.cast(self._pads, C.POINTER(C.c_void_p))
        a.world, a.rank = self.world, self.rank
        segs = self._segments(first, last)
        a.n_segments = len(segs)
        for j, (o, n, code) in enumerate(segs):
            a.segments[j].offset_bytes, a.segments[j].bytes, a.segments[j].dtype = o, n, code
        a.blocks = self.blocks
        if stream is None:
            sp = int(torch.cuda.current_stream(self.device).cuda_stream)
        else:
            sp = int(stream.cuda_stream) if isinstance(stream, torch.cuda.Stream) else int(stream)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load_library().ge2b_allreduce_nvls(C.byref(a), sp), "allreduce_nvls")
