"""The allocation-free backward entry point (ge2_launch_gemm_bias_act_bwd_noalloc).

It serves callers that cannot allocate device memory themselves and cannot let the library do it either -- a
plugin running under a framework whose memory pool already owns the whole GPU, or a loop in which allocator
calls are banned -- by keeping the gZ scratch in a fixed 16 MiB array inside the library.  The test calls it
through the C ABI twice in a row, with different inputs, and compares each result with the ordinary entry point
given an explicit scratch buffer: gA and gB must be bit-identical (same kernels, same order), gBias within the
tolerance the other GPU tests use for it (it is summed with fp32 atomics).  The file name sorts last so that
the test runs after every other one; it also passes alone in a fresh process.

`test_noalloc_first_call_in_fresh_process_allocates_nothing` starts a new interpreter, makes the allocation-free
call the FIRST thing the library does there (at a shape whose dX and dW launches are split along the reduction, which
is where the ordinary entry creates a 64 MiB scratch): the first call may cost at most the loading of the library's
device image (code and the fixed array: 32 MiB observed, below that scratch), every later call must leave the device's
free memory exactly as it was.
"""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
ROOT = Path(__file__).resolve().parent.parent


def _call(pkg, lib, entry, A, W, gY, Z, act, scratch):
    L = pkg._lib
    M, K = A.shape
    N = W.shape[1]
    gA, gB = torch.full_like(A, float("nan")), torch.full_like(W, float("nan"))
    gBias = torch.full((N,), float("nan"), device="cuda")
    p = L.ParamsBwdTyped()
    p.base.M, p.base.N, p.base.K = M, N, K
    p.base.alpha, p.base.beta = 1.0, 0.0
    p.base.bias_kind, p.base.act_kind, p.base.leaky_slope = L.BIAS_PER_N, L.ACT[act], 0.01
    dt = {torch.float32: L.DT_F32, torch.bfloat16: L.DT_BF16}[A.dtype]
    p.dtype, p.z_dtype, p.math = dt, dt, L.MATH_TENSOR
    ptrs = [A.data_ptr(), W.data_ptr(), 0, gY.data_ptr(), Z.data_ptr(), gA.data_ptr(), gB.data_ptr(), 0,
            gBias.data_ptr()]
    if scratch is not None:
        ptrs.append(scratch.data_ptr())
        p.scratch_bytes = scratch.numel() * scratch.element_size()
    bufs = L.make_bufs(ptrs, p)
    rc = getattr(lib, entry)(bufs, len(bufs), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return gA, gB, gBias


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(640, 384, 512), (256, 512, 6144)])      # the second: dX is split along its reduction
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_backward_matches_ordinary_entry_twice(pkg, lib, dtype, shape):
    M, K, N = shape
    if dtype == torch.float32 and M * N * 4 > pkg._lib.NOALLOC_SCRATCH_BYTES:
        N //= 2
    for seed, act in ((0, "gelu"), (1, "relu")):        # two calls in a row share the fixed scratch
        g = torch.Generator(device="cuda").manual_seed(seed)
        A = torch.randn((M, K), device="cuda", generator=g).to(dtype)
        W = (torch.randn((K, N), device="cuda", generator=g) / 16).to(dtype)
        gY = torch.randn((M, N), device="cuda", generator=g).to(dtype)
        Z = torch.randn((M, N), device="cuda", generator=g).to(dtype)
        scratch = torch.empty((M, N), device="cuda", dtype=dtype)
        want = _call(pkg, lib, "ge2_launch_gemm_bias_act_bwd_typed", A, W, gY, Z, act, scratch)
        got = _call(pkg, lib, "ge2_launch_gemm_bias_act_bwd_noalloc", A, W, gY, Z, act, None)
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
        np.testing.assert_allclose(got[2].cpu().numpy(), want[2].cpu().numpy(), rtol=1e-4, atol=3e-4)
    assert lib.ge2b_device_status(1) == 0


_FRESH = textwrap.dedent('''
    import importlib, sys
    sys.path.insert(0, {root!r})
    import torch
    pkg = importlib.import_module("ai_framework-dev_b200")
    lib = pkg.load_library()
    L = pkg._lib
    torch.cuda.set_device(0)
    first_delta = []
    for dtype, code in ((torch.float32, L.DT_F32), (torch.bfloat16, L.DT_BF16)):
        # dX = gZ.W^T reduces over N: 96 k-blocks (of 32 fp32 / 64 bf16 elements) on 2 output tiles, which the launch
        # layer cuts into 4 slices along the reduction -- the case in which the ordinary entry creates its scratch
        M, K, N = (256, 512, 3072) if dtype == torch.float32 else (256, 512, 6144)
        g = torch.Generator(device="cuda").manual_seed(3)
        A = torch.randn((M, K), device="cuda", generator=g).to(dtype)
        W = (torch.randn((K, N), device="cuda", generator=g) / 16).to(dtype)
        gY = torch.randn((M, N), device="cuda", generator=g).to(dtype)
        Z = torch.randn((M, N), device="cuda", generator=g).to(dtype)
        gA, gB = torch.empty_like(A), torch.empty_like(W)
        gBias = torch.empty((N,), device="cuda")
        p = L.ParamsBwdTyped()
        p.base.M, p.base.N, p.base.K = M, N, K
        p.base.alpha, p.base.beta = 1.0, 0.0
        p.base.bias_kind, p.base.act_kind, p.base.leaky_slope = L.BIAS_PER_N, L.ACT["gelu"], 0.01
        p.dtype, p.z_dtype, p.math = code, code, L.MATH_TENSOR
        bufs = L.make_bufs([A.data_ptr(), W.data_ptr(), 0, gY.data_ptr(), Z.data_ptr(), gA.data_ptr(), gB.data_ptr(), 0,
                            gBias.data_ptr()], p)
        s = torch.cuda.current_stream().cuda_stream
        torch.cuda.synchronize()
        # First call of this kernel family in the process: the driver loads the library's device image now -- code
        # plus the fixed 16 MiB array itself, 32 MiB observed on B200 -- but neither the 64 MiB split-K scratch the
        # ordinary entry would create nor a stream-ordered pool for the fp32 mode's operand copies may come on top.
        free0 = torch.cuda.mem_get_info()[0]
        assert lib.ge2_launch_gemm_bias_act_bwd_noalloc(bufs, len(bufs), s) == 0
        torch.cuda.synchronize()
        free1 = torch.cuda.mem_get_info()[0]
        assert free0 - free1 < (48 << 20), ("the first allocation-free call took device memory", dtype, free0 - free1)
        first_delta.append(free0 - free1)
        for _ in range(2):                             # later calls: not a byte
            assert lib.ge2_launch_gemm_bias_act_bwd_noalloc(bufs, len(bufs), s) == 0
        torch.cuda.synchronize()
        free2 = torch.cuda.mem_get_info()[0]
        assert free2 == free1, ("device memory changed across the allocation-free call", dtype, free1 - free2)
        assert torch.isfinite(gA.float()).all() and torch.isfinite(gB.float()).all()
    assert lib.ge2b_device_status(1) == 0
    print("NOALLOC_OK", lib.ge2b_split_unavailable_total(), first_delta)
''')


@pytest.mark.gpu
def test_noalloc_first_call_in_fresh_process_allocates_nothing(lib):
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")      # code is loaded with the library, not at first launch
    r = subprocess.run([sys.executable, "-c", _FRESH.format(root=str(ROOT))], capture_output=True, text=True, timeout=600,
                       env=env)
    assert r.returncode == 0 and "NOALLOC_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_noalloc_backward_rejects_oversize(pkg, lib):
    """M*N*sizeof(element) beyond the fixed scratch is refused before anything touches the GPU."""
    L = pkg._lib
    p = L.ParamsBwdTyped()
    p.base.M, p.base.N, p.base.K = 4096, 4096, 64        # 64 MiB of fp32 gZ > 16 MiB
    p.dtype, p.z_dtype = L.DT_F32, L.DT_F32
    bufs = L.make_bufs([0] * 9, p)
    assert lib.ge2_launch_gemm_bias_act_bwd_noalloc(bufs, len(bufs), None) == -1
    p.base.M, p.base.N = 2048, 4096                      # 16 MiB of bf16: exactly the limit is accepted size-wise,
    p.dtype, p.z_dtype = L.DT_BF16, L.DT_BF16            # so the next refusal must come from the null pointers
    assert L.NOALLOC_SCRATCH_BYTES == 2048 * 4096 * 2
