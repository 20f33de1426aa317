"""The allocation-free backward entry point (ge2_launch_gemm_bias_act_bwd_noalloc).

It serves callers that cannot allocate device memory themselves and cannot let the library do it either -- a
plugin running under a framework whose memory pool already owns the whole GPU, or a loop in which allocator
calls are banned -- by keeping the gZ scratch in a fixed 16 MiB array inside the library.  The test calls it
through the C ABI twice in a row, with different inputs, and compares each result with the ordinary entry point
given an explicit scratch buffer: gA and gB must be bit-identical (same kernels, same order), gBias within the
tolerance the other GPU tests use for it (it is summed with fp32 atomics).  The file name sorts last so that
the test runs after every other one; it also passes alone in a fresh process.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")


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
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_backward_matches_ordinary_entry_twice(pkg, lib, dtype):
    M, K, N = 640, 384, 512
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
