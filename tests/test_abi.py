"""The C-ABI library loads and exports every symbol include/ge2_b200.h declares; struct layouts used by the
Python binding match the header; argument errors are reported with the reference's codes.  No compute."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_exports_every_declared_symbol(pkg, lib):
    header = (ROOT / "include" / "ge2_b200.h").read_text()
    declared = set(re.findall(r"\b(ge2b?_[a-z0-9_]+)\s*\(", header))
    declared -= {n for n in declared if n.endswith("_t")}
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(pkg._lib.EXPORTS) == declared


def test_struct_sizes_match_the_header(pkg, tmp_path):
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "ge2_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n",'
                   "sizeof(ge2_gemm_bias_act_params_t),sizeof(ge2_gemm_bias_act_params_ex_t),"
                   "sizeof(ge2_gemm_bias_act_bwd_params_t),sizeof(ge2_gemm_typed_params_t),"
                   "sizeof(ge2_gemm_bwd_typed_params_t),sizeof(ge2b_conv2d_params_t),"
                   "sizeof(ge2_softmax_ce_params_t),sizeof(ge2_sgd_params_t),sizeof(ge2b_allreduce_nvls_t),"
                   "sizeof(ge2b_mlp_config_t),sizeof(ge2b_sdpa_params_t));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    sizes = list(map(int, subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()))
    L = pkg._lib
    assert sizes == [C.sizeof(L.ParamsLegacy), C.sizeof(L.ParamsEx), C.sizeof(L.ParamsBwd), C.sizeof(L.ParamsTyped),
                     C.sizeof(L.ParamsBwdTyped), C.sizeof(L.ParamsConv2D), C.sizeof(L.ParamsSoftmaxCE), C.sizeof(L.ParamsSGD),
                     C.sizeof(L.AllreduceNvls), C.sizeof(L.MlpConfig), C.sizeof(L.ParamsSdpa)]


def test_argument_errors_use_reference_codes(pkg, lib):
    L = pkg._lib
    assert lib.ge2_launch(None, None, 0, None) == -1
    p = L.ParamsEx()
    bufs = L.make_bufs([0, 0, 0], p)
    assert lib.ge2_launch(b"no_such_kernel", bufs, len(bufs), None) == -1
    assert lib.ge2_launch(b"gemm_bias_act_f32_ex", bufs, 2, None) == -1          # too few buffers
    assert lib.ge2_launch(b"gemm_bias_act_bwd_f32_ex", bufs, 4, None) == -1      # backward wants 10 slots
    assert lib.ge2_launch(b"gemm_bias_act_f32_ex", bufs, len(bufs), None) == -1  # null pointers, zero sizes
    assert lib.ge2b_backward_scratch_bytes(8, 16) == 8 * 16 * 4
    assert lib.ge2b_backward_scratch_bytes(0, 16) == 0
    assert b"sm_100a" in lib.ge2b_version()


def test_missing_library_is_a_loud_error(pkg, monkeypatch, tmp_path):
    import pytest
    L = pkg._lib
    monkeypatch.setattr(L, "_LIB", None)
    monkeypatch.setattr(L, "library_path", lambda: tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or eager fallback"):
        L.load_library()


def test_cpp_registry_and_operator_api_validation(pkg, lib, tmp_path):
    """Compiles tests/cpp/dispatch_check.cpp against the library (g++, host only) and runs it."""
    exe = tmp_path / "dispatch_check"
    libdir = pkg.library_path().parent
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), str(ROOT / "tests" / "cpp" / "dispatch_check.cpp"),
                    "-o", str(exe), "-L", str(libdir), "-lge2_b200", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_parameter_block_and_registry_on_gpu(pkg, lib, tmp_path):
    """Compiles tests/cpp/param_block_gpu_check.cpp (g++, links the library and cudart) and runs it on the device:
    gemm_bias_act_f32 / _f32_ex / _bwd_f32 with the reference's parameter blocks and gemm_run_ex / gemm_bwd_run
    through the registry, Z and the ReLU output bit-exact against an ascending-k fmaf loop."""
    exe = tmp_path / "param_block_gpu_check"
    libdir = pkg.library_path().parent
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include",
                    str(ROOT / "tests" / "cpp" / "param_block_gpu_check.cpp"), "-o", str(exe),
                    "-L", str(libdir), "-lge2_b200", "-L", "/usr/local/cuda/lib64", "-lcudart",
                    f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stdout + r.stderr


def test_mixed_device_call_is_refused_before_any_launch(pkg):
    """All tensors of one call must be on one GPU; checked in Python before the C ABI is reached (no GPU needed:
    the tensors are stand-ins that only carry a device)."""
    from unittest import mock
    import torch
    a, b = mock.Mock(spec=torch.Tensor), mock.Mock(spec=torch.Tensor)
    a.is_cuda = b.is_cuda = True
    a.device, b.device = torch.device("cuda", 0), torch.device("cuda", 1)
    with pytest.raises(ValueError, match="different devices"):
        pkg.ops_gemm._one_device(a, None, b)
    assert pkg.ops_gemm._one_device(a, None, a) == torch.device("cuda", 0)
    with pytest.raises(ValueError):
        pkg.ops_gemm._one_device(torch.zeros(2))            # a CPU tensor
    with pytest.raises(ValueError):
        pkg.ops_gemm.forward_into(torch.zeros(2, 2), torch.zeros(2, 2), out=torch.zeros(2, 2))
