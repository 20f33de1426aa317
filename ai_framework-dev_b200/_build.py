"""Builds the CUDA launch layer (libge2_b200.so) in-tree with nvcc for sm_100a.

Incremental: a source is recompiled only when it or a header is newer than its object file.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
OBJ_DIR = PKG / "build"
LIB = LIB_DIR / "libge2_b200.so"

SOURCES = ["runtime.cu", "gemm_simt.cu", "gemm_tc.cu", "bwd_prologue.cu", "dense_ops.cu", "c_api.cu", "op_api.cu",
           "host_api.cu", "bwd_noalloc.cu", "train_step.cu", "dispatch.cu", "conv2d.cu", "conv2d_implicit.cu", "conv2d_patch.cu", "selftest.cu", "allreduce_nvls.cu", "mlp_plan.cu", "fp32x3.cu", "sdpa_fused.cu"] + \
          [f"gemm_tc_inst_{t}_{o}.cu" for t in ("16bit", "tf32") for o in ("kk", "km", "mk", "mm")]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fvisibility=default",
    "-diag-suppress", "177",
    "-DAI_USE_NVTX",        # the reference's switch for its profiler ranges (header-only NVTX from the CUDA toolkit)
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA launch layer cannot be built")
    return exe


def _newest_header() -> float:
    hdrs = list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h*"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, obj: Path, verbose: bool) -> None:
    cmd = [nvcc(), *NVCC_FLAGS, "-I", str(PKG.parent / "include"), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build(force: bool = False, verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    hdr_time = _newest_header()
    todo, objs = [], []
    for name in SOURCES:
        src = CSRC / name
        if not src.exists():
            continue
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            todo.append((src, obj))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for fut in [ex.submit(_compile, s, o, verbose) for s, o in todo]:
                fut.result()
    if todo or not LIB.exists():
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True))
