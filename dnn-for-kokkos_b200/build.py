"""Builds libkdnn_b200.so (the CUDA kernels and the C ABI) in-tree with nvcc for
sm_100a. Run as ``python build.py`` from this folder, or call ``build_library()``."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["kdnn_gemv.cu", "kdnn_gemm.cu", "kdnn_moe.cu", "kdnn_dequant.cu", "kdnn_capi.cu"]
HEADERS = ["kdnn_common.cuh", "kdnn_tile.cuh", "kdnn_grouped.cuh", "kdnn_mma.cuh", "kdnn_umma.cuh", os.path.join("..", "..", "include", "kdnn_b200.h")]
LIB = os.path.join(HERE, "libkdnn_b200.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libkdnn_b200.so cannot be built")


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, "csrc", s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []),
           *[os.path.join(HERE, "csrc", s) for s in SOURCES], "-o", LIB]
    env = dict(os.environ)
    env.pop("CC", None)   # the image's CC/CXX point at a compiler front-end nvcc cannot drive
    env.pop("CXX", None)
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libkdnn_b200.so")
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
