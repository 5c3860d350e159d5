"""Builds libkdnn_b200.so (the CUDA kernels and the C ABI) in-tree with nvcc for
sm_100a. Run as ``python build.py`` from this folder, or call ``build_library()``."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["kdnn_gemv.cu", "kdnn_gemm.cu", "kdnn_moe.cu", "kdnn_dequant.cu", "kdnn_elementwise.cu", "kdnn_capi.cu"]
HEADERS = ["kdnn_common.cuh", "kdnn_tile.cuh", "kdnn_grouped.cuh", "kdnn_mma.cuh", "kdnn_tc.cuh", os.path.join("..", "..", "include", "kdnn_b200.h")]
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
    """Compiles every translation unit in parallel (objects in a temporary folder), then links.
    The library is written next to this file under a temporary name and renamed at the end, so a
    reader never sees a half-written file."""
    if not force and not is_stale():
        return LIB
    import tempfile
    from concurrent.futures import ThreadPoolExecutor
    env = dict(os.environ)
    env.pop("CC", None)   # the image's CC/CXX point at a compiler front-end nvcc cannot drive
    env.pop("CXX", None)
    nvcc = _nvcc()
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + os.environ.get("KDNN_NVCC_EXTRA", "").split()
    with tempfile.TemporaryDirectory(prefix="kdnn_build_") as tmp:
        def compile_one(src: str):
            obj = os.path.join(tmp, src.replace(".cu", ".o"))
            cmd = [nvcc, *flags, *(["-Xptxas", "-v"] if verbose else []), "-c",
                   os.path.join(HERE, "csrc", src), "-o", obj]
            return obj, subprocess.run(cmd, env=env, capture_output=True, text=True)
        with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
            results = list(pool.map(compile_one, SOURCES))
        for _, res in results:
            if verbose or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
        if any(res.returncode != 0 for _, res in results):
            raise RuntimeError("nvcc failed building libkdnn_b200.so")
        tmp_lib = LIB + ".tmp"
        link = subprocess.run([nvcc, "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
                               *[obj for obj, _ in results], "-o", tmp_lib], env=env, capture_output=True, text=True)
        if link.returncode != 0:
            sys.stderr.write(link.stdout + link.stderr)
            raise RuntimeError("nvcc failed linking libkdnn_b200.so")
        os.replace(tmp_lib, LIB)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
