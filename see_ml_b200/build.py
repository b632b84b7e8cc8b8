"""Builds see_ml_b200/libseeml_b200.so in-tree: CUDA kernels for sm_100a (nvcc) and
the C++ host side (g++ -std=c++23), linked into one shared library with a C ABI.

    python -m see_ml_b200.build [--force]

nvcc cross-compiles without a GPU. The library links cudart statically and resolves
the driver entry points it needs at run time, so it loads (and reports "no CUDA
device") on a machine without a GPU driver.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libseeml_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA, "bin", "nvcc")
GXX = "g++"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++20", "-lineinfo", "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC,
              "--expt-relaxed-constexpr", "-ccbin", GXX] + ARCH
# Per-file extras: the memory-bound kernels keep separate multiply/add roundings so that
# their expressions match the scalar CPU runtime bit for bit.
EXTRA = {"kernels_mem.cu": ["-fmad=false"]}
GXX_FLAGS = ["-O2", "-std=c++23", "-fPIC", "-pthread", "-I" + INCLUDE, "-I" + CSRC,
             "-I" + os.path.join(CUDA, "include"), "-Wall", "-Wextra", "-Wno-unused-parameter"]

CU_SRCS = ["kernels_mem.cu", "kernels_gemm_simt.cu", "kernels_skinny.cu", "gemm_tc.cu", "backend.cu", "xent_noalloc.cu"]
CC_SRCS = ["validate.cc", "dataset.cc", "engine.cc", "comm.cc"]


def _stale(src, obj, deps):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in [src] + deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inc"))]
    headers.append(os.path.join(INCLUDE, "seeml_b200.h"))
    jobs = []
    objs = []
    for s in CU_SRCS:
        src, obj = os.path.join(CSRC, s), os.path.join(OBJ, s + ".o")
        objs.append(obj)
        if force or _stale(src, obj, headers):
            jobs.append([NVCC] + NVCC_FLAGS + EXTRA.get(s, []) + ["-c", src, "-o", obj])
    for s in CC_SRCS:
        src, obj = os.path.join(CSRC, s), os.path.join(OBJ, s + ".o")
        objs.append(obj)
        if force or _stale(src, obj, headers):
            jobs.append([GXX] + GXX_FLAGS + ["-c", src, "-o", obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("build failed: " + " ".join(cmd[:1] + cmd[-3:]))
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([GXX, "-shared", "-pthread", "-o", LIB] + objs +
            ["-L" + os.path.join(CUDA, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lstdc++", "-lm"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
