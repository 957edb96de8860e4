"""Builds the CUDA library in-tree with nvcc for sm_100a (cross-compiles without a GPU).

``python -m ccfuser_b200.build`` or ``ccfuser_b200.build.build()``. The result is
``ccfuser_b200/lib/libccfuser_b200.so``; it is rebuilt only when a source is newer than it.
The reference builds a torch CUDAExtension against NVSHMEM and MPI with relocatable device code
(mix_moe/setup.py:108-196); this library has no dependency besides the CUDA runtime.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libccfuser_b200.so")
SOURCES = ["gemm.cu", "gemm2.cu", "moe_kernels.cu", "router.cu", "runtime.cu", "no_alloc.cu", "norm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    return nvcc


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    objs = []
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    tmp = LIB_PATH + ".tmp"
    subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", tmp, *objs, "-lcudart"])
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


def build_selftest() -> str:
    """Build ``lib/ccf_selftest``, the stand-alone C++ check of the library (csrc/selftest.cu: numerics against a CPU
    loop, throughput against cuBLAS). Not part of the default build: it links cuBLAS."""
    build()
    exe = os.path.join(LIB_DIR, "ccf_selftest")
    subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
                           os.path.join(CSRC, "selftest.cu"), "-o", exe, "-L", LIB_DIR, "-lccfuser_b200", "-lcublas",
                           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"])
    return exe


if __name__ == "__main__":
    if "--selftest" in sys.argv:
        print(build_selftest())
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
