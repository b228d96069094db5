"""Builds libflashMoe.so in-tree with nvcc for sm_100a (no JIT cache, no torch headers).

    python -m flash_distributed_moe_b200.build [--force]

The library holds the CUDA kernels, the C++ host launcher and the C ABI declared in
include/iMoeKernelLauncher.h and include/flashmoe_c.h.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB = os.path.join(_HERE, "libflashMoe.so")
SOURCES = ["moe_kernel.cu", "no_alloc.cu", "launcher.cpp", "bootstrap.cpp"]
HEADERS = ["moe_types.h", "ptx.cuh", "bootstrap.h", "host_layout.h", "lib.version",
           os.path.join("..", "..", "include", "iMoeKernelLauncher.h"),
           os.path.join("..", "..", "include", "flashmoe_c.h")]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
        "-Xlinker", "--version-script=" + os.path.join(CSRC, "lib.version"),
        "-o", LIB,
    ] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
