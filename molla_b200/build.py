"""Compile the CUDA library in-tree: molla_b200/lib/libmolla_sample.so (sm_100a only)."""
from __future__ import annotations

import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SRC = [os.path.join(_HERE, "csrc", "molla_sample.cu"), os.path.join(_HERE, "csrc", "molla_cluster.cu")]
DEPS = SRC + [os.path.join(_HERE, "csrc", "molla_device.cuh"), os.path.join(_HERE, "csrc", "molla_exact.cuh"),
              os.path.join(_HERE, "csrc", "molla_cluster.h"),
              os.path.join(os.path.dirname(_HERE), "include", "molla_sample.h")]
OUT = os.path.join(_HERE, "lib", "libmolla_sample.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # every fp32 operation of the reference is rounded on its own: no implicit fused multiply-add
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared", "-t", "2",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(d) > t for d in DEPS if os.path.exists(d))


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT] + SRC
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
