"""Compile the CUDA library in-tree: molla_b200/lib/libmolla_sample.so (sm_100a only)."""
from __future__ import annotations

import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SRC = [os.path.join(_HERE, "csrc", "molla_sample.cu"), os.path.join(_HERE, "csrc", "molla_cluster.cu"),
       os.path.join(_HERE, "csrc", "molla_sharded.cu")]
DEPS = SRC + [os.path.join(_HERE, "csrc", "molla_device.cuh"), os.path.join(_HERE, "csrc", "molla_exact.cuh"),
              os.path.join(_HERE, "csrc", "molla_cluster.h"),
              os.path.join(os.path.dirname(_HERE), "include", "molla_sample.h"),
              os.path.join(os.path.dirname(_HERE), "include", "molla_sample_testing.h")]
OUT = os.path.join(_HERE, "lib", "libmolla_sample.so")
# the same sources with -DMOLLA_SAMPLE_TESTING: profiling stamps, experiment switches and the
# exports of include/molla_sample_testing.h, for the tests and for profiling sessions
OUT_TESTING = os.path.join(_HERE, "lib", "libmolla_sample_testing.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # every fp32 operation of the reference is rounded on its own: no implicit fused multiply-add
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared", "-ldl", "-t", "3",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def stale(out: str = OUT) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in DEPS if os.path.exists(d))


def build_library(force: bool = False, verbose: bool = False, testing: bool = False) -> str:
    """Builds libmolla_sample.so (or, with `testing`, libmolla_sample_testing.so) if it is out of date."""
    out = OUT_TESTING if testing else OUT
    if not force and not stale(out):
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = ([nvcc()] + NVCC_FLAGS + (["-DMOLLA_SAMPLE_TESTING"] if testing else [])
           + (["-Xptxas", "-v"] if verbose else []) + ["-o", out] + SRC)
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
    print(build_library(force=True, testing=True))
