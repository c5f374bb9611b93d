"""Builds ``libphiltorch_b200.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python philtorch_b200/build.py [-v]      (by path: works even when the built library is stale)

The library has no torch dependency; it links the CUDA runtime only.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libphiltorch_b200.so")
ROOT_INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-cudart", "shared", "--threads", "0",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps() -> list[str]:
    return (sources() + glob.glob(os.path.join(CSRC, "*.cuh"))
            + glob.glob(os.path.join(ROOT_INCLUDE, "*.h")))


def up_to_date() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(s) <= t for s in _deps())


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + sources() + ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libphiltorch_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force=True))
