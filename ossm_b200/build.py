"""Builds ``libossm_b200.so`` (hand-written CUDA for sm_100a) in-tree with nvcc.

    python -m ossm_b200.build [-v] [--force]
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.environ.get("OSSM_B200_LIB") or os.path.join(PKG, "libossm_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _sources():
    files = glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    files.append(os.path.join(ROOT, "include", "ossm_b200.h"))
    return files


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > built for f in _sources() if os.path.exists(f))


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libossm_b200.so")
    cmd = [nvcc, *NVCC_FLAGS]
    cmd += os.environ.get("OSSM_B200_NVCC_FLAGS", "").split()   # extra flags for experiments (e.g. -DNAME)
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB, os.path.join(CSRC, "ossm_b200_all.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
