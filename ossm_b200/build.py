"""Builds ``libossm_b200.so`` (hand-written CUDA for sm_100a) in-tree with nvcc.

    python -m ossm_b200.build [-v] [--force]

Every ``csrc/*.cu`` is its own translation unit; they are compiled side by side
and linked into one shared library.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ_DIR = os.path.join(PKG, "build")
LIB = os.environ.get("OSSM_B200_LIB") or os.path.join(PKG, "libossm_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _units():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(ROOT, "include", "ossm_b200.h")]


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > built for f in _units() + _headers() if os.path.exists(f))


def _include_dirs():
    """Extra header trees: the CUTLASS / CuTe headers shipped inside Python packages of this image
    (only descriptor bit-field definitions are used from them, by the tensor-core kernels)."""
    dirs = []
    for env in os.environ.get("OSSM_B200_CUTLASS_INCLUDE", "").split(os.pathsep):
        if env:
            dirs.append(env)
    return dirs


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libossm_b200.so")
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = os.environ.get("OSSM_B200_NVCC_FLAGS", "").split()   # extra flags for experiments (e.g. -DNAME)
    incs = [f"-I{d}" for d in _include_dirs()]
    newest_header = max((os.path.getmtime(h) for h in _headers() if os.path.exists(h)), default=0.0)

    def compile_unit(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if (not force and not extra and os.path.exists(obj)
                and os.path.getmtime(obj) > max(os.path.getmtime(src), newest_header)):
            return obj, ""
        cmd = [nvcc, *NVCC_FLAGS, *incs, *extra]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-c", "-o", obj, src]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n" + res.stdout + res.stderr)
        return obj, res.stdout + res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_unit, _units()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    link = [nvcc, "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB]
    link += [obj for obj, _ in results]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc link failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
