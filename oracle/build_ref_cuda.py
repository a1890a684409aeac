"""Recipe that compiles the reference's own extension WITH its CUDA kernels into ``oracle/_ref/``.

TEST / MEASUREMENT INFRASTRUCTURE ONLY.  The result (``oracle/_ref/ossm_ref_kernels_cuda.so``) is the
unmodified ossm extension -- ``src/ossm/csrc/*.cpp`` and ``*.cu`` of the reference checkout, bound by
its own ``bindings.cpp``, ``WITH_CUDA`` defined -- built where the sources lie with the flags of the
reference's ``setup.py:47-78`` and ``-gencode arch=compute_100,code=sm_100`` (the reference's generic
kernels, recompiled; nothing of it is copied or shipped).  ``oracle/time_ref_cuda.py`` times these
kernels on the same GPU as a comparison point.  Nothing in the product package may import it.

Usage:  python oracle/build_ref_cuda.py [--reference /path/to/ossm/checkout]
"""
from __future__ import annotations

import argparse
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "ossm_ref_kernels_cuda"


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(" ".join(cmd[:3]) + " ... failed:\n" + res.stderr[-4000:])
    return cmd[-1]


def build(reference: str, verbose: bool = False) -> str:
    csrc = os.path.join(reference, "src", "ossm", "csrc")
    cpp = sorted(glob.glob(os.path.join(csrc, "*.cpp")))
    cu = sorted(glob.glob(os.path.join(csrc, "*.cu")))
    if not cpp or not cu:
        raise FileNotFoundError(f"no reference sources under {csrc}")
    from torch.utils.cpp_extension import include_paths, library_paths

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    build_dir = os.path.join(OUT, "build_cuda")
    os.makedirs(build_dir, exist_ok=True)
    incs = []
    for inc in include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        incs += ["-isystem", inc]
    common = [f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H", "-DWITH_CUDA", "-I" + csrc]
    cxx = os.environ.get("CXX", "g++")
    cxxflags = ["-O3", "-std=c++17", "-march=x86-64-v3", "-ffast-math", "-fno-math-errno", "-fno-trapping-math",
                "-fopenmp", "-fPIC"]
    nvflags = ["-O3", "--use_fast_math", "-lineinfo", "--expt-relaxed-constexpr", "-std=c++17", "-Xcudafe",
               "--diag_suppress=20012", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
               "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__", "-allow-unsupported-compiler",
               "-gencode=arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC"]
    jobs, objs = [], []
    for src in cpp + cu:
        obj = os.path.join(build_dir, os.path.basename(src).replace(".", "_") + ".o")
        objs.append(obj)
        if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
            continue
        if src.endswith(".cu"):
            jobs.append([nvcc, *nvflags, *common, *incs, "-c", src, "-o", obj])
        else:
            jobs.append([cxx, *cxxflags, *common, *incs, "-c", src, "-o", obj])
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        for obj in pool.map(_run, jobs):
            if verbose:
                print("compiled", obj, flush=True)
    dst = os.path.join(OUT, NAME + ".so")
    link = [cxx, *objs, "-shared"]
    for lib in library_paths("cuda"):
        link += ["-L" + lib, "-Wl,-rpath," + lib]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart", "-o", dst]
    for extra in (["-fopenmp"], ["-lgomp"], []):
        res = subprocess.run(link + extra, capture_output=True, text=True)
        if res.returncode == 0:
            break
    else:
        raise RuntimeError("link failed:\n" + res.stderr[-4000:])
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    here = os.path.dirname(HERE)
    ap.add_argument("--reference", default=os.environ.get("OSSM_REFERENCE") or os.path.join(os.path.dirname(here), "reference"),
                    help="ossm checkout (default: $OSSM_REFERENCE, else a directory 'reference' beside this repository)")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args()
    print(build(args.reference, args.verbose))
