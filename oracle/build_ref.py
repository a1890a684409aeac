"""Recipe that compiles the reference's own CPU kernels into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  The result (``oracle/_ref/ossm_ref_kernels.so``) is
the unmodified ossm CPU extension (``src/ossm/csrc/*.cpp`` of the reference
checkout, bound by its own ``bindings.cpp``) built where the sources lie; no
reference source is copied.  It is used (a) to validate the restatements in
``oracle/`` and (b) as the timed CPU baseline of ``bench.py``.  Nothing in the
product package may import it.

Flags follow the reference's ``setup.py:47-55`` except that ``-march=native``
becomes ``-march=x86-64-v3`` (the object must also run on a different host CPU
than the one that compiled it) and ``-fopenmp`` is kept for compilation but
dropped at link time when the toolchain cannot link libgomp.

``stage_package`` additionally places a copy of the reference's Python package (``src/ossm``,
Python files only) under the git-ignored ``oracle/_ref/pkg/`` next to the compiled kernels.  It
is what the drop-in tests import on a machine that has no ossm checkout (the GPU box): they put
this library behind the unmodified ossm layers and compare results.  It is never committed and
nothing in the product package reads it.

Usage:  python oracle/build_ref.py [--reference /path/to/ossm/checkout]
"""
from __future__ import annotations

import argparse
import glob
import os
import concurrent.futures
import shutil
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "ossm_ref_kernels"


def _compile_one(args):
    cmd, obj = args
    subprocess.run(cmd, check=True)
    return obj


def build(reference: str, verbose: bool = False) -> str:
    csrc = os.path.join(reference, "src", "ossm", "csrc")
    sources = sorted(glob.glob(os.path.join(csrc, "*.cpp")))
    if not sources:
        raise FileNotFoundError(f"no reference sources under {csrc}")
    from torch.utils.cpp_extension import include_paths, library_paths

    build_dir = os.path.join(OUT, "build")
    os.makedirs(build_dir, exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    cflags = ["-O3", "-std=c++17", "-march=x86-64-v3", "-ffast-math",
              "-fno-math-errno", "-fno-trapping-math", "-fopenmp", "-fPIC",
              f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-I" + csrc]
    for inc in include_paths() + [sysconfig.get_paths()["include"]]:
        cflags += ["-isystem", inc]
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(build_dir, os.path.basename(src)[:-4] + ".o")
        objs.append(obj)
        if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
            continue
        jobs.append(([cxx, *cflags, "-c", src, "-o", obj], obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        for obj in pool.map(_compile_one, jobs):
            if verbose:
                print("compiled", obj)
    dst = os.path.join(OUT, NAME + ".so")
    link = [cxx, *objs, "-shared"]
    for lib in library_paths():
        link += ["-L" + lib, "-Wl,-rpath," + lib]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-o", dst]
    # ``-fopenmp`` at link time needs libgomp.spec, which some toolchain
    # wrappers cannot find; libgomp is then taken from the already loaded torch.
    for extra in (["-fopenmp"], ["-lgomp"], []):
        res = subprocess.run(link + extra, capture_output=True, text=True)
        if res.returncode == 0:
            break
    else:
        raise RuntimeError("link failed:\n" + res.stderr)
    return dst


def stage_package(reference: str) -> str:
    """Copies ``<reference>/src/ossm`` (``*.py`` only) to ``oracle/_ref/pkg/ossm``."""
    src = os.path.join(reference, "src", "ossm")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"no ossm package under {src}")
    dst_root = os.path.join(OUT, "pkg")
    dst = os.path.join(dst_root, "ossm")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=lambda d, names: [n for n in names
                                                      if not (n.endswith(".py") or os.path.isdir(os.path.join(d, n)))
                                                      or n in ("csrc", "__pycache__")])
    return dst_root


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--reference", default=os.environ.get("OSSM_REFERENCE") or os.path.join(os.path.dirname(here), "reference"),
                    help="ossm checkout (default: $OSSM_REFERENCE, else a directory 'reference' beside this repository)")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args()
    print(build(args.reference, args.verbose))
    print(stage_package(args.reference))
