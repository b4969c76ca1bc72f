"""In-tree build of ``libdsb200.so`` with nvcc for sm_100a.

``python -m ds_splat_b200.build`` (or ``build()``) compiles every ``csrc/*.cu`` to an object file and
links them into ``ds_splat_b200/libdsb200.so`` next to this file.  Objects are rebuilt only when their
source (or a header) is newer.  ``--use_fast_math`` is deliberate: the integer stages (radii, tile
rectangles, depth keys) must agree bit for bit with the reference, whose pip build uses that flag
(setup.py:8 there), so the same approximate rcp/sqrt/rsqrt/ex2 and FMA contraction are wanted here.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "obj")
LIB_PATH = os.path.join(HERE, "libdsb200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = ["-O3", "--use_fast_math", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC"]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False, extra_flags=()) -> str:
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    os.makedirs(OBJ_DIR, exist_ok=True)
    header_time = _newest(headers)
    jobs = []
    objects = []
    for src in sources:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), header_time):
            jobs.append(["nvcc", *NVCC_FLAGS, *extra_flags, "-I", INCLUDE, "-c", src, "-o", obj])

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0 or (verbose and (res.stdout or res.stderr)):
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < _newest(objects):
        run(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objects, "-o", LIB_PATH])
    return LIB_PATH


if __name__ == "__main__":
    flags = ["-Xptxas", "-v"] if "--ptxas" in sys.argv else []
    print(build(force="--force" in sys.argv, verbose=True, extra_flags=flags))
