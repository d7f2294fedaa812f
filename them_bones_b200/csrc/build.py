"""Builds the native library ``them_bones_b200/lib/libbones_b200.so`` for sm_100a with nvcc.

Each ``.cu`` file is compiled to an object (in parallel, only when it or a header changed) and the objects are linked
into one shared library that ``ops._lib`` loads with ctypes.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(os.path.dirname(HERE), "lib")
LIB = os.path.join(LIB_DIR, "libbones_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _newer(a, b):
    return not os.path.exists(b) or os.path.getmtime(a) > os.path.getmtime(b)


LIB_DEBUG = os.path.join(LIB_DIR, "libbones_b200_dbg.so")
LIB_MEASURE = os.path.join(LIB_DIR, "libbones_b200_prof.so")
MEASURE_DEFINES = ("BONES_MX_PROF", "BONES_ATTN_PROF")


def build(verbose: bool = False, force: bool = False, debug_bounds: bool = False, measure: bool = False) -> str:
    """``debug_bounds``: the second library, compiled with ``-DBONES_DEBUG_BOUNDS`` (every data-dependent index is checked,
    a miss is counted and skipped; see ``csrc/common.cuh``), loaded instead of the release one when
    ``BONES_DEBUG_BOUNDS=1``.  ``measure``: a third library whose tensor-core kernels account the clocks each of their
    roles spends waiting and issuing (``-DBONES_MX_PROF -DBONES_ATTN_PROF``); ``ops.microbench mxroles / attnroles``
    read it when ``BONES_LIB`` points at it.  Neither is needed to train."""
    os.makedirs(LIB_DIR, exist_ok=True)
    objdir = os.path.join(LIB_DIR, "obj_prof" if measure else "obj_dbg" if debug_bounds else "obj")
    lib = LIB_MEASURE if measure else LIB_DEBUG if debug_bounds else LIB
    flags = FLAGS + (["-DBONES_DEBUG_BOUNDS"] if debug_bounds else []) + ([f"-D{d}" for d in MEASURE_DEFINES] if measure else [])
    os.makedirs(objdir, exist_ok=True)
    srcs = sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))
    hdrs = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    jobs = []
    for s in srcs:
        src, obj = os.path.join(HERE, s), os.path.join(objdir, s[:-3] + ".o")
        if force or _newer(src, obj) or any(_newer(h, obj) for h in hdrs):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        r = subprocess.run([NVCC, *flags, "-c", src, "-o", obj], capture_output=True, text=True)
        return src, r

    failed = False
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(compile_one, jobs):
            log = (r.stdout + r.stderr)
            with open(os.path.join(objdir, os.path.basename(src) + ".log"), "w") as fh:
                fh.write(log)
            if r.returncode != 0:
                failed = True
                sys.stderr.write(log)
            elif verbose:
                sys.stderr.write(log)
    if failed:
        raise RuntimeError("nvcc failed")
    objs = [os.path.join(objdir, s[:-3] + ".o") for s in srcs]
    if jobs or not os.path.exists(lib):
        r = subprocess.run([NVCC, "-shared", "-o", lib, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, debug_bounds=True))
    if "--measure" in sys.argv:
        print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, measure=True))
