"""Builds the native library in-tree with nvcc for sm_100a only.

``python -m deeplearning4j_b200.csrc.build`` compiles every ``.cu`` in this directory into
``libdl4j_b200.so`` next to the sources.  Object files are cached by source mtime so that a
rebuild after touching one kernel takes seconds.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libdl4j_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


DEBUG_LIB = os.path.join(HERE, "libdl4j_b200_dbg.so")
ASAN_LIB = os.path.join(HERE, "libdl4j_b200_asan.so")


def build(verbose: bool = False, force: bool = False, debug_bounds: bool = False, asan: bool = False) -> str:
    """Default: the optimised library.  ``debug_bounds``: a second library with ``-DDL4J_DEBUG_BOUNDS`` (kernels check the element
    offsets they wrap in ``DL4J_IN_BOUNDS``, record the first violation and skip the access; relocatable device code so that
    every translation unit shares one record).  ``asan``: a third library whose *host* code is instrumented with
    AddressSanitizer + UndefinedBehaviorSanitizer; load it in a process started with ``LD_PRELOAD=$(gcc -print-file-name=libasan.so)``."""
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    global_flags = list(FLAGS)
    lib, objname = LIB, "build"
    if debug_bounds:
        global_flags += ["-DDL4J_DEBUG_BOUNDS", "-rdc=true"]
        lib, objname = DEBUG_LIB, "build_dbg"
    elif asan:
        global_flags = [f for f in global_flags if f != "-O3"] + ["-O1", "-Xcompiler", "-fsanitize=address", "-Xcompiler", "-fsanitize=undefined",
                                                                   "-Xcompiler", "-fno-omit-frame-pointer"]
        lib, objname = ASAN_LIB, "build_asan"
    objdir = os.path.join(HERE, objname)
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for s in sources():
        src = os.path.join(HERE, s)
        obj = os.path.join(objdir, s[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC] + ARCH + global_flags + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, r in ex.map(compile_one, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(f"--- {os.path.basename(src)}\n{r.stdout}{r.stderr}\n")
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed for {src}")
    objs = [os.path.join(objdir, s[:-3] + ".o") for s in sources()]
    if force or jobs or _stale(lib, objs):
        cmd = [NVCC] + ARCH + ["-shared", "-o", lib] + objs + ["-lcudart_static", "-ldl", "-lrt", "-lpthread"]
        if asan:
            cmd += ["-Xcompiler", "-fsanitize=address", "-Xcompiler", "-fsanitize=undefined"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, debug_bounds="--debug-bounds" in sys.argv, asan="--asan" in sys.argv))
