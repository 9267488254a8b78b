"""Builds libkq.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python karume_b200/build.py [--verbose] [--force]

Every translation unit is compiled to an object file of its own (in parallel, and only when
it or a header changed), then linked.  The shared library lands next to this file so that it
travels with the source tree; nothing is installed into site-packages and nothing is
JIT-compiled at import time.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
OUT = os.path.join(HERE, "libkq.so")

SOURCES = ["kq_api.cu", "kq_generic.cu", "kq_qgemv_i4.cu", "kq_qgemv_i4_tc.cu", "kq_plan.cu", "kq_qgemm_i4.cu", "kq_qgemm_i4_x32.cu", "kq_qgemv_i8.cu",
           "kq_comm.cu", "kq_idot.cu", "kq_fused_ops.cu", "kq_container.cu"]
HEADERS = ["kq_common.cuh", "kq_gemv_core.cuh", "kq_umma.cuh", "kq_gemm_stream.h", "kq_internal.h", os.path.join("..", "..", "include", "kq.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: libkq has no other build path")
    return found


def _newest_header() -> float:
    deps = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    return max(os.path.getmtime(d) for d in deps)


def _compile_one(args):
    src, obj, verbose, extra_flags = args
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags, "-c", "-o", obj, src]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    if os.path.exists("/usr/bin/g++"):  # the distribution's g++ is the host compiler nvcc is validated with here
        cmd += ["-ccbin", "/usr/bin/g++"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    return src, proc.returncode, proc.stdout + proc.stderr, cmd


def build(force: bool = False, verbose: bool = False, extra_flags=(), out: str = OUT) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = _newest_header()
    jobs, objects = [], []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s.replace(".cu", ".o"))
        objects.append(obj)
        stale = force or extra_flags or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), headers)
        if stale:
            jobs.append((src, obj, verbose, tuple(extra_flags)))
    failed = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        for src, rc, log, cmd in pool.map(_compile_one, jobs):
            if verbose or rc != 0:
                sys.stderr.write(f"---- {os.path.basename(src)}\n{log}")
            if rc != 0:
                failed.append(" ".join(cmd))
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
    if jobs or not os.path.exists(out) or out != OUT:
        cmd = [_nvcc(), "--shared", "-cudart", "shared", "-o", out, *objects]
        if os.path.exists("/usr/bin/g++"):
            cmd += ["-ccbin", "/usr/bin/g++"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError(f"link failed ({proc.returncode}): {' '.join(cmd)}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
