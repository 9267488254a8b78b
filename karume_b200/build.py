"""Builds libkq.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python karume_b200/build.py [--verbose] [--force]

The shared library lands next to this file so that it travels with the source tree;
nothing is installed into site-packages and nothing is JIT-compiled at import time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libkq.so")

SOURCES = ["kq_api.cu", "kq_generic.cu", "kq_qgemv_i4.cu", "kq_plan.cu", "kq_qgemm_i4.cu", "kq_qgemv_i8.cu", "kq_comm.cu", "kq_idot.cu"]
HEADERS = ["kq_common.cuh", "kq_gemv_core.cuh", "kq_internal.h", os.path.join("..", "..", "include", "kq.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "shared",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: libkq has no other build path")
    return found


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=(), out: str = OUT) -> str:
    if not force and out == OUT and not _stale():
        return out
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", out] + [os.path.join(CSRC, s) for s in SOURCES]
    env = dict(os.environ)
    # the distribution's g++ is the host compiler nvcc is validated with here
    if os.path.exists("/usr/bin/g++"):
        cmd += ["-ccbin", "/usr/bin/g++"]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
