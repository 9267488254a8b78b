"""The streamed prefill GEMM deals (pair tile, k-step) units to the SM pairs with a few lines of
integer arithmetic shared by the kernel and its launcher (karume_b200/csrc/kq_gemm_stream.h).
This compiles a host program around that header and checks the partition's invariants over a
grid of tile counts, k-step counts and pair counts: every unit exactly once, one owner per
tile, the owner's partner count equal to the number of later holders, pieces always a pair's
first fragment, and the streaming rule on the shapes it was measured on."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_partition_invariants_hold(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host C++ compiler")
    exe = tmp_path / "gemm_stream_check"
    subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "karume_b200", "csrc"),
                    os.path.join(ROOT, "tests", "native", "gemm_stream_check.cpp"), "-o", str(exe)], check=True)
    done = subprocess.run([str(exe)], capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
    assert done.stdout.startswith("ok "), done.stdout
