"""The C++ host layer (fastnn_b200/host/fastnn_host.hpp): buffer cache, context, tensor-level
matmul dispatch and Linear -- the part of FastNN that is Rust in the reference.

* CPU: compiled against a fake device (host memory, plain-loop GEMM) and run here.
* GPU: compiled against libfastnn_b200.so and the C oracle, run on the B200.
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "host_cpp", "_bin")


def _compile(src, out, extra):
    os.makedirs(BIN, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-o", out, src] + extra
    subprocess.check_call(cmd)
    return out


def test_host_layer_on_fake_device():
    exe = _compile(os.path.join(ROOT, "tests", "host_cpp", "test_host_fake.cpp"),
                   os.path.join(BIN, "test_host_fake"), [])
    res = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    sys.stdout.write(res.stdout)
    assert res.returncode == 0, res.stdout + res.stderr


def test_host_layer_links_against_the_library(built_library):
    """Link check on CPU: every C-ABI symbol the header-only layer references resolves."""
    libdir = os.path.dirname(built_library)
    _compile(os.path.join(ROOT, "tests", "host_cpp", "test_host_gpu.cpp"),
             os.path.join(BIN, "test_host_gpu"),
             ["-x", "c", os.path.join(ROOT, "oracle", "fastnn_cpu_oracle.c"), "-x", "none",
              "-ffp-contract=off", "-L", libdir, "-lfastnn_b200", f"-Wl,-rpath,{libdir}", "-lm", "-pthread"])


@pytest.mark.gpu
def test_host_layer_on_gpu(gpu, built_library):
    exe = os.path.join(BIN, "test_host_gpu")
    if not os.path.exists(exe):
        test_host_layer_links_against_the_library(built_library)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    sys.stdout.write(res.stdout)
    assert res.returncode == 0, res.stdout + res.stderr
