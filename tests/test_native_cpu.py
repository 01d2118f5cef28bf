"""Builds and runs the C++ tests of the library's host logic (tests/cpp/test_core.cpp):
scheduler coverage, allocator state machine on a simulated driver with fault
injection, topology analysis on synthetic latencies, stage bookkeeping of the bulk-copy kernels when loads never arrive.  No GPU involved."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "_bin", "test_core")
CSRC = os.path.join(ROOT, "l2_torch_alloc_b200", "csrc")


@pytest.fixture(scope="module")
def core_binary():
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    srcs = [os.path.join(ROOT, "tests", "cpp", "test_core.cpp"), os.path.join(CSRC, "sa_alloc.cpp"),
            os.path.join(CSRC, "sa_topology.cpp")]
    deps = srcs + [os.path.join(CSRC, f) for f in ("sa_alloc.hpp", "sa_probe.hpp", "sa_sched.cuh", "sa_bulk.cuh")]
    if not os.path.exists(BIN) or any(os.path.getmtime(d) > os.path.getmtime(BIN) for d in deps):
        subprocess.check_call(["g++", "-O1", "-std=c++17", "-I/usr/local/cuda/include", *srcs, "-o", BIN, "-lpthread"])
    return BIN


@pytest.mark.parametrize("suite", ["sched", "alloc", "chunks", "topology", "ring"])
def test_core_suite(core_binary, suite):
    r = subprocess.run([core_binary, suite], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "OK" in r.stdout
