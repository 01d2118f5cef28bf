"""This library's memcpy next to the REFERENCE's own GPU path on the same B200: the reference
sideaware.cu compiled in place into oracle/_ref/sideaware_reference.so (its allocator, its
NVRTC-JIT-ed kernel for sm_100), timed by the same script in separate processes.
Skipped where the compiled reference is not present."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "sideaware_reference.so")
OURS = os.path.join(ROOT, "l2_torch_alloc_b200", "sideaware.so")


def run(lib, sizes):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "memcpy_timing_script.py"), lib, sizes],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert lines, r.stdout[-2000:] + r.stderr[-2000:]
    return json.loads(lines[-1][7:])


@pytest.mark.skipif(not os.path.exists(REF), reason="compiled reference not present")
def test_memcpy_faster_than_the_reference_kernel():
    sizes = f"{64 << 20},{1 << 30}"
    ref = run(REF, sizes)
    ours = run(OURS, sizes)
    print("reference:", json.dumps(ref))
    print("ours:     ", json.dumps(ours))
    assert ref["summary"][0] == ours["summary"][0]
    for n in ref["sizes"]:
        assert ref["sizes"][n]["exact"] and ours["sizes"][n]["exact"]
    one_gib = str(1 << 30)
    assert ours["sizes"][one_gib]["gbs"] > ref["sizes"][one_gib]["gbs"], "the bar is beating the reference's kernel on the same box"


@pytest.mark.skipif(not os.path.exists(REF), reason="compiled reference not present")
def test_rope_example_shape_level_with_the_reference_template():
    """The same fp32 RoPE functor header through both libraries' NVRTC paths (the reference's kernel
    template vs this library's), at the reference example's shape, each checked against the oracle."""
    out = {}
    for name, lib in (("reference", REF), ("ours", OURS)):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "rope_functor_timing_script.py"), lib],
                           capture_output=True, text=True, timeout=600, cwd=ROOT)
        lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
        assert lines, r.stdout[-2000:] + r.stderr[-2000:]
        out[name] = json.loads(lines[-1][7:])
        print(name, json.dumps(out[name]))
    assert out["ours"]["bit_exact"], "this library's functor path must reproduce the oracle bit for bit"
    assert out["reference"]["within_1e-6"], "the reference's fast-math JIT stays within its own tolerance"
    # At this small shape (100 MB, a 90 us kernel) the two libraries lie within a few percent of each other, by GPU:
    # the reference's static assignment uses 2 x min(SMs per side) SMs, all 148 on a GPU split 74/74 (6 100 GB/s
    # measured) but 140 on one split 70/78 (5 050-5 840), while this library's kernels give 5 900-5 970 on every box.
    # So this comparison guards against a regression; the strict one is at the benchmark shape (next test).
    assert out["ours"]["aot_gbs"] >= 0.95 * out["reference"]["gbs"]
    assert out["ours"]["gbs"] >= 0.93 * out["reference"]["gbs"]


@pytest.mark.skipif(not os.path.exists(REF), reason="compiled reference not present")
def test_rope_faster_than_the_reference_at_the_benchmark_shape():
    """bf16 RoPE at the Llama-3-8B shape of the benchmark: the reference's kernel template (given a header generated for
    that shape; its own kernel_rope.cuh hard-codes another one) against this library's RoPE kernel and this library's
    template with the same header, per launch, each checked against the oracle.  The bar is beating the reference."""
    out = {}
    for name, lib in (("reference", REF), ("ours", OURS)):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "rope_llama_timing_script.py"), lib],
                           capture_output=True, text=True, timeout=900, cwd=ROOT)
        lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
        assert lines, r.stdout[-2000:] + r.stderr[-2000:]
        out[name] = json.loads(lines[-1][7:])
        print(name, json.dumps(out[name]))
    assert out["ours"]["max_bf16_ulp_vs_oracle"] == 0 and out["reference"]["max_bf16_ulp_vs_oracle"] <= 1
    assert out["ours"]["aot_gbs"] > out["reference"]["functor_gbs"]
    assert out["ours"]["functor_gbs"] > out["reference"]["functor_gbs"]


def launch_rates(lib):
    """Builds tests/cpp/launch_rate.cpp once and runs it on `lib`: {KiB: (issue us per call, us per call in all)}."""
    binary = os.path.join(ROOT, "tests", "cpp", "_bin", "launch_rate")
    src = os.path.join(ROOT, "tests", "cpp", "launch_rate.cpp")
    if not os.path.exists(binary) or os.path.getmtime(src) > os.path.getmtime(binary):
        os.makedirs(os.path.dirname(binary), exist_ok=True)
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-I/usr/local/cuda/include", src, "-o", binary,
                               "-L/usr/local/cuda/lib64", "-lcudart", "-ldl", "-Wl,-rpath,/usr/local/cuda/lib64"])
    r = subprocess.run([binary, lib], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = {}
    for line in r.stdout.splitlines():
        if line.startswith("RATE "):
            _, kib, issue, total = line.split()
            out[int(kib)] = (float(issue), float(total))
    assert out, r.stdout[-2000:]
    return out


@pytest.mark.skipif(not os.path.exists(REF), reason="compiled reference not present")
def test_short_copies_follow_one_another_no_slower_than_with_the_reference_library():
    """20 000 copies of 64 KiB .. 16 MiB issued by a C++ loop on one stream: what one call costs when nothing else
    limits it (measured: 3.4 us here, 3.9-4.1 us for the reference's library up to 4 MiB; 5.3 against 5.8 us at 16 MiB).
    Bound loosely: shared hosts vary."""
    ours, ref = launch_rates(OURS), launch_rates(REF)
    print("ours:     ", ours)
    print("reference:", ref)
    for kib in ours:
        assert ours[kib][1] <= 1.25 * ref[kib][1], (kib, ours[kib], ref[kib])
