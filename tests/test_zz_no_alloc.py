"""sideaware_memcpy_noalloc: the copy for callers that cannot allocate device memory
(a server whose pool already owns all of HBM, code inside another allocator's callback,
an error path after an out-of-memory condition).  It keeps its work counters in a fixed
array inside the library instead of an allocated buffer.

Checked here, through the C ABI, on two calls in a row: the bytes it produces are identical
to what the ordinary sideaware_memcpy produces, it refuses oversized requests with a clear
error, and its second call leaves the amount of free device memory unchanged.

The file is named to be collected last.  It passes on its own in a fresh process (the
device has then not been set up by any allocating call, so the copy runs side-unaware)
and after the other tests (the side table exists, so the copy runs side-aware)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_BYTES = 1 << 36


@pytest.fixture(scope="module")
def sa():
    import torch
    assert torch.cuda.is_available()
    import l2_torch_alloc_b200 as pkg
    return pkg.SideAware()


def test_noalloc_copy_matches_ordinary_copy_twice_in_a_row(sa):
    import torch
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    sizes = [(96 << 20) + 4096 + 48, 1 << 20]  # a large ragged copy, then a small one
    gen = torch.Generator(device="cuda").manual_seed(0xB200 + 9)
    srcs = [torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=gen) for n in sizes]
    outs = [torch.zeros(n + 64, dtype=torch.uint8, device="cuda") for n in sizes]  # 64 spare bytes catch overruns
    refs = [torch.zeros(n + 64, dtype=torch.uint8, device="cuda") for n in sizes]
    torch.cuda.synchronize()

    # two calls back to back on one stream, before anything else in this test touches the library
    for src, out, n in zip(srcs, outs, sizes):
        rc = sa.lib.sideaware_memcpy_noalloc(out.data_ptr(), src.data_ptr(), n, 0, stream)
        assert rc == 0, sa.last_error()
    torch.cuda.synchronize()

    # the existing entry point on the same inputs
    for src, ref, n in zip(srcs, refs, sizes):
        sa.memcpy_ptr(ref.data_ptr(), src.data_ptr(), n, 0, stream)
    torch.cuda.synchronize()
    for src, out, ref, n in zip(srcs, outs, refs, sizes):
        assert torch.equal(out, ref), "noalloc copy differs from sideaware_memcpy"
        assert torch.equal(out[:n], src) and not out[n:].any()

    # now the device is set up (the ordinary call did that): repeat, twice, on the side-aware path,
    # and check that the calls themselves take no device memory
    for out in outs:
        out.zero_()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        for src, out, n in zip(srcs, outs, sizes):
            assert sa.lib.sideaware_memcpy_noalloc(out.data_ptr(), src.data_ptr(), n, 0, stream) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the allocation-free entry point changed the free device memory"
    for out, ref in zip(outs, refs):
        assert torch.equal(out, ref)


def test_noalloc_rejects_what_it_cannot_do(sa):
    import torch
    t = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    before = sa.error_count()
    assert sa.lib.sideaware_memcpy_noalloc(t.data_ptr(), t.data_ptr(), MAX_BYTES + 16, 0, None) == 1
    assert "more than this entry point accepts" in sa.last_error()
    assert sa.lib.sideaware_memcpy_noalloc(t.data_ptr(), t.data_ptr(), 100, 0, None) == 1
    assert sa.lib.sideaware_memcpy_noalloc(t.data_ptr() + 8, t.data_ptr(), 64, 0, None) == 1
    assert sa.lib.sideaware_memcpy_noalloc(None, t.data_ptr(), 64, 0, None) == 1
    assert sa.error_count() == before + 4
    assert sa.lib.sideaware_memcpy_noalloc(t.data_ptr(), t.data_ptr(), 0, 0, None) == 0  # empty copy: nothing to do
    torch.cuda.synchronize()
    assert not t.any()


def test_noalloc_as_the_first_call_of_a_process():
    """In this test run the device has long been set up by earlier tests, so the branch the entry point exists
    for (nothing allocated yet: symbol address looked up, no side table, side-unaware copy) is run in a
    process of its own, where the allocation-free copy is the library's very first call."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    so = os.path.join(root, "l2_torch_alloc_b200", "sideaware.so")
    r = subprocess.run([sys.executable, os.path.join(root, "tests", "noalloc_first_call_script.py"), so],
                       capture_output=True, text=True, timeout=600, cwd=root)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads(lines[-1][7:])
    assert res["rcs"] == [0, 0] and res["equal"] == [True, True] and res["errors"] == 0, res
    assert res["free_after_second"] == res["free_between"], "a call took device memory"
    print("free device memory before the first call minus after it:", res["free_before_first"] - res["free_between"])
