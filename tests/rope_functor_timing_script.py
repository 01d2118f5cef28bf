"""Times an fp32 RoPE functor header through sideaware_create_kernel + sideaware_elementwise of the
library given by path (this project's or the compiled reference: the header contract is the same),
at the shape of the reference's own example (B=8 T=1024 32+32+32 heads HS=128, example_llmc_rope.cu:246-249),
in place on a block from the library's allocator.  Checks the result against the oracle.  One JSON line.

    python rope_functor_timing_script.py <library> [include]

With "include" the header registered is the literal text the reference's example registers,
#include "kernel_rope.cuh" (example_llmc_rope.cu:135-144): NVRTC resolves it against the working
directory, so the caller runs this script from the directory that holds the reference's header."""
import ctypes
import json
import os
import statistics
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from l2_torch_alloc_b200 import functors  # noqa: E402  (header text only; no library code involved)
from oracle import oracle  # noqa: E402


def main():
    path = sys.argv[1]
    B, T, NH, HS = 8, 1024, 32, 128
    lib = ctypes.CDLL(path)
    lib.sideaware_malloc_async.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t, ctypes.c_void_p]
    lib.sideaware_create_kernel.argtypes = [ctypes.c_char_p]
    lib.sideaware_create_kernel.restype = ctypes.c_int
    lib.sideaware_memcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    lib.sideaware_memcpy.restype = None
    lib.sideaware_elementwise.argtypes = [ctypes.c_int, ctypes.c_size_t] + [ctypes.c_void_p] * 9 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
    lib.sideaware_elementwise.restype = None
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    sp = torch.cuda.current_stream().cuda_stream
    n = B * T * 3 * NH * HS
    x = np.random.default_rng(0xB200 + 1).uniform(-1, 1, size=(B, T, 3 * NH, HS)).astype(np.float32)
    table = oracle.freqs_cis(HS, T, 10000.0, 1)
    want = oracle.rope_forward_f32(x, table, B, T, NH, NH, HS)
    tx = torch.from_numpy(x).cuda()
    tt = torch.from_numpy(table).cuda()
    buf = ctypes.c_void_p()
    assert lib.sideaware_malloc_async(ctypes.byref(buf), 4 * n, sp) == 0
    literal_include = len(sys.argv) > 2 and sys.argv[2] == "include"
    header = b'#include "kernel_rope.cuh"' if literal_include else functors.rope_forward(T, NH, NH, HS, False).encode()
    kid = lib.sideaware_create_kernel(header)
    assert kid >= 1

    def run():
        lib.sideaware_elementwise(kid, 4 * n, buf, None, None, None, buf, tt.data_ptr(), None, None, None, 0, 0, 0, 0, sp)

    lib.sideaware_memcpy(buf, tx.data_ptr(), 4 * n, 0, sp)
    run()
    out = torch.empty_like(tx)
    lib.sideaware_memcpy(out.data_ptr(), buf, 4 * n, 0, sp)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    exact = got.tobytes() == want.tobytes()
    close = bool(np.allclose(got, want, rtol=1e-6, atol=1e-6))
    # the reference's own criterion (validate_result, example_llmc_common.h:312-351, called with 1e-5)
    ref_tol = bool((np.abs(got - want) <= 1e-5 + np.abs(want) * np.finfo(np.float32).eps).all())
    for _ in range(5):
        run()
    torch.cuda.synchronize()
    reps = 50
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    ev[0].record()
    for i in range(reps):
        run()
        ev[i + 1].record()
    torch.cuda.synchronize()
    ms = statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))
    moved = 2 * B * T * 2 * NH * HS * 4 + table.nbytes  # q and k read and written, table once
    res = {"lib": path, "ms": ms, "gbs": moved / ms / 1e6, "bit_exact": exact, "within_1e-6": close,
           "within_reference_tolerance": ref_tol, "header": "literal include" if literal_include else "generated"}
    if hasattr(lib, "sideaware_rope_forward"):  # this project's ahead-of-time kernel on the same shape
        lib.sideaware_rope_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 7 + [ctypes.c_void_p]
        aot = lambda: lib.sideaware_rope_forward(buf, tt.data_ptr(), B, T, NH, NH, HS, 0, 0, sp)  # noqa: E731
        for _ in range(5):
            aot()
        torch.cuda.synchronize()
        ev[0].record()
        for i in range(reps):
            aot()
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms2 = statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))
        res["aot_ms"] = ms2
        res["aot_gbs"] = moved / ms2 / 1e6
    print("RESULT " + json.dumps(res))


if __name__ == "__main__":
    main()
