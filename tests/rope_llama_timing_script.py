"""The benchmark's RoPE shape (bf16, B=8 T=8192, 32 query + 8 key + 8 value heads, HS=128, theta 500000, in place) through
sideaware_create_kernel + sideaware_elementwise of the library given by path: this project's, or the compiled
reference, whose kernel template takes the same generated header (the header contract is the same).  The first
batch entry is checked against the oracle.  Where the library has the ahead-of-time kernel (sideaware_rope_forward),
that is timed on the same tensor as well.  One JSON line.

    python rope_llama_timing_script.py <library>
"""
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


def timed(run, reps=30):
    for _ in range(5):
        run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    ev[0].record()
    for i in range(reps):
        run()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))


def main():
    path = sys.argv[1]
    B, T, Nq, Nkv, HS = 8, 8192, 32, 8, 128
    H = Nq + 2 * Nkv
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
    n = B * T * H * HS
    one = oracle.f32_to_bf16(np.random.default_rng(0xB200 + 3).standard_normal(size=(1, T, H, HS)).astype(np.float32))
    table = oracle.freqs_cis(HS, T, 500000.0, 0)
    want = oracle.rope_forward_bf16(one, table, 1, T, Nq, Nkv, HS, threads=os.cpu_count() or 1)
    tx = torch.from_numpy(one.view(np.int16)).cuda().repeat(B, 1, 1, 1).contiguous()  # every batch entry the same input
    tt = torch.from_numpy(table).cuda()
    buf = ctypes.c_void_p()
    assert lib.sideaware_malloc_async(ctypes.byref(buf), 2 * n, sp) == 0
    kid = lib.sideaware_create_kernel(functors.rope_forward(T, Nq, Nkv, HS, True).encode())
    assert kid >= 1

    def functor():
        # three 256-thread groups per block: the generated bf16 header bounds its blocks at 768 threads (the reference
        # launches as many groups as it is told to, sideaware.cu:1407; this library clamps to the header's bound by itself)
        lib.sideaware_elementwise(kid, 2 * n, buf, None, None, None, buf, tt.data_ptr(), None, None, None, 0, 3, 0, 0, sp)

    lib.sideaware_memcpy(buf, tx.data_ptr(), 2 * n, 0, sp)
    functor()
    out = torch.empty_like(tx)
    lib.sideaware_memcpy(out.data_ptr(), buf, 2 * n, 0, sp)
    torch.cuda.synchronize()
    got = out[B - 1:].cpu().numpy().view(np.uint16)
    ulps = int(oracle.ulp_diff_bf16(got, want).max())
    moved = 2 * B * T * (Nq + Nkv) * HS * 2 + table.nbytes  # q and k read and written, table once
    ms = timed(functor)
    res = {"lib": path, "functor_ms": ms, "functor_gbs": moved / ms / 1e6, "max_bf16_ulp_vs_oracle": ulps}
    if hasattr(lib, "sideaware_rope_forward"):
        lib.sideaware_rope_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 7 + [ctypes.c_void_p]
        ms2 = timed(lambda: lib.sideaware_rope_forward(buf, tt.data_ptr(), B, T, Nq, Nkv, HS, 1, 0, sp))
        res["aot_ms"] = ms2
        res["aot_gbs"] = moved / ms2 / 1e6
    print("RESULT " + json.dumps(res))


if __name__ == "__main__":
    main()
