"""Drives the reference's own example_wrapper.py (staged unmodified under oracle/_ref by oracle/Makefile)
against this project's sideaware.so, in a process of its own: sideaware_init installs the pluggable
allocator and registers torch.ops.sideaware.*, then the three ops run on tensors that torch allocated
through the library.  One JSON line.

    python reference_wrapper_script.py <directory holding example_wrapper.py> <path to sideaware.so>
"""
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from l2_torch_alloc_b200 import functors  # noqa: E402  (header texts only)


def main():
    staged, so = sys.argv[1], sys.argv[2]
    sys.path.insert(0, staged)
    # The wrapper keeps its torch.library.Library in a local variable of sideaware_init (example_wrapper.py:82-92).
    # This torch version unregisters a library's operators when the Library object is collected, i.e. when
    # sideaware_init returns.  The wrapper's text stays as it is; this harness keeps every Library it creates alive.
    kept = []
    original_library = torch.library.Library

    class KeptLibrary(original_library):
        def __init__(self, *a, **k):
            super().__init__(*a, **k)
            kept.append(self)

    torch.library.Library = KeptLibrary
    import example_wrapper as ew  # the reference's file, unmodified

    ew.sideaware_init(so)
    res = {"enabled": ew.sideaware_enabled(), "info": ew.sideaware_info(), "raw": list(ew.sideaware_info_raw())}
    n_sms = res["info"]["num_sms"]
    index = ew.sideaware_torch_side_index().cpu()
    cpu_index = ctypes.string_at(ew.sideaware_cpu_side_index(), n_sms)
    res["side_index_consistent"] = bytes(index.numpy().tobytes()) == cpu_index and ew.sideaware_gpu_side_index() is not None
    res["side_counts_ok"] = (int((index & 1).sum()) == res["info"]["side1"] and res["info"]["side0"] + res["info"]["side1"] == n_sms
                             and res["info"]["min"] == min(res["info"]["side0"], res["info"]["side1"]))

    # memcpy: a small block (runtime pool) and two large ones (side-aware blocks, one needing 64-bit indexing)
    ok = True
    for n in (4 * 777 * 4, 12 << 20, (2 << 30) + 4096):  # bytes; the first is test.py's (4, 777) fp32 tensor
        src = torch.arange(n // 4, dtype=torch.int32, device="cuda")
        dst = torch.zeros_like(src)
        torch.ops.sideaware.memcpy(dst, src)
        ok = ok and bool(torch.equal(dst, src))
        del src, dst
    res["memcpy_exact"] = ok

    # one_to_one with the memcpy functor through NVRTC
    kid = ew.sideaware_create_kernel(functors.MEMCPY.encode())
    src = torch.randint(0, 2**31 - 1, (6 << 20,), dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    torch.ops.sideaware.one_to_one(kid, dst, src)
    res["one_to_one_exact"] = bool(torch.equal(dst, src)) and kid >= 1
    res["same_header_same_id"] = ew.sideaware_create_kernel(functors.MEMCPY.encode()) == kid

    # elementwise: out = bf16(a * sigmoid(a) * b * 0.5), scale passed as the bits of sideband_value
    import numpy as np
    kid2 = ew.sideaware_create_kernel(functors.silu_mul_bf16().encode())
    a = torch.randn(5 << 20, device="cuda").to(torch.bfloat16)
    b = torch.randn(5 << 20, device="cuda").to(torch.bfloat16)
    out = torch.zeros_like(a)
    torch.ops.sideaware.elementwise(kid2, out, None, None, None, a, b, None, None, None,
                                    int(np.float32(0.5).view(np.int32)), 0, 0)
    af, bf = a.float(), b.float()
    want = (((af * torch.sigmoid(af)) * bf) * 0.5).to(torch.bfloat16)
    ulp = (out.view(torch.int16).int() - want.view(torch.int16).int()).abs().max().item()
    res["elementwise_max_bf16_ulp"] = int(ulp)

    @torch.compile(fullgraph=True)
    def compiled(dst, src):
        torch.ops.sideaware.memcpy(dst, src)
        return dst

    src = torch.full((1 << 20,), 3.0, device="cuda")
    res["compiled_memcpy_exact"] = bool(torch.equal(compiled(torch.zeros_like(src), src), src))
    torch.cuda.synchronize()
    print("RESULT " + json.dumps(res))


if __name__ == "__main__":
    main()
