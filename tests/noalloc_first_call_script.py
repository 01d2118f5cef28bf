"""sideaware_memcpy_noalloc as the FIRST thing a process asks of the library: no allocating call has set the
device up, so the entry point looks up the address of its built-in counter array, has no SM side table yet
and copies side-unaware.  The bytes must equal the source.  Free device memory is read before the first
call, between the two calls and after the second: the second call must leave it exactly as it found it
(the first launch of a kernel may make the CUDA runtime load the library's code onto the device, which is
not an allocation the entry point makes, so that difference is only reported).  One JSON line.

    python noalloc_first_call_script.py <path to sideaware.so>
"""
import ctypes
import json
import sys

import torch


def main():
    lib = ctypes.CDLL(sys.argv[1])
    lib.sideaware_memcpy_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    lib.sideaware_memcpy_noalloc.restype = ctypes.c_int
    lib.sideaware_error_count.restype = ctypes.c_ulonglong
    torch.cuda.set_device(0)
    n = (80 << 20) + 4096 + 32
    src = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")
    outs = [torch.zeros(n + 64, dtype=torch.uint8, device="cuda") for _ in range(2)]
    ref = torch.zeros(n + 64, dtype=torch.uint8, device="cuda")
    ref[:n].copy_(src)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    rcs, free = [], [free_before]
    for o in outs:  # two calls in a row
        rcs.append(lib.sideaware_memcpy_noalloc(o.data_ptr(), src.data_ptr(), n, 0, stream))
        torch.cuda.synchronize()
        free.append(torch.cuda.mem_get_info()[0])
    res = {"rcs": rcs, "equal": [bool(torch.equal(o, ref)) for o in outs], "free_before_first": free[0],
           "free_between": free[1], "free_after_second": free[2], "errors": int(lib.sideaware_error_count())}
    print("RESULT " + json.dumps(res))


if __name__ == "__main__":
    main()
