"""Times sideaware_memcpy of a library given by path, in a process of its own:
blocks from the library's own sideaware_malloc_async, CUDA events; per launch (median and mean, an event after
every launch) and launched back to back.
Works for any library with the reference's C ABI (sideaware.cu:1280, :1414), so the same
script measures this project's sideaware.so and the compiled reference.  One JSON line."""
import ctypes
import json
import statistics
import sys

import torch


def main():
    path = sys.argv[1]
    sizes = [int(s) for s in sys.argv[2].split(",")] if len(sys.argv) > 2 else [64 << 20, 1 << 30]
    lib = ctypes.CDLL(path)
    lib.sideaware_malloc_async.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t, ctypes.c_void_p]
    lib.sideaware_malloc_async.restype = ctypes.c_int
    lib.sideaware_free_async.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.sideaware_memcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    lib.sideaware_memcpy.restype = None
    lib.sideaware_sm_side_summary.restype = ctypes.POINTER(ctypes.c_int * 5)
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    sp = torch.cuda.current_stream().cuda_stream
    out = {"lib": path, "summary": list(lib.sideaware_sm_side_summary().contents), "sizes": {}}
    for n in sizes:
        a, b = ctypes.c_void_p(), ctypes.c_void_p()
        assert lib.sideaware_malloc_async(ctypes.byref(a), n, sp) == 0
        assert lib.sideaware_malloc_async(ctypes.byref(b), n, sp) == 0
        seed = torch.randint(0, 2**31 - 1, (n // 4,), dtype=torch.int32, device="cuda")
        lib.sideaware_memcpy(a, seed.data_ptr(), n, 0, sp)
        for _ in range(5):
            lib.sideaware_memcpy(b, a, n, 0, sp)
        torch.cuda.synchronize()
        reps = 30 if n > (256 << 20) else 100
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        ev[0].record()
        for i in range(reps):
            lib.sideaware_memcpy(b, a, n, 0, sp)
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(reps)]
        # event timestamps step by about a microsecond: for short launches the mean over the whole run is finer than the median
        mean_ms = ev[0].elapsed_time(ev[reps]) / reps
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        for i in range(reps):
            lib.sideaware_memcpy(b, a, n, 0, sp)
        last.record()
        torch.cuda.synchronize()
        back_to_back_ms = first.elapsed_time(last) / reps
        back = torch.empty_like(seed)
        lib.sideaware_memcpy(back.data_ptr(), b, n, 0, sp)
        torch.cuda.synchronize()
        out["sizes"][str(n)] = {"median_ms": statistics.median(ms), "gbs": 2 * n / statistics.median(ms) / 1e6,
                                "best_gbs": 2 * n / min(ms) / 1e6, "mean_ms": mean_ms, "back_to_back_ms": back_to_back_ms,
                                "exact": bool(torch.equal(back, seed))}
        lib.sideaware_free_async(a, sp)
        lib.sideaware_free_async(b, sp)
        del seed, back
    print("RESULT " + json.dumps(out))


if __name__ == "__main__":
    main()
