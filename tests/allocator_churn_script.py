"""Allocator churn through torch: `ops` seeded malloc/free operations, sizes log-uniform 4 KiB .. 2 GiB rounded up to
16 bytes, live set capped at 32 GiB, every allocation a torch.empty(size, dtype=uint8) and every free the drop of the
tensor.  Arm "pluggable": the process first installs this library as torch's CUDAPluggableAllocator
(sideaware_malloc_auto / sideaware_free_auto, as test.py:14-15 does); arm "torch": torch's own caching allocator.
Two passes over the same sequence are timed: the first grows the mapped set, the second finds it mapped.
One JSON line.

    python allocator_churn_script.py <pluggable|torch> <ops> [path to sideaware.so]
"""
import ctypes
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def churn(ops):
    rng = np.random.default_rng(0xB200 + 5)
    live, live_bytes, peak = [], 0, 0
    t_small, t_large, t_free = [], [], []
    t_start = time.perf_counter()
    for _ in range(ops):
        if live and (live_bytes > (32 << 30) or rng.random() < 0.45):
            t, size = live.pop(int(rng.integers(len(live))))
            t0 = time.perf_counter_ns()
            del t
            t_free.append(time.perf_counter_ns() - t0)
            live_bytes -= size
        else:
            size = int(np.exp(rng.uniform(np.log(4096), np.log(2 << 30))))
            size = (size + 15) // 16 * 16
            t0 = time.perf_counter_ns()
            try:
                t = torch.empty(size, dtype=torch.uint8, device="cuda")
            except torch.OutOfMemoryError:
                continue
            dt = time.perf_counter_ns() - t0
            (t_large if size >= (8 << 20) else t_small).append(dt)
            live.append((t, size))
            live_bytes += size
            peak = max(peak, live_bytes)
    live.clear()
    elapsed = time.perf_counter() - t_start

    def pct(v, q):
        return float(np.percentile(v, q)) / 1e3 if v else None

    return {"ops": ops, "ops_per_s": ops / elapsed, "seconds": elapsed, "peak_live_gib": peak / 2**30,
            "malloc_small_us_p50": pct(t_small, 50), "malloc_small_us_p99": pct(t_small, 99),
            "malloc_large_us_p50": pct(t_large, 50), "malloc_large_us_p99": pct(t_large, 99),
            "free_us_p50": pct(t_free, 50), "free_us_p99": pct(t_free, 99)}


def main():
    arm, ops = sys.argv[1], int(sys.argv[2])
    so = sys.argv[3] if len(sys.argv) > 3 else os.path.join(ROOT, "l2_torch_alloc_b200", "sideaware.so")
    lib = None
    if arm == "pluggable":
        alloc = torch.cuda.memory.CUDAPluggableAllocator(so, "sideaware_malloc_auto", "sideaware_free_auto")
        torch.cuda.memory.change_current_allocator(alloc)
        lib = ctypes.CDLL(so)
    torch.cuda.set_device(0)
    torch.empty(16, device="cuda")
    torch.cuda.synchronize()
    out = {"arm": arm, "first_pass": churn(ops)}
    torch.cuda.synchronize()
    out["second_pass"] = churn(ops)
    torch.cuda.synchronize()
    if lib is not None and hasattr(lib, "sideaware_error_count"):
        lib.sideaware_error_count.restype = ctypes.c_ulonglong
        out["library_errors"] = int(lib.sideaware_error_count())
    print("RESULT " + json.dumps(out))


if __name__ == "__main__":
    main()
