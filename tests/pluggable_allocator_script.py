"""Runs in a process of its own (torch's allocator can only be replaced before the first
CUDA allocation): the flow of the reference's test.py, re-stated - pluggable allocator
installed, custom ops registered, memcpy on small / odd / >2 GiB tensors compared with
Tensor.copy_, an allocation churn, and the stats afterwards.  Prints one JSON line."""
import json
import sys
import time

import numpy as np
import torch

import l2_torch_alloc_b200 as pkg


def main():
    churn_ops = int(sys.argv[1]) if len(sys.argv) > 1 else 400
    sa = pkg.sideaware_init()
    res = {"summary": sa.summary_dict()}
    ok = True

    def copy_matches(shape, dtype, start=0):
        n = int(np.prod(shape))
        src = torch.arange(n, dtype=dtype, device="cuda").reshape(shape)
        a, b = torch.zeros_like(src), torch.zeros_like(src)
        torch.ops.sideaware.memcpy(a[start:], src[start:])
        b[start:].copy_(src[start:])
        return bool(torch.equal(a, b))

    res["copy_tiny"] = copy_matches((4, 777), torch.float32)
    res["copy_int16"] = copy_matches((1000, 1000), torch.int16)
    res["copy_f64"] = copy_matches((1000, 1000), torch.float64)
    res["copy_40mb"] = copy_matches((10000, 1000), torch.float32)
    res["copy_slice"] = copy_matches((10000, 1000), torch.float32, start=3)
    res["copy_3gb"] = copy_matches((50000, 15000), torch.float32)  # > 2 GiB: 64-bit indexing
    big = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    res["large_tensor_2mib_aligned"] = big.data_ptr() % (2 << 20) == 0
    small = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    res["stats_mid"] = sa.stats()
    del big, small

    # allocation churn: log-uniform sizes 4 KiB .. 2 GiB, bounded live set
    rng = np.random.default_rng(0xB200 + 5)
    live, live_bytes, t0 = [], 0, time.perf_counter()
    for _ in range(churn_ops):
        if live and (live_bytes > (24 << 30) or rng.random() < 0.45):
            t = live.pop(int(rng.integers(len(live))))
            live_bytes -= t.numel()
            del t
        else:
            size = int(np.exp(rng.uniform(np.log(4096), np.log(2 << 30))))
            size = (size + 15) // 16 * 16
            t = torch.empty(size, dtype=torch.uint8, device="cuda")
            t[:: max(1, size // 7)] = 1  # touch it
            live.append(t)
            live_bytes += size
    torch.cuda.synchronize()
    res["churn_ops_per_s"] = churn_ops / (time.perf_counter() - t0)
    live.clear()
    res["stats_end"] = sa.stats()
    res["errors"] = sa.error_count()
    for k, v in res.items():
        if k.startswith("copy_") or k == "large_tensor_2mib_aligned":
            ok = ok and bool(v)
    res["ok"] = ok and res["errors"] == 0
    print("RESULT " + json.dumps(res))
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
