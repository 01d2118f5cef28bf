"""Small, self-terminating workloads for profiler captures.

    python -m tests.profile_case memcpy   [--mib 256] [--reps 4] [--placement aware]
    python -m tests.profile_case rope     [--batch 2]  [--reps 4] [--rope-engine 0]
    python -m tests.profile_case functor  [--mib 256] [--reps 4]
    python -m tests.profile_case functor-jit [--mib 256] [--reps 4]   (the same functor through NVRTC)
    python -m tests.profile_case mxfp8    [--mib 256] [--reps 3]      (bf16 -> MXFP8 functor; --mib is the input size)
    python -m tests.profile_case growth   [--mib 1024] [--reps 3]     (no kernel of interest: host time of
                                                         first-touch allocation and the driver calls it took, as JSON)

Each case touches more than the 126 MB L2 but well under 2 GB of device memory and
launches the kernel of interest a handful of times, so a multi-pass capture ends by itself.
"""
from __future__ import annotations

import argparse

import torch

import l2_torch_alloc_b200 as pkg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["memcpy", "rope", "functor", "functor-jit", "mxfp8", "growth"])
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--placement", default="aware", choices=["aware", "unaware", "wrong"])
    ap.add_argument("--engine", type=int, default=1, help="memcpy engine: 1 = bulk copies (default), 0 = vector")
    ap.add_argument("--rope-engine", type=int, default=0, help="RoPE engine: 0 = vector (default), 1 = staged through shared memory")
    args = ap.parse_args()
    sa = pkg.SideAware()
    sa.set_placement(args.placement)
    sa.lib.sideaware_set_memcpy_engine(args.engine)
    sa.lib.sideaware_set_rope_engine(args.rope_engine)
    torch.cuda.set_device(0)
    if args.case == "growth":
        import json
        import time
        n = args.mib << 20
        out = {"block_mib": args.mib, "blocks": []}
        ptrs = []
        for _ in range(args.reps):
            before = sa.driver_call_times()
            t0 = time.perf_counter()
            p = sa.malloc(n)
            dt = time.perf_counter() - t0
            after = sa.driver_call_times()
            ptrs.append(p)
            out["blocks"].append({"ms": round(dt * 1e3, 2), "us_per_2MiB_page": round(dt * 1e6 / (n / (2 << 20)), 1),
                                  "chunks_not_on_predicted_side_of_512": sa.verify_chunk_sides(p, n, 512, 1),
                                  "driver_calls": {k: {"calls": after[k]["calls"] - before[k]["calls"],
                                                       "ms": round(after[k]["ms"] - before[k]["ms"], 2)} for k in after}})
        st = sa.stats()
        out["stats"] = {k: st[k] for k in ("pages_created", "handles_created", "handles_discarded", "cross_side_pages", "extensions")}
        t0 = time.perf_counter()
        for p in ptrs:
            sa.free(p)
        q = sa.malloc(n)  # served from what is mapped
        out["malloc_after_free_us"] = round((time.perf_counter() - t0) * 1e6, 1)
        sa.free(q)
        print("GROWTH", json.dumps(out))
    elif args.case == "memcpy":
        n = args.mib << 20
        seed = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")
        a, b = sa.malloc(n), sa.malloc(n)
        sa.memcpy_ptr(a, seed.data_ptr(), n)
        for _ in range(args.reps):
            sa.memcpy_ptr(b, a, n)
        out = torch.empty_like(seed)
        sa.memcpy_ptr(out.data_ptr(), b, n)
        torch.cuda.synchronize()
        assert torch.equal(out, seed)
    elif args.case == "mxfp8":
        from l2_torch_alloc_b200 import functors
        n = (args.mib << 20) // 2  # elements
        x = torch.randn(n, device="cuda").to(torch.bfloat16)
        a, o, sc = sa.malloc(2 * n), sa.malloc(max(n, 8 << 20)), sa.malloc(8 << 20)
        sa.memcpy_ptr(a, x.data_ptr(), 2 * n)
        kid = sa.create_kernel(functors.mxfp8_quantize_bf16())
        sp = torch.cuda.current_stream().cuda_stream
        for _ in range(args.reps):
            sa.lib.sideaware_elementwise(kid, 2 * n, o, None, None, None, a, None, None, None, sc, n // 8, 0, 0, 0, sp)
        torch.cuda.synchronize()
    elif args.case == "rope":
        B, T, Nq, Nkv, HS = args.batch, 8192, 32, 8, 128
        n = B * T * (Nq + 2 * Nkv) * HS
        x = torch.randn(n, device="cuda").to(torch.bfloat16)
        half = HS // 2
        inv = 1.0 / (500000.0 ** (torch.arange(0, half, dtype=torch.float32) * 2 / HS))
        ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None, :]
        table = torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous().cuda()
        q = sa.malloc(2 * n)
        sa.memcpy_ptr(q, x.data_ptr(), 2 * n)
        for _ in range(args.reps):
            sa.rope_forward_ptr(q, table.data_ptr(), B, T, Nq, Nkv, HS, True)
        torch.cuda.synchronize()
    else:
        n = (args.mib << 20) // 2
        a = sa.malloc(2 * n)
        b = sa.malloc(2 * n)
        o = sa.malloc(2 * n)
        x = torch.randn(n, device="cuda").to(torch.bfloat16)
        sa.memcpy_ptr(a, x.data_ptr(), 2 * n)
        sa.memcpy_ptr(b, x.data_ptr(), 2 * n)
        if args.case == "functor-jit":
            import numpy as np
            from l2_torch_alloc_b200 import functors
            kid = sa.create_kernel(functors.silu_mul_bf16())
            scale_bits = int(np.float32(0.5).view(np.int32))
            sp = torch.cuda.current_stream().cuda_stream
            for _ in range(args.reps):
                sa.lib.sideaware_elementwise(kid, 2 * n, o, None, None, None, a, b, None, None, None, scale_bits, 0, 0, 0, sp)
        else:
            for _ in range(args.reps):
                sa.silu_mul_ptr(o, a, b, 0.5, n)
        torch.cuda.synchronize()
    assert sa.error_count() == 0, sa.last_error()
    print("profile case done:", args.case, sa.summary_dict())


if __name__ == "__main__":
    main()
