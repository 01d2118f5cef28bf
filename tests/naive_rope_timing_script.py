"""Times llm.c's naive in-place RoPE kernel (example_llmc_rope.cu:89-121, compiled from the reference's sources
into oracle/_ref/libref_rope.so) on this GPU: fp32, at the reference example's shape and at the Llama-3-8B head
geometry, block size 256, CUDA events, median of the repeats.  Checks the first result against the oracle.
One JSON line.  It is a comparison baseline only."""
import ctypes
import json
import os
import statistics
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402


def main():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_rope.so"))
    fn = lib.ref_rope_forward_inplace_kernel1
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    torch.cuda.set_device(0)
    sp = torch.cuda.current_stream().cuda_stream
    res = {}
    for name, (B, T, Nq, Nkv, HS, theta) in (("reference_example_shape", (8, 1024, 32, 32, 128, 10000.0)),
                                             ("llama3_8b_heads_fp32", (8, 8192, 32, 8, 128, 500000.0))):
        H = Nq + 2 * Nkv
        table = oracle.freqs_cis(HS, T, theta, 0)
        tt = torch.from_numpy(table).cuda()
        x = torch.empty((B, T, H, HS), dtype=torch.float32, device="cuda").uniform_(-1, 1)
        if name == "reference_example_shape":
            want = oracle.rope_forward_f32(x[:1].cpu().numpy(), table, 1, T, Nq, Nkv, HS)
        buf = x.clone()
        run = lambda: fn(buf.data_ptr(), tt.data_ptr(), B, T, Nq, Nkv, HS, 256, sp)  # noqa: E731
        assert run() == 0
        torch.cuda.synchronize()
        entry = {}
        if name == "reference_example_shape":
            got = buf[:1].cpu().numpy()
            entry["within_reference_tolerance"] = bool((np.abs(got - want) <= 1e-5 + np.abs(want) * np.finfo(np.float32).eps).all())
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        reps = 20
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        ev[0].record()
        for i in range(reps):
            run()
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))
        moved = 2 * B * T * (Nq + Nkv) * HS * 4 + table.nbytes  # q and k read and written, table once
        entry.update({"ms": ms, "gbs": moved / ms / 1e6, "shape": f"fp32 B={B} T={T} {Nq}q+{Nkv}k+{Nkv}v HS={HS}"})
        res[name] = entry
        del x, buf, tt
    print("RESULT " + json.dumps(res))


if __name__ == "__main__":
    main()
