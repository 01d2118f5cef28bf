"""First use of device 0 in a fresh process, timed, with whatever SIDEAWARE_TOPOLOGY_CACHE says.
Prints the topology, whether it came from the cache file, how long the first use took, and how many of 256
re-measured 4 KiB chunks of a fresh 64 MiB block lie on the side the topology predicts.  One JSON line."""
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import l2_torch_alloc_b200 as pkg  # noqa: E402


def main():
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    torch.cuda.synchronize()
    sa = pkg.SideAware()
    t0 = time.perf_counter()
    summary = sa.summary_dict()
    init_ms = (time.perf_counter() - t0) * 1e3
    topo = json.loads(sa.topology_json())
    p = sa.malloc(64 << 20)
    wrong = sa.verify_chunk_sides(p, 64 << 20, 256, 5)
    sa.free(p)
    print("RESULT " + json.dumps({"summary": summary, "from_cache": bool(topo.get("from_cache")), "init_ms": init_ms,
                                  "side_index": sa.cpu_side_index().hex(), "chunks_on_the_wrong_side": wrong,
                                  "errors": sa.error_count()}))


if __name__ == "__main__":
    main()
