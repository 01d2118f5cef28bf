#!/usr/bin/env python
"""Benchmark of the side-aware hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (one "step"): a side-aware memcpy of a 1 GiB uint8 buffer of
seeded random bytes between two blocks obtained from sideaware_malloc_auto (the
PyTorch pluggable-allocator entry point), launched through the C ABI
(sideaware_memcpy).  The metric is GB/s counting read + written bytes.  With
N > 1 every rank runs an independent replica on its own GPU (the path has no
cross-GPU exchange, so there is no data-path collective); value is the sum of
the ranks' bytes over the slowest rank's time.

One JSON line is printed by rank 0.  Besides the contract keys it carries the
same measurement for the RoPE (bf16, Llama-3-8B shape) and functor workloads
and for the comparison set: the same kernel run side-unaware and on the wrong
side, cudaMemcpyAsync and torch's copy_.

--impl reference times the CPU stand-in on the host cores: the reference has no
CPU memcpy of its own (its check is dst == src, test.py:290-294), so libc memcpy
over all cores is timed for the headline metric, and the reference's own CPU
RoPE (oracle/_ref, compiled from example_llmc_rope.cu in place) is reported
beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GiB = 1 << 30
MEMCPY_BYTES = 1 * GiB
METRIC = "side-aware memcpy & RoPE GB/s per B200 vs 8 TB/s peak and vs side-unaware copy"
ROPE_SHAPE = dict(B=8, T=8192, Nq=32, Nkv=8, HS=128)  # Llama-3-8B heads, bf16, in place on q and k
FUNCTOR_ELEMS = 1 << 30
HBM_FALLBACK_GBS = 6650.0
SPEC_GBS = 8000.0
WORKLOAD = "memcpy 1 GiB uint8 (seeded uniform random bytes)"
# dram__bytes_read.sum + dram__bytes_write.sum of one 1 GiB launch, per kernel, from an ncu capture of that
# kernel at that size.  A profiler cannot run inside a timed benchmark, so this is NOT measured in the run:
# the line says so (traffic_source) and carries null for a kernel that has no capture.
PROFILED_DRAM_TRAFFIC_BYTES = {"sa_memcpy_bulk_kernel": 2085908736}


def bench_config(n_gpus):
    """The workload description; identical in both arms (how each arm runs it is in the line's `path`)."""
    return {"workload": WORKLOAD, "bytes": MEMCPY_BYTES,
            "l2": "inputs larger than L2 (2 GiB touched per step vs 126 MB)",
            "parallelism": f"{n_gpus} independent replicas, no collective"}


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return HBM_FALLBACK_GBS, "fallback"


# ---------------------------------------------------------------------------
# rank plumbing: barrier and max over ranks (gloo on CPU: no GPU data is exchanged)
# ---------------------------------------------------------------------------
class Ranks:
    def __init__(self, gpus: int):
        self.rank = env_int("RANK", 0)
        self.local_rank = env_int("LOCAL_RANK", 0)
        self.world = env_int("WORLD_SIZE", 1)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            dist.init_process_group(backend="gloo", rank=self.rank, world_size=self.world)
            self.dist = dist
        elif gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max(self, value: float) -> float:
        if not self.dist:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def sum(self, value: float) -> float:
        if not self.dist:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t[0])

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


# ---------------------------------------------------------------------------
# clocks during the timed region (NVML, read only)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting", 0x10: "sync_boost",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _once(self):
        nv = self.nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            try:
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:  # noqa: BLE001
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
            self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
        except Exception:  # noqa: BLE001
            pass

    def _run(self):
        while not self._stop.is_set():
            self._once()
            time.sleep(0.002)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()
            self._once()

    def report(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": max(self.power) if self.power else None}


# ---------------------------------------------------------------------------
# timing helpers (CUDA events on the launching stream)
# ---------------------------------------------------------------------------
def time_launches(torch, fn, steps, warmup, ranks=None, per_launch=False):
    """Returns (total_ms, [per-launch ms]) for `steps` calls of fn() after `warmup` untimed calls."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if ranks:
        ranks.barrier()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)] if per_launch else None
    start.record(stream)
    if per_launch:
        marks[0].record(stream)
    for i in range(steps):
        fn()
        if per_launch:
            marks[i + 1].record(stream)
    end.record(stream)
    torch.cuda.synchronize()
    if ranks:
        ranks.barrier()
    total = start.elapsed_time(end)
    each = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)] if per_launch else []
    return total, each


def time_pipeline(torch, step, streams, steps, warmup, ranks=None):
    """Total ms for `steps` calls of step(), which queues its work on `streams` (not on the current stream): the
    streams start behind an event on the current stream and the closing event waits for all of them."""
    cur = torch.cuda.current_stream()
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if ranks:
        ranks.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(cur)
    for st_ in streams:
        st_.wait_event(start)
    for _ in range(steps):
        step()
    for st_ in streams:
        done = torch.cuda.Event()
        done.record(st_)
        cur.wait_event(done)
    end.record(cur)
    torch.cuda.synchronize()
    if ranks:
        ranks.barrier()
    return start.elapsed_time(end)


def compiled_baseline(torch, fn, nbytes):
    """fn() through torch.compile (inductor), as a comparison line only; the library itself uses no compiler of that kind."""
    try:
        t0 = time.perf_counter()
        cfn = torch.compile(fn)
        cfn()
        torch.cuda.synchronize()
        compile_s = time.perf_counter() - t0
        ms, ea = time_launches(torch, cfn, 5, 2, None, per_launch=True)
        return {"gbs": gbs(nbytes, statistics.mean(ea)), "ms": statistics.mean(ea), "compile_s": compile_s}
    except Exception as exc:  # no compiler on the box, unsupported construct ...: the baseline is optional
        return {"unavailable": repr(exc)[:200]}


def load_cudart(torch):
    """The CUDA runtime torch already loaded, for cudaMemcpyAsync on raw pointers."""
    import ctypes
    import glob
    cands = glob.glob(os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cuda_runtime", "lib", "libcudart.so*"))
    for c in cands + ["libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so.12"]:
        try:
            rt = ctypes.CDLL(c)
            break
        except OSError:
            continue
    else:
        raise SystemExit("CUDA runtime library not found")
    rt.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    rt.cudaMallocAsync.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t, ctypes.c_void_p]
    rt.cudaFreeAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return rt


def gbs(nbytes, ms):
    return nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0


# ---------------------------------------------------------------------------
# CPU legs (the only place this file touches oracle/)
# ---------------------------------------------------------------------------
def cpu_memcpy_gbs(nbytes, reps, threads):
    import numpy as np
    from oracle import oracle
    src = np.random.default_rng(0xB200 + 2).integers(0, 256, size=nbytes, dtype=np.uint8)
    dst = np.zeros_like(src)
    lib = oracle.lib()
    lib.oracle_memcpy_mt(dst.ctypes.data, src.ctypes.data, nbytes, threads)  # warm, faults pages in
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        lib.oracle_memcpy_mt(dst.ctypes.data, src.ctypes.data, nbytes, threads)
        times.append(time.perf_counter() - t0)
    assert dst[:: 4097].tobytes() == src[:: 4097].tobytes()
    return 2 * nbytes / statistics.median(times) / 1e9, times


def cpu_rope_reference():
    """The reference's own CPU RoPE at its CPU config (B=4 T=1024 NH=12 HS=64 fp32), single thread
    as written, from oracle/_ref when present, else the C restatement."""
    import numpy as np
    from oracle import oracle
    B, T, NH, HS = 4, 1024, 12, 64
    x = np.random.default_rng(0xB200 + 1).uniform(-1, 1, size=(B, T, 3 * NH, HS)).astype(np.float32)
    tab = oracle.freqs_cis(HS, T, 10000.0, 0)
    out = np.empty_like(x)
    kind = "port"
    if oracle.ref_available():
        try:
            R = oracle.ref()
            fn = lambda: R.ref_apply_rotary_emb_forward(oracle._ptr(out, oracle._f32p), oracle._ptr(x, oracle._f32p),  # noqa: E731
                                                        oracle._ptr(tab, oracle._f32p), B, T, NH, HS)
            fn()
            kind = "reference"
        except Exception:  # noqa: BLE001
            kind = "port"
    if kind == "port":
        L = oracle.lib()
        fn = lambda: L.oracle_rope_forward_f32(oracle._ptr(out, oracle._f32p), oracle._ptr(x, oracle._f32p),  # noqa: E731
                                               oracle._ptr(tab, oracle._f32p), B, T, NH, NH, HS)
        fn()
    times = []
    for _ in range(10):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    best = min(times)
    res = {"kind": kind, "ms": best * 1e3, "gbs": 2 * x.nbytes / best / 1e9, "cores": 1,
           "config": "fp32 B=4 T=1024 NH=12 HS=64"}
    # the same function over all host cores: the batch is cut into shards (the rotation of one batch entry does
    # not depend on the others) and every shard is one call from its own thread (ctypes releases the GIL)
    cores = os.cpu_count() or 1
    Bm = 4 * cores
    xm = np.random.default_rng(0xB200 + 1).uniform(-1, 1, size=(Bm, T, 3 * NH, HS)).astype(np.float32)
    om = np.empty_like(xm)
    per = Bm // cores

    def shard(i):
        xi, oi = xm[i * per:(i + 1) * per], om[i * per:(i + 1) * per]
        if kind == "reference":
            oracle.ref().ref_apply_rotary_emb_forward(oracle._ptr(oi, oracle._f32p), oracle._ptr(xi, oracle._f32p),
                                                      oracle._ptr(tab, oracle._f32p), per, T, NH, HS)
        else:
            oracle.lib().oracle_rope_forward_f32(oracle._ptr(oi, oracle._f32p), oracle._ptr(xi, oracle._f32p),
                                                 oracle._ptr(tab, oracle._f32p), per, T, NH, NH, HS)

    def all_cores():
        ts = [threading.Thread(target=shard, args=(i,)) for i in range(cores)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()

    all_cores()
    mt = []
    for _ in range(5):
        t0 = time.perf_counter()
        all_cores()
        mt.append(time.perf_counter() - t0)
    res["all_cores"] = {"cores": cores, "ms": min(mt) * 1e3, "gbs": 2 * xm.nbytes / min(mt) / 1e9,
                        "config": f"fp32 B={Bm} T=1024 NH=12 HS=64, one shard of {per} per thread"}
    return res


def run_reference(args, ranks):
    if ranks.rank != 0:
        ranks.close()
        return 0
    threads = os.cpu_count() or 1
    # each step = one 1 GiB copy over all cores; bounded so K steps end within minutes
    steps = max(1, min(args.steps, 200))
    warm = max(1, min(args.warmup, 5))
    value, times = cpu_memcpy_gbs(MEMCPY_BYTES, warm + steps, threads)
    times = times[warm:]
    total = sum(times)
    value = 2 * MEMCPY_BYTES * len(times) / total / 1e9
    rope = cpu_rope_reference()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": warm, "ms_per_step": total / len(times) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": bench_config(args.gpus), "path": "libc memcpy on the host cores (rank 0 only)",
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{len(times)} x 1 GiB libc memcpy over {threads} threads "
                                   "(the reference ships no CPU memcpy; its check is dst == src)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "rope_cpu": rope,
    }
    print(json.dumps(line), flush=True)
    ranks.close()
    return 0



# ---------------------------------------------------------------------------
# allocator churn and power (extras, rank 0 at N = 1)
# ---------------------------------------------------------------------------
def allocator_churn(lib, rt, dev, sp, ops, arm="sideaware"):
    """`ops` seeded malloc/free calls, sizes log-uniform 4 KiB .. 2 GiB rounded up to 16 B, live set capped
    at 32 GiB.  arm "sideaware": sideaware_malloc_auto / sideaware_free_auto (what torch's pluggable allocator
    calls); for comparison "cudaMallocAsync": the runtime's stream-ordered pool.  The same sequence through
    torch.empty (pluggable allocator, torch's own caching allocator) runs in tests/allocator_churn_script.py."""
    import ctypes
    import numpy as np
    rng = np.random.default_rng(0xB200 + 5)
    live, live_bytes, peak = [], 0, 0
    t_malloc_small, t_malloc_large, t_free = [], [], []
    p = ctypes.c_void_p()

    def do_malloc(size):
        if arm == "cudaMallocAsync":
            rc = rt.cudaMallocAsync(ctypes.byref(p), size, sp)
            return p.value if rc == 0 else None
        return lib.sideaware_malloc_auto(size, dev, sp)

    def do_free(ptr, size):
        if arm == "cudaMallocAsync":
            rt.cudaFreeAsync(ptr, sp)
        else:
            lib.sideaware_free_auto(ptr, size, dev, sp)

    t_start = time.perf_counter()
    for _ in range(ops):
        if live and (live_bytes > (32 << 30) or rng.random() < 0.45):
            ptr, size = live.pop(int(rng.integers(len(live))))
            t0 = time.perf_counter_ns()
            do_free(ptr, size)
            ptr = None
            t_free.append(time.perf_counter_ns() - t0)
            live_bytes -= size
        else:
            size = int(np.exp(rng.uniform(np.log(4096), np.log(2 << 30))))
            size = (size + 15) // 16 * 16
            t0 = time.perf_counter_ns()
            ptr = do_malloc(size)
            dt = time.perf_counter_ns() - t0
            if not ptr:
                continue
            (t_malloc_large if size >= (8 << 20) else t_malloc_small).append(dt)
            live.append((ptr, size))
            live_bytes += size
            peak = max(peak, live_bytes)
    while live:
        ptr, size = live.pop()
        do_free(ptr, size)
        ptr = None
    elapsed = time.perf_counter() - t_start

    def pct(v, q):
        return float(np.percentile(v, q)) / 1e3 if v else None

    return {"ops": ops, "ops_per_s": ops / elapsed, "seconds": elapsed, "peak_live_gib": peak / 2**30,
            "malloc_small_us_p50": pct(t_malloc_small, 50), "malloc_small_us_p99": pct(t_malloc_small, 99),
            "malloc_large_us_p50": pct(t_malloc_large, 50), "malloc_large_us_p99": pct(t_malloc_large, 99),
            "malloc_large_us_max": max(t_malloc_large) / 1e3 if t_malloc_large else None,
            "malloc_large_calls": len(t_malloc_large), "malloc_large_over_5ms": sum(1 for t in t_malloc_large if t > 5e6),
            "free_us_p50": pct(t_free, 50), "free_us_p99": pct(t_free, 99)}


def power_run(torch, fn, nbytes, seconds, index):
    """Runs fn() back to back for about `seconds` and samples board power through NVML."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
    except Exception:  # noqa: BLE001
        return None
    samples, stop = [], threading.Event()

    def sampler():
        while not stop.is_set():
            try:
                samples.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.01)

    for _ in range(20):
        fn()
    torch.cuda.synchronize()
    th = threading.Thread(target=sampler, daemon=True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    th.start()
    t0 = time.perf_counter()
    n = 0
    start.record()
    while time.perf_counter() - t0 < seconds:
        for _ in range(50):
            fn()
        n += 50
        torch.cuda.synchronize()
    end.record()
    torch.cuda.synchronize()
    stop.set()
    th.join()
    ms = start.elapsed_time(end)
    tail = samples[len(samples) // 3:] or samples  # the power reading lags: use the settled part
    watts = statistics.mean(tail) if tail else None
    rate = n * nbytes / (ms * 1e-3) / 1e9
    return {"watts": watts, "gbs": rate, "joule_per_gb": (watts / rate) if watts else None, "samples": len(samples)}

# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class Ctx:
    """What the sections of the GPU arm share."""

    def __init__(self, args, ranks):
        import torch

        import l2_torch_alloc_b200 as pkg
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
        self.torch, self.args, self.ranks = torch, args, ranks
        self.dev = ranks.local_rank % torch.cuda.device_count()
        torch.cuda.set_device(self.dev)
        torch.zeros(1, device="cuda")
        torch.cuda.synchronize()
        self.sa = pkg.SideAware()  # raises if sideaware.so has not been built
        self.lib = self.sa.lib
        t0 = time.perf_counter()
        self.summary = self.sa.summary_dict()  # first use of the device: context check, probe page, discovery, side table
        self.summary["init_ms"] = (time.perf_counter() - t0) * 1e3
        self.stream = torch.cuda.current_stream()
        self.sp = self.stream.cuda_stream
        self.rt = load_cudart(torch)
        self.peak, self.peak_kind = measured_peak()

    def alloc(self, nbytes):
        p = self.lib.sideaware_malloc_auto(nbytes, self.dev, self.sp)
        if not p:
            raise MemoryError(self.sa.last_error())
        return p

    def free(self, p, nbytes):
        self.lib.sideaware_free_auto(p, nbytes, self.dev, self.sp)

    def kernel_entry(self, kernel, config, nbytes, fn, steps, warmup=3):
        """One entry of roofline.kernels: `steps` launches back to back between two events (the way the headline is
        timed: achieved = algorithmic bytes / average launch duration), plus a pass with an event after every launch."""
        tot, _ = time_launches(self.torch, fn, steps, warmup, None, per_launch=False)
        _, each = time_launches(self.torch, fn, steps, warmup, None, per_launch=True)
        ms = tot / steps
        return {"kernel": kernel, "config": config, "algorithmic_bytes": nbytes, "ms": ms, "achieved": gbs(nbytes, ms),
                "frac": gbs(nbytes, ms) / self.peak, "launches": steps,
                "event_per_launch_ms": statistics.mean(each), "event_per_launch_best_ms": min(each),
                "event_per_launch_gbs": gbs(nbytes, statistics.mean(each))}


def headline_memcpy(c):
    """The timed region of the bench contract: K 1 GiB copies back to back, max over ranks."""
    torch, lib, args, ranks = c.torch, c.lib, c.args, c.ranks
    gen = torch.Generator(device="cuda").manual_seed(0xB200 + 2 + ranks.rank)
    c.seed_t = torch.randint(0, 256, (MEMCPY_BYTES,), dtype=torch.uint8, device="cuda", generator=gen)
    c.src, c.dst = c.alloc(MEMCPY_BYTES), c.alloc(MEMCPY_BYTES)
    lib.sideaware_memcpy(c.src, c.seed_t.data_ptr(), MEMCPY_BYTES, c.dev, c.sp)
    torch.cuda.synchronize()
    launches_before = c.sa.stats()["kernel_launches"]

    def step():
        lib.sideaware_memcpy(c.dst, c.src, MEMCPY_BYTES, c.dev, c.sp)

    c.step = step
    c.sa.set_placement("aware")
    # K launches back to back, one event before and one after (an event between two launches would keep
    # consecutive kernels from overlapping launch and tail)
    with ClockSampler(c.dev) as clocks:
        total_ms, _ = time_launches(torch, step, args.steps, args.warmup, ranks, per_launch=False)
    launches = c.sa.stats()["kernel_launches"] - launches_before - args.warmup  # counted by the library itself
    worst_ms = ranks.max(total_ms)
    value = ranks.world * args.steps * 2 * MEMCPY_BYTES / (worst_ms * 1e-3) / 1e9
    # the same launches for about a second, only to give the clock sampler more than a handful of samples
    long_steps = max(args.steps, int(1000.0 / max(total_ms / args.steps, 1e-3)))
    with ClockSampler(c.dev) as clocks_long:
        time_launches(torch, step, long_steps, 0, None, per_launch=False)
    _, each = time_launches(torch, step, min(args.steps, 50), 3, None, per_launch=True)
    # parity spot check of what was just timed
    back = torch.empty_like(c.seed_t)
    lib.sideaware_memcpy(back.data_ptr(), c.dst, MEMCPY_BYTES, c.dev, c.sp)
    torch.cuda.synchronize()
    if not torch.equal(back, c.seed_t):
        raise SystemExit("bench: the timed copy is not bit-exact")
    del back
    avg_launch_ms = total_ms / args.steps
    achieved = gbs(2 * MEMCPY_BYTES, avg_launch_ms)
    kernel = "sa_memcpy_bulk_kernel" if lib.sideaware_get_memcpy_engine() == 1 else "sa_memcpy_kernel"
    traffic = PROFILED_DRAM_TRAFFIC_BYTES.get(kernel)
    roofline = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": c.peak, "unit": "GB/s",
                "frac": achieved / c.peak, "peak_kind": f"of {c.peak_kind}", "frac_of_spec_8000": achieved / SPEC_GBS,
                "traffic": traffic,
                "traffic_source": ("ncu capture of one 1 GiB launch of this kernel (dram__bytes_read.sum + dram__bytes_write.sum); "
                                   "not measured in this run") if traffic else None,
                "algorithmic_bytes_per_launch": 2 * MEMCPY_BYTES,
                "best_launch_ms": min(each), "median_launch_ms": statistics.median(each)}
    entry = {"kernel": kernel, "config": "1 GiB uint8 copy, side-aware blocks", "algorithmic_bytes": 2 * MEMCPY_BYTES,
             "ms": avg_launch_ms, "achieved": achieved, "frac": achieved / c.peak, "launches": args.steps,
             "event_per_launch_ms": statistics.mean(each), "event_per_launch_best_ms": min(each),
             "event_per_launch_gbs": gbs(2 * MEMCPY_BYTES, statistics.mean(each))}
    rep = clocks.report()
    rep["one_second_of_the_same_launches"] = clocks_long.report()
    return value, worst_ms, roofline, entry, rep, int(launches)


def pcie_limits(c):
    """Pinned-memory copy rates of this box: each direction alone and both at once (what bounds any end-to-end figure)."""
    torch, rt = c.torch, c.rt
    n = 256 << 20
    h_a = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    h_b = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    d_a = torch.empty(n, dtype=torch.uint8, device="cuda")
    d_b = torch.empty(n, dtype=torch.uint8, device="cuda")
    s2 = torch.cuda.Stream()
    ms_up, _ = time_launches(torch, lambda: rt.cudaMemcpyAsync(d_a.data_ptr(), h_a.data_ptr(), n, 1, c.sp), 8, 2)
    ms_dn, _ = time_launches(torch, lambda: rt.cudaMemcpyAsync(h_b.data_ptr(), d_b.data_ptr(), n, 2, c.sp), 8, 2)
    ev0, ev1 = torch.cuda.Event(), torch.cuda.Event()

    def both():
        ev0.record(c.stream)
        s2.wait_event(ev0)
        rt.cudaMemcpyAsync(d_a.data_ptr(), h_a.data_ptr(), n, 1, c.sp)
        rt.cudaMemcpyAsync(h_b.data_ptr(), d_b.data_ptr(), n, 2, s2.cuda_stream)
        ev1.record(s2)
        c.stream.wait_event(ev1)

    ms_both, _ = time_launches(torch, both, 8, 2)
    return {"h2d_gbs": gbs(n, ms_up / 8), "d2h_gbs": gbs(n, ms_dn / 8), "both_directions_each_gbs": gbs(n, ms_both / 8),
            "note": "pinned host memory, 256 MiB copies; an end-to-end step moves its bytes once in each direction, so "
                    "its GB/s (read + written bytes) cannot exceed twice the both-directions rate"}


def e2e_memcpy(c):
    """Host buffer -> device -> side-aware copy -> device -> host buffer, per step, pipelined over pieces on three streams."""
    torch, lib, rt, ranks = c.torch, c.lib, c.rt, c.ranks
    e2e_steps = max(3, min(c.args.steps, 10))
    h_src = torch.empty(MEMCPY_BYTES, dtype=torch.uint8, pin_memory=True)
    h_dst = torch.empty(MEMCPY_BYTES, dtype=torch.uint8, pin_memory=True)
    h_src.copy_(c.seed_t)
    torch.cuda.synchronize()
    piece = c.args.e2e_piece_mib << 20
    n_pieces = MEMCPY_BYTES // piece
    s_up, s_k, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_up = [torch.cuda.Event() for _ in range(n_pieces)]
    ev_k = [torch.cuda.Event() for _ in range(n_pieces)]
    ev_down = [torch.cuda.Event() for _ in range(n_pieces)]

    def e2e_step():
        # Steps follow one another like buffers in a stream of work: nothing waits for a whole step, only for what a
        # piece needs (its upload before its kernel before its download; and, against the step before, the kernel that
        # read a source piece before that piece is overwritten, the download that read a destination piece likewise).
        for i in range(n_pieces):
            off = i * piece
            s_up.wait_event(ev_k[i])
            rt.cudaMemcpyAsync(c.src + off, h_src.data_ptr() + off, piece, 1, s_up.cuda_stream)
            ev_up[i].record(s_up)
            s_k.wait_event(ev_up[i])
            s_k.wait_event(ev_down[i])
            lib.sideaware_memcpy(c.dst + off, c.src + off, piece, c.dev, s_k.cuda_stream)
            ev_k[i].record(s_k)
            s_down.wait_event(ev_k[i])
            rt.cudaMemcpyAsync(h_dst.data_ptr() + off, c.dst + off, piece, 2, s_down.cuda_stream)
            ev_down[i].record(s_down)

    e2e_ms = time_pipeline(torch, e2e_step, (s_up, s_k, s_down), e2e_steps, 2, ranks)
    e2e_worst = ranks.max(e2e_ms)
    e2e_value = ranks.world * e2e_steps * 2 * MEMCPY_BYTES / (e2e_worst * 1e-3) / 1e9
    h_dst.zero_()
    e2e_step()
    torch.cuda.synchronize()
    if not torch.equal(h_dst, h_src):
        raise SystemExit("bench: end-to-end copy mismatch")
    return {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": MEMCPY_BYTES, "d2h_bytes_per_step": MEMCPY_BYTES,
            "steps": e2e_steps, "ms_per_step": e2e_worst / e2e_steps,
            "pipeline": f"{n_pieces} pieces of {piece >> 20} MiB on 3 streams (upload / kernel / download overlap); steps follow "
                        "one another without a wait in between, every step uploads its input and downloads its result"}


def flushed_launch_ms(c, fn, reps, flush_buf):
    """Median duration of fn() when an L2-sized memset runs before every launch (the reference's timing method,
    example_llmc_common.h:364-372): events bracket the launch only."""
    torch = c.torch
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for _ in range(2):
        fn()
    for a, b in ev:
        flush_buf.zero_()
        a.record(c.stream)
        fn()
        b.record(c.stream)
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in ev)


def run_script(script, *argv, timeout=900, cwd=None):
    """Runs one of the committed timing scripts in a process of its own and returns its RESULT line."""
    import subprocess
    try:
        r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", script), *argv], capture_output=True, text=True,
                           timeout=timeout, cwd=cwd or ROOT)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"{script} did not finish in {timeout} s"}
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")]
    if r.returncode != 0 or not lines:
        return {"unavailable": (r.stderr or r.stdout)[-300:]}
    return json.loads(lines[-1][7:])


def comparison_memcpy(c):
    """The same 1 GiB copy by: both engines, the three placements, cudaMemcpyAsync, torch copy_, and the reference's
    own library (its allocator and its JIT-ed kernel, compiled from the reference's sources) in a process of its own."""
    torch, lib, rt, sa = c.torch, c.lib, c.rt, c.sa
    sub_steps = max(5, min(c.args.steps, 30))
    nb = 2 * MEMCPY_BYTES

    def measure(fn):
        _, ea = time_launches(torch, fn, sub_steps, 3, None, per_launch=True)
        tot, _ = time_launches(torch, fn, sub_steps, 3, None, per_launch=False)
        return {"gbs": gbs(nb, statistics.mean(ea)), "best_gbs": gbs(nb, min(ea)), "back_to_back_gbs": gbs(nb, tot / sub_steps)}

    comp = {}
    lib.sideaware_set_memcpy_engine(0)  # the 128-bit vector engine, for comparison with the default bulk engine
    comp["kernel_vector_engine_aware"] = measure(c.step)
    lib.sideaware_set_memcpy_engine(1)
    for mode in ("aware", "unaware", "wrong"):
        sa.set_placement(mode)
        comp[f"kernel_{mode}"] = measure(c.step)
    sa.set_placement("aware")
    comp["cudaMemcpyAsync_d2d"] = measure(lambda: rt.cudaMemcpyAsync(c.dst, c.src, MEMCPY_BYTES, 3, c.sp))
    t_dst = torch.empty_like(c.seed_t)
    comp["torch_copy_"] = measure(lambda: t_dst.copy_(c.seed_t))
    del t_dst
    return comp


def reference_gpu_library(c):
    """The reference's own GPU path on this box, where oracle/_ref holds it: memcpy at 1 GiB, its RoPE header through
    its NVRTC template at the reference example's shape, and llm.c's naive RoPE kernel at the same shape.  Each runs
    in a process of its own, outside every timed region of this file (the two libraries export the same symbols)."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    ref_so = os.path.join(ref_dir, "sideaware_reference.so")
    ours_so = os.path.join(ROOT, "l2_torch_alloc_b200", "sideaware.so")
    if not os.path.exists(ref_so):
        return None, None
    mem, rope = {}, {}
    one_gib = str(1 << 30)
    for name, so in (("reference_library", ref_so), ("this_library_same_script", ours_so)):
        r = run_script("memcpy_timing_script.py", so, one_gib)
        mem[name] = r["sizes"][one_gib] if "sizes" in r else r
    for name, so in (("reference_library_nvrtc", ref_so), ("this_library_nvrtc", ours_so)):
        rope[name] = run_script("rope_functor_timing_script.py", so)
    if os.path.exists(os.path.join(ref_dir, "kernel_rope.cuh")):
        rope["this_library_nvrtc_reference_header_included"] = run_script("rope_functor_timing_script.py", ours_so, "include", cwd=ref_dir)
        rope["reference_library_nvrtc_reference_header_included"] = run_script("rope_functor_timing_script.py", ref_so, "include", cwd=ref_dir)
    rope["llmc_naive_kernel1"] = run_script("naive_rope_timing_script.py")
    rope["config"] = "fp32 B=8 T=1024 32+32+32 heads HS=128 in place (the reference example's shape)"
    return mem, rope


def power_section(c):
    """Board power while copying (the reference's headline claim is power, sideaware.cu:4)."""
    power = {}
    for mode in ("aware", "unaware"):
        c.sa.set_placement(mode)
        power[f"kernel_{mode}"] = power_run(c.torch, c.step, 2 * MEMCPY_BYTES, c.args.power_seconds, c.dev)
    c.sa.set_placement("aware")
    power["cudaMemcpyAsync_d2d"] = power_run(c.torch, lambda: c.rt.cudaMemcpyAsync(c.dst, c.src, MEMCPY_BYTES, 3, c.sp),
                                             2 * MEMCPY_BYTES, c.args.power_seconds, c.dev)
    return power


def sweep_memcpy(c):
    """4 MiB .. 8 GiB (threshold lowered so 4 MiB blocks are side-aware too).  Sizes whose source and destination fit
    the 126 MB L2 together are L2 figures when launched back to back, so every size up to 256 MiB is also timed with an
    L2-sized memset before each launch."""
    torch, lib, rt = c.torch, c.lib, c.rt
    sweep = {}
    flush_buf = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2
    lib.sideaware_alloc_threshold(4 << 20)
    for shift in range(22, 34):
        n = 1 << shift
        try:
            a, b = c.alloc(n), c.alloc(n)
        except MemoryError:
            break
        f = lambda: lib.sideaware_memcpy(b, a, n, c.dev, c.sp)  # noqa: E731
        g = lambda: rt.cudaMemcpyAsync(b, a, n, 3, c.sp)  # noqa: E731
        reps = 40 if n <= (256 << 20) else 10
        _, ea = time_launches(torch, f, reps, 3, None, per_launch=True)
        tot, _ = time_launches(torch, f, reps, 3, None, per_launch=False)
        tot_rt, _ = time_launches(torch, g, reps, 3, None, per_launch=False)
        row = {"gbs": gbs(2 * n, statistics.median(ea)), "us": statistics.median(ea) * 1e3,
               "back_to_back_us": tot / reps * 1e3, "back_to_back_gbs": gbs(2 * n, tot / reps),
               "cudaMemcpyAsync_back_to_back_us": tot_rt / reps * 1e3,
               "cudaMemcpyAsync_back_to_back_gbs": gbs(2 * n, tot_rt / reps),
               "back_to_back_is": ("L2-resident" if 2 * n <= 126_000_000 else
                                   "partly L2-resident" if n <= 126_000_000 else "larger than L2")}
        if n <= (256 << 20):
            ms_f = flushed_launch_ms(c, f, 20, flush_buf)
            ms_g = flushed_launch_ms(c, g, 20, flush_buf)
            row.update({"l2_flushed_us": ms_f * 1e3, "l2_flushed_gbs": gbs(2 * n, ms_f),
                        "cudaMemcpyAsync_l2_flushed_us": ms_g * 1e3, "cudaMemcpyAsync_l2_flushed_gbs": gbs(2 * n, ms_g)})
        sweep[str(n)] = row
        c.free(a, n)
        c.free(b, n)
    lib.sideaware_alloc_threshold(8 << 20)
    lib.sideaware_release_unused()
    del flush_buf
    return sweep


def rope_section(c):
    """RoPE bf16 at the Llama-3-8B shape; every rank runs it on its own batch shard."""
    torch, lib, sa, ranks = c.torch, c.lib, c.sa, c.ranks
    S = ROPE_SHAPE
    H = S["Nq"] + 2 * S["Nkv"]
    rope_elems = S["B"] * S["T"] * H * S["HS"]
    moved = 2 * S["B"] * S["T"] * (S["Nq"] + S["Nkv"]) * S["HS"] * 2 + S["T"] * S["HS"] * 4
    gen = torch.Generator(device="cuda").manual_seed(0xB200 + 3 + ranks.rank)
    x = torch.randn(rope_elems, dtype=torch.float32, device="cuda", generator=gen).to(torch.bfloat16)
    qkv = c.alloc(rope_elems * 2)
    lib.sideaware_memcpy(qkv, x.data_ptr(), rope_elems * 2, c.dev, c.sp)
    half = S["HS"] // 2
    inv = 1.0 / (500000.0 ** (torch.arange(0, half, dtype=torch.float32) * 2 / S["HS"]))
    ang = torch.arange(S["T"], dtype=torch.float32)[:, None] * inv[None, :]
    table = torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous().cuda()
    cfg = "bf16 B=8 T=8192 32q+8kv HS=128 theta=500000 in place"

    def rope_step():
        rc = lib.sideaware_rope_forward(qkv, table.data_ptr(), S["B"], S["T"], S["Nq"], S["Nkv"], S["HS"], 1, c.dev, c.sp)
        if rc:
            raise SystemExit(f"rope launch failed: {sa.last_error()}")

    steps = max(5, min(c.args.steps, 50))
    rope = {"algorithmic_bytes": moved, "config": cfg}
    # the job-wide figure: all ranks together, slowest rank's time, launches back to back as for the headline
    tot, _ = time_launches(torch, rope_step, steps, 3, ranks, per_launch=False)
    rope["aggregate_gbs"] = ranks.world * steps * moved / (ranks.max(tot) * 1e-3) / 1e9
    entries = []
    default_engine = lib.sideaware_get_rope_engine()
    kernel_names = {0: "sa_rope_kernel<bf16>", 1: "sa_rope_bulk_kernel<bf16>"}
    entries.append(c.kernel_entry(kernel_names[default_engine], cfg, moved, rope_step, steps))
    rope["aware"] = {"gbs": entries[0]["event_per_launch_gbs"], "best_gbs": gbs(moved, entries[0]["event_per_launch_best_ms"]),
                     "back_to_back_gbs": entries[0]["achieved"], "ms": entries[0]["event_per_launch_ms"]}
    rope["frac_of_peak"] = entries[0]["frac"]
    if ranks.rank == 0:
        for mode in ("unaware", "wrong"):
            sa.set_placement(mode)
            _, ea = time_launches(torch, rope_step, steps, 3, None, per_launch=True)
            tot, _ = time_launches(torch, rope_step, steps, 3, None, per_launch=False)
            rope[mode] = {"gbs": gbs(moved, statistics.mean(ea)), "best_gbs": gbs(moved, min(ea)),
                          "back_to_back_gbs": gbs(moved, tot / steps), "ms": statistics.mean(ea)}
        sa.set_placement("aware")
        other = 1 - default_engine
        lib.sideaware_set_rope_engine(other)
        e = c.kernel_entry(kernel_names[other], cfg + " (the engine that is not the default)", moved, rope_step, steps)
        lib.sideaware_set_rope_engine(default_engine)
        rope["other_engine"] = e

        # end to end for RoPE: pinned host tensor -> device -> rotation in place -> pinned host, per step, one batch
        # entry at a time on three streams so that upload, kernel and download overlap
        if ranks.world == 1:
            nbytes = rope_elems * 2
            per_b = nbytes // S["B"]
            h = torch.empty(rope_elems, dtype=torch.bfloat16, pin_memory=True)
            h.copy_(x)
            torch.cuda.synchronize()
            s_up, s_k, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
            ev_up = [torch.cuda.Event() for _ in range(S["B"])]
            ev_k = [torch.cuda.Event() for _ in range(S["B"])]
            ev_down = [torch.cuda.Event() for _ in range(S["B"])]

            def e2e_rope_step():
                for b in range(S["B"]):
                    off = b * per_b
                    s_up.wait_event(ev_down[b])  # the step before has read this entry back
                    c.rt.cudaMemcpyAsync(qkv + off, h.data_ptr() + off, per_b, 1, s_up.cuda_stream)
                    ev_up[b].record(s_up)
                    s_k.wait_event(ev_up[b])
                    lib.sideaware_rope_forward(qkv + off, table.data_ptr(), 1, S["T"], S["Nq"], S["Nkv"], S["HS"], 1, c.dev, s_k.cuda_stream)
                    ev_k[b].record(s_k)
                    s_down.wait_event(ev_k[b])
                    c.rt.cudaMemcpyAsync(h.data_ptr() + off, qkv + off, per_b, 2, s_down.cuda_stream)
                    ev_down[b].record(s_down)

            ms = time_pipeline(torch, e2e_rope_step, (s_up, s_k, s_down), 4, 1, None)
            rope["e2e"] = {"value": gbs(moved, ms / 4), "unit": "GB/s (same algorithmic bytes as the kernel figure)",
                           "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "ms_per_step": ms / 4,
                           "pipeline": "8 batch entries on 3 streams (upload / kernel / download overlap), steps one behind the other without a wait; V heads travel too"}
            del h

        # torch eager on the same packed tensor (fp32 math on the q,k heads, written back as bf16), as a baseline
        xt = x.view(S["B"], S["T"], H, S["HS"])
        rot = S["Nq"] + S["Nkv"]
        cos = table[:, :, 0][None, :, None, :]
        sin = table[:, :, 1][None, :, None, :]

        def eager_rope():
            qk = xt[:, :, :rot, :].float().view(S["B"], S["T"], rot, half, 2)
            re = qk[..., 0] * cos - qk[..., 1] * sin
            im = qk[..., 0] * sin + qk[..., 1] * cos
            xt[:, :, :rot, :] = torch.stack((re, im), dim=-1).view(S["B"], S["T"], rot, S["HS"]).to(torch.bfloat16)

        _, ea = time_launches(torch, eager_rope, 5, 2, None, per_launch=True)
        rope["torch_eager"] = {"gbs": gbs(moved, statistics.mean(ea)), "ms": statistics.mean(ea)}
        if ranks.world == 1 and not c.args.no_torch_compile:
            rope["torch_compile"] = compiled_baseline(torch, eager_rope, moved)
        del xt, cos, sin
    c.free(qkv, rope_elems * 2)
    del x, table
    return rope, entries


def functor_section(c):
    """out = bf16(a * sigmoid(a) * b * 0.5) over 2^30 elements (ahead-of-time kernel and the same functor through
    NVRTC), and the bf16 -> MXFP8 functor over the same input."""
    import numpy as np
    from l2_torch_alloc_b200 import functors
    torch, lib, sa = c.torch, c.lib, c.sa
    n = FUNCTOR_ELEMS
    a, b, o = c.alloc(2 * n), c.alloc(2 * n), c.alloc(2 * n)
    g2 = torch.Generator(device="cuda").manual_seed(0xB200 + 4)
    chunk = 1 << 27
    for off in range(0, n, chunk):
        for buf in (a, b):
            t = torch.randn(chunk, dtype=torch.float32, device="cuda", generator=g2).to(torch.bfloat16)
            lib.sideaware_memcpy(buf + 2 * off, t.data_ptr(), 2 * chunk, c.dev, c.sp)
    torch.cuda.synchronize()
    kid = sa.create_kernel(functors.silu_mul_bf16())
    scale_bits = int(np.float32(0.5).view(np.int32))
    f_jit = lambda: lib.sideaware_elementwise(kid, 2 * n, o, None, None, None, a, b, None, None, None, scale_bits, 0, 0, c.dev, c.sp)  # noqa: E731
    f_aot = lambda: lib.sideaware_silu_mul_bf16(o, a, b, 0.5, n, c.dev, c.sp)  # noqa: E731
    cfg = "bf16 2^30 elements, three side-tagged buffers"
    functor = {"algorithmic_bytes": 6 * n, "config": cfg}
    entries = [c.kernel_entry("sa_silu_mul_kernel", cfg, 6 * n, f_aot, 10, 2),
               c.kernel_entry("sideaware_elementwise (NVRTC, silu-mul functor)", cfg, 6 * n, f_jit, 10, 2)]
    for name, e in zip(("aot", "nvrtc"), entries):
        functor[f"{name}_aware"] = {"gbs": e["event_per_launch_gbs"], "ms": e["event_per_launch_ms"], "back_to_back_gbs": e["achieved"]}
    sa.set_placement("unaware")
    for name, f in (("aot", f_aot), ("nvrtc", f_jit)):
        _, ea = time_launches(torch, f, 10, 2, None, per_launch=True)
        functor[f"{name}_unaware"] = {"gbs": gbs(6 * n, statistics.mean(ea)), "ms": statistics.mean(ea)}
    sa.set_placement("aware")
    functor["frac_of_peak"] = entries[0]["frac"]

    # bf16 -> MXFP8: 2 bytes read, 1 byte + 1/32 byte written per element; the output reuses `o`, the scales `b`
    kid_mx = sa.create_kernel(functors.mxfp8_quantize_bf16())
    mx_bytes = 2 * n + n + n // 32
    f_mx = lambda: lib.sideaware_elementwise(kid_mx, 2 * n, o, None, None, None, a, None, None, None, b, n // 8, 0, 0, c.dev, c.sp)  # noqa: E731
    mx_cfg = "bf16 -> E4M3 + E8M0 block scales, 2^30 elements"
    entries.append(c.kernel_entry("sideaware_elementwise (NVRTC, MXFP8 functor)", mx_cfg, mx_bytes, f_mx, 10, 2))
    sa.set_placement("unaware")
    _, ea = time_launches(torch, f_mx, 10, 2, None, per_launch=True)
    sa.set_placement("aware")
    functor["mxfp8"] = {"algorithmic_bytes": mx_bytes, "config": mx_cfg, "aware_gbs": entries[2]["event_per_launch_gbs"],
                        "aware_back_to_back_gbs": entries[2]["achieved"], "unaware_gbs": gbs(mx_bytes, statistics.mean(ea))}
    for buf in (a, b, o):
        c.free(buf, 2 * n)
    # torch eager F.silu(a) * b * 0.5 on torch-allocated tensors of the same size, as a baseline
    ta = torch.empty(n, dtype=torch.bfloat16, device="cuda").normal_(generator=g2)
    tb = torch.empty(n, dtype=torch.bfloat16, device="cuda").normal_(generator=g2)
    _, ea = time_launches(torch, lambda: torch.nn.functional.silu(ta) * tb * 0.5, 5, 2, None, per_launch=True)
    functor["torch_eager"] = {"gbs": gbs(6 * n, statistics.mean(ea)), "ms": statistics.mean(ea),
                              "note": "three kernels with bf16 temporaries; GB/s counts the same 6 bytes per element"}
    if c.ranks.world == 1 and not c.args.no_torch_compile:
        functor["torch_compile"] = compiled_baseline(torch, lambda: torch.nn.functional.silu(ta) * tb * 0.5, 6 * n)
    del ta, tb
    if sa.error_count():
        functor["errors"] = sa.last_error()
    return functor, entries


def churn_section(c):
    """The allocator churn of the benchmark configuration, two ways: through torch.empty under the pluggable allocator
    in a process of its own (what the configuration names), and by calling the two entry points directly from here.
    Beside them the same sequence on cudaMallocAsync and on torch's own caching allocator."""
    ops = c.args.churn_ops
    c.lib.sideaware_release_unused()
    c.torch.cuda.synchronize()
    churn = {"ops": ops, "sizes": "log-uniform 4 KiB .. 2 GiB, rounded up to 16 B; live set capped at 32 GiB"}
    direct = allocator_churn(c.lib, c.rt, c.dev, c.sp, ops)
    direct["stats"] = c.sa.stats()
    # the same sequence again with what the first pass mapped still mapped: the steady state of a program
    # whose sizes repeat (no driver calls at all if every request finds a free run)
    before = c.sa.stats()
    second = allocator_churn(c.lib, c.rt, c.dev, c.sp, ops)
    after = c.sa.stats()
    second["handles_created"] = after["handles_created"] - before["handles_created"]
    second["served_from_mapped_runs"] = after["reuse_hits"] - before["reuse_hits"]
    second["large_allocs"] = after["large_allocs"] - before["large_allocs"]
    churn["sideaware_direct_calls"] = direct
    churn["sideaware_direct_calls_second_pass"] = second
    churn["driver_call_times"] = c.sa.driver_call_times()

    def released():
        c.lib.sideaware_release_unused()
        c.torch.cuda.synchronize()

    # First passes depend on what the driver did just before (the first arm after a large release has measured up to
    # 1.5 x slower than the same arm later), so the two allocators take turns and every run is kept.
    released()
    churn["cudaMallocAsync"] = allocator_churn(c.lib, c.rt, c.dev, c.sp, ops, arm="cudaMallocAsync")
    released()
    # the same first pass with the reference's own knob turned up (sideaware.cu:1475-1478): whenever the mapped set has to
    # grow it grows by 2 GiB more than asked for, so fewer calls pay for driver work and each of those pays more
    c.lib.sideaware_prealloc_config(1, 1024)
    roomy = allocator_churn(c.lib, c.rt, c.dev, c.sp, ops)
    roomy["prealloc_config"] = {"extra_required": 1, "extra_alloc": 1024}
    churn["sideaware_direct_calls_2GiB_headroom"] = roomy
    c.lib.sideaware_prealloc_config(1, 10)
    released()
    churn["sideaware_direct_calls_again"] = allocator_churn(c.lib, c.rt, c.dev, c.sp, ops)
    released()
    churn["cudaMallocAsync_again"] = allocator_churn(c.lib, c.rt, c.dev, c.sp, ops, arm="cudaMallocAsync")
    churn["first_pass_seconds"] = {
        "order": "sideaware, (second pass), cudaMallocAsync, sideaware with 2 GiB headroom, sideaware, cudaMallocAsync",
        "sideaware": [direct["seconds"], churn["sideaware_direct_calls_again"]["seconds"]],
        "sideaware_2GiB_headroom": [roomy["seconds"]],
        "cudaMallocAsync": [churn["cudaMallocAsync"]["seconds"], churn["cudaMallocAsync_again"]["seconds"]]}
    fp = churn["first_pass_seconds"]
    fp["best"] = {"sideaware": min(fp["sideaware"]), "cudaMallocAsync": min(fp["cudaMallocAsync"]),
                  "note": "driver calls on a shared host scatter by 2-3 x from one pass to the next whatever precedes them"}
    c.torch.cuda.synchronize()
    c.torch.cuda.empty_cache()
    # torch routes, each in a fresh process (the pluggable allocator has to be installed before the first allocation);
    # this process keeps only its context while they run
    churn["sideaware_via_torch_pluggable_allocator"] = run_script("allocator_churn_script.py", "pluggable", str(ops), timeout=1200)
    churn["torch_caching_allocator"] = run_script("allocator_churn_script.py", "torch", str(ops), timeout=1200)
    return churn


def run_ours(args, ranks):
    c = Ctx(args, ranks)
    torch, lib = c.torch, c.lib
    first = ranks.rank == 0
    value, worst_ms, roofline, memcpy_entry, clocks, launches = headline_memcpy(c)
    e2e = e2e_memcpy(c)
    limits = comparison = power = sweep = None
    if first:
        limits = pcie_limits(c)
        e2e["limit"] = dict(limits, bound=f"{2 * limits['both_directions_each_gbs']:.1f} GB/s for a step that moves its bytes "
                                         "host -> device and device -> host at the same time")
        comparison = comparison_memcpy(c)
        if ranks.world == 1 and args.power_seconds > 0:
            power = power_section(c)
        sweep = sweep_memcpy(c)
    c.free(c.src, MEMCPY_BYTES)
    c.free(c.dst, MEMCPY_BYTES)
    del c.seed_t
    torch.cuda.synchronize()

    rope, rope_entries = rope_section(c)
    functor, functor_entries = functor_section(c) if first else (None, [])
    roofline["kernels"] = [memcpy_entry] + rope_entries + functor_entries

    churn = ref_mem = ref_rope = None
    if first and ranks.world == 1:
        if args.churn_ops > 0:
            churn = churn_section(c)
        if not args.no_reference_library:
            lib.sideaware_release_unused()
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
            ref_mem, ref_rope = reference_gpu_library(c)
    if comparison is not None and ref_mem:
        comparison.update(ref_mem)

    if first:
        cpu = None
        if ranks.world == 1:
            threads = os.cpu_count() or 1
            v, _ = cpu_memcpy_gbs(MEMCPY_BYTES, 12, threads)
            v1, _ = cpu_memcpy_gbs(MEMCPY_BYTES, 4, 1)
            cpu = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                   "sample": f"12 x 1 GiB libc memcpy over {threads} threads (the reference has no CPU memcpy)",
                   "one_thread_gbs": v1, "rope": cpu_rope_reference()}
        # Key order matters to whoever keeps only the end of the line: the long sweep goes early, the summaries last.
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": ranks.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": worst_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic", "config": bench_config(ranks.world),
            "path": "sideaware_malloc_auto + sideaware_memcpy through the C ABI",
            "memcpy_sweep": sweep, "power": power,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches * ranks.world,
            "clocks": clocks, "topology": c.summary,
            "rope": rope, "functor": functor, "allocator_churn": churn,
            "memcpy_comparison": comparison, "rope_comparison": ref_rope,
        }
        print(json.dumps(line), flush=True)
    ranks.close()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-torch-compile", action="store_true", help="skip the torch.compile comparison lines")
    ap.add_argument("--churn-ops", type=int, default=10000,
                    help="allocator churn operations (N = 1 only; 0 = skip; 10000 is the benchmark configuration)")
    ap.add_argument("--no-reference-library", action="store_true",
                    help="skip the comparison runs of the reference's own GPU library (oracle/_ref, N = 1 only)")
    ap.add_argument("--power-seconds", type=float, default=2.0, help="length of each power sampling loop (0 = skip)")
    ap.add_argument("--e2e-piece-mib", type=int, default=64, choices=[4, 8, 16, 32, 64, 128, 256],
                    help="piece size of the pipelined end-to-end step (upload / kernel / download overlap piece by piece)")
    ap.add_argument("--check-ranks", action="store_true",
                    help="exercise only the rank plumbing (barrier, max/sum over ranks, rank 0 prints); needs no GPU")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    ranks = Ranks(args.gpus)
    if args.check_ranks:
        # every rank pretends to have moved (rank + 1) GB in (rank + 1) ms; the job value uses the slowest rank
        ranks.barrier()
        worst = ranks.max(float(ranks.rank + 1))
        total = ranks.sum(float(ranks.rank + 1))
        if ranks.rank == 0:
            print(json.dumps({"check_ranks": True, "world": ranks.world, "max_ms": worst, "sum_gb": total,
                              "value": total / (worst * 1e-3)}), flush=True)
        ranks.close()
        return 0
    if args.impl == "reference":
        return run_reference(args, ranks)
    return run_ours(args, ranks)


if __name__ == "__main__":
    sys.exit(main())
