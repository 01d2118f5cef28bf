"""Several GPUs driven from ONE process: every device gets its own context (its own discovery,
pools, ticket slots and JIT cache), selected by the `device` argument while the caller's current
device stays what it was (the reference keys everything by device and wraps calls in
ScopedSetDevice, sideaware.cu:610-625, :741-769).  Skipped on a single-GPU machine."""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    assert torch.cuda.is_available()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import l2_torch_alloc_b200 as pkg
    return pkg.SideAware(), torch


def test_each_device_has_its_own_context(env):
    sa, torch = env
    lib = sa.lib
    torch.cuda.set_device(0)
    n = 48 << 20
    results = {}
    for dev in (1, 0):
        a = lib.sideaware_malloc_auto(n, dev, None)
        b = lib.sideaware_malloc_auto(n, dev, None)
        assert a and b and a % (2 << 20) == 0
        src = torch.randint(0, 2**31 - 1, (n // 4,), dtype=torch.int32, device=f"cuda:{dev}")
        back = torch.zeros_like(src)
        stream = torch.cuda.current_stream(dev).cuda_stream
        lib.sideaware_memcpy(a, src.data_ptr(), n, dev, stream)
        lib.sideaware_memcpy(b, a, n, dev, stream)
        lib.sideaware_memcpy(back.data_ptr(), b, n, dev, stream)
        torch.cuda.synchronize(dev)
        assert torch.equal(back, src), f"copy on device {dev} is not exact"
        assert torch.cuda.current_device() == 0, "the caller's current device must be restored"
        results[dev] = (a, b)
    assert sa.error_count() == 0, sa.last_error()
    # per-device metadata is reachable by making the device current
    summaries = []
    for dev in (0, 1):
        torch.cuda.set_device(dev)
        summaries.append(sa.summary())
        st = sa.stats()
        assert st["bytes_mapped_live"] == 2 * n, f"device {dev} should hold exactly its own two blocks"
    torch.cuda.set_device(0)
    assert summaries[0][0] == summaries[1][0] == 148 or summaries[0][0] > 0
    for dev in (0, 1):
        for p in results[dev]:
            lib.sideaware_free_auto(p, n, dev, None)
    for dev in (0, 1):
        torch.cuda.set_device(dev)
        assert sa.stats()["bytes_mapped_live"] == 0
    torch.cuda.set_device(0)


def test_functor_ids_are_shared_and_compiled_per_device(env):
    sa, torch = env
    from l2_torch_alloc_b200 import functors
    kid = sa.create_kernel(functors.MEMCPY + "// multi-device test\n")
    for dev in (0, 1):
        with torch.cuda.device(dev):
            src = torch.randint(0, 1000, (1 << 20,), dtype=torch.int32, device=f"cuda:{dev}")
            dst = torch.zeros_like(src)
            sa.one_to_one(kid, dst, src)
            torch.cuda.synchronize(dev)
            assert torch.equal(dst, src)
            assert sa.stats()["jit_compiles"] >= 1, "each device compiles its own module"


def test_rope_on_second_device_matches_oracle(env):
    sa, torch = env
    from oracle import oracle
    B, T, Nq, Nkv, HS = 2, 128, 8, 2, 64
    x = np.random.default_rng(5).uniform(-1, 1, (B, T, Nq + 2 * Nkv, HS)).astype(np.float32)
    table = oracle.freqs_cis(HS, T, 10000.0, 0)
    want = oracle.rope_forward_f32(x, table, B, T, Nq, Nkv, HS)
    torch.cuda.set_device(0)
    tx = torch.from_numpy(x).to("cuda:1")
    tt = torch.from_numpy(table).to("cuda:1")
    sa.rope_forward(tx, tt, Nq, Nkv)  # device taken from the tensor, current device is 0
    torch.cuda.synchronize(1)
    assert tx.cpu().numpy().tobytes() == want.tobytes()
    assert torch.cuda.current_device() == 0


def test_devices_in_parallel_threads(env):
    sa, torch = env
    lib = sa.lib
    errors = []

    def worker(dev):
        try:
            torch.cuda.set_device(dev)
            n = 32 << 20
            for i in range(10):
                a = lib.sideaware_malloc_auto(n + i * (2 << 20), dev, None)
                b = lib.sideaware_malloc_auto(n + i * (2 << 20), dev, None)
                src = torch.full((n // 4,), dev * 100 + i, dtype=torch.int32, device=f"cuda:{dev}")
                out = torch.zeros_like(src)
                s = torch.cuda.current_stream(dev).cuda_stream
                lib.sideaware_memcpy(a, src.data_ptr(), n, dev, s)
                lib.sideaware_memcpy(b, a, n, dev, s)
                lib.sideaware_memcpy(out.data_ptr(), b, n, dev, s)
                torch.cuda.synchronize(dev)
                assert torch.equal(out, src)
                lib.sideaware_free_auto(a, n, dev, None)
                lib.sideaware_free_auto(b, n, dev, None)
        except Exception as e:  # noqa: BLE001
            errors.append((dev, e))

    threads = [threading.Thread(target=worker, args=(d,)) for d in (0, 1)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert sa.error_count() == 0, sa.last_error()
