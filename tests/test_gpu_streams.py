"""Launches on several streams at once stay exact.

Every launch works from three ticket counters in device memory.  The counters of a launch must
not be shared with a launch that runs at the same time, whichever streams the two are on and
however long one of them takes: a long copy on one stream while another stream issues hundreds
of short ones, many short launches queued behind a long one on the same stream, and more
streams than one block of counters serves.  All checks are bit-exact comparisons with the
source bytes (the reference's own criterion for copies, test.py:290-294).
"""
import ctypes

import numpy as np
import pytest

from tests import cuda_helpers as ch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sa():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import l2_torch_alloc_b200 as pkg
    s = pkg.SideAware()
    yield s
    s.set_placement("aware")
    s.lib.sideaware_set_memcpy_engine(1)


def make_streams(n):
    rt = ch.cudart()
    rt.cudaStreamCreate.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    rt.cudaStreamDestroy.argtypes = [ctypes.c_void_p]
    out = []
    for _ in range(n):
        s = ctypes.c_void_p()
        ch.check(rt.cudaStreamCreate(ctypes.byref(s)), "cudaStreamCreate")
        out.append(s)
    return out


def destroy_streams(streams):
    for s in streams:
        ch.check(ch.cudart().cudaStreamDestroy(s), "cudaStreamDestroy")


def device_bytes(sa, nbytes, seed):
    """A side-aware buffer filled with seeded random bytes, and the bytes."""
    host = np.random.default_rng(seed).integers(0, 256, size=nbytes, dtype=np.uint8)
    ptr = sa.malloc(nbytes)
    ch.h2d(ptr, host)
    return ptr, host


@pytest.mark.parametrize("engine", [1, 0])
def test_long_copy_beside_hundreds_of_short_ones(sa, engine):
    sa.lib.sideaware_set_memcpy_engine(engine)
    dev = 0
    errors_before = sa.error_count()
    big = 1 << 30
    small = 8 << 20
    n_small_streams, n_small = 3, 400
    streams = make_streams(1 + n_small_streams)
    big_src, big_host = device_bytes(sa, big, 1)
    big_dst = sa.malloc(big)
    ch.memset(big_dst, 0, big)
    small_src, small_host, small_dst = [], [], []
    for k in range(n_small_streams):
        p, h = device_bytes(sa, small, 10 + k)
        small_src.append(p)
        small_host.append(h)
        # ping-pong pair: the data goes back and forth, so a lost chunk in ANY launch shows at the end
        d = [sa.malloc(small), sa.malloc(small)]
        ch.memset(d[0], 0, small)
        ch.memset(d[1], 0, small)
        small_dst.append(d)
    ch.sync()
    lib = sa.lib
    for rep in range(4):  # the long copies keep stream 0 busy for milliseconds
        lib.sideaware_memcpy(big_dst, big_src, big, dev, streams[0])
    for i in range(n_small):
        for k in range(n_small_streams):
            src = small_src[k] if i == 0 else small_dst[k][(i - 1) & 1]
            lib.sideaware_memcpy(small_dst[k][i & 1], src, small, dev, streams[1 + k])
    for rep in range(2):
        lib.sideaware_memcpy(big_dst, big_src, big, dev, streams[0])
    ch.sync()
    assert sa.error_count() == errors_before, sa.last_error()
    assert np.array_equal(ch.d2h(big_dst, big), big_host)
    for k in range(n_small_streams):
        assert np.array_equal(ch.d2h(small_dst[k][(n_small - 1) & 1], small), small_host[k]), f"stream {k}"
    assert sa.stats()["kernel_wait_timeouts"] == 0
    for p in [big_src, big_dst] + small_src + [x for d in small_dst for x in d]:
        sa.free(p)
    destroy_streams(streams)
    sa.lib.sideaware_set_memcpy_engine(1)


def test_many_short_launches_queued_behind_a_long_one(sa):
    """300 tiny copies wait on one stream behind 1 GiB copies: more launches than a stream's ring
    of counters has slots, all issued before the first of them can run."""
    dev = 0
    errors_before = sa.error_count()
    big = 1 << 30
    tiny = 64 << 10
    n = 300
    (stream,) = make_streams(1)
    big_src, big_host = device_bytes(sa, big, 2)
    big_dst = sa.malloc(big)
    src, host = device_bytes(sa, tiny * n, 3)
    dst = sa.malloc(tiny * n)
    ch.memset(dst, 0, tiny * n)
    ch.sync()
    lib = sa.lib
    for rep in range(3):
        lib.sideaware_memcpy(big_dst, big_src, big, dev, stream)
    for i in range(n):
        lib.sideaware_memcpy(dst + i * tiny, src + i * tiny, tiny, dev, stream)
    ch.sync()
    assert sa.error_count() == errors_before, sa.last_error()
    assert np.array_equal(ch.d2h(dst, tiny * n), host)
    assert np.array_equal(ch.d2h(big_dst, big), big_host)
    for p in (big_src, big_dst, src, dst):
        sa.free(p)
    destroy_streams([stream])


def test_more_streams_than_one_block_of_rings(sa):
    """150 streams alive at once (one block of counters serves 64), two rounds of copies on each."""
    dev = 0
    errors_before = sa.error_count()
    n_streams = 150
    piece = 256 << 10
    streams = make_streams(n_streams)
    src, host = device_bytes(sa, piece * n_streams, 4)
    mid = sa.malloc(piece * n_streams)
    dst = sa.malloc(piece * n_streams)
    ch.memset(mid, 0, piece * n_streams)
    ch.memset(dst, 0, piece * n_streams)
    ch.sync()
    lib = sa.lib
    for k, s in enumerate(streams):
        lib.sideaware_memcpy(mid + k * piece, src + k * piece, piece, dev, s)
    for k, s in enumerate(streams):
        lib.sideaware_memcpy(dst + k * piece, mid + k * piece, piece, dev, s)
    ch.sync()
    assert sa.error_count() == errors_before, sa.last_error()
    assert np.array_equal(ch.d2h(dst, piece * n_streams), host)
    assert sa.stats()["kernel_wait_timeouts"] == 0
    for p in (src, mid, dst):
        sa.free(p)
    destroy_streams(streams)


def test_block_reused_on_another_stream_waits_for_its_previous_user(sa):
    """A block freed on stream A while A still has copies into it queued, then handed to stream B: B's
    work on it must run after A's (the allocator orders the streams on the device, sideaware.cu:1209-1214
    blocks the host instead).  B writes other bytes; they must be what is there in the end."""
    dev = 0
    n = 256 << 20
    a_stream, b_stream = make_streams(2)
    src1, _ = device_bytes(sa, n, 21)
    src2, host2 = device_bytes(sa, n, 22)
    ch.sync()
    for attempt in range(3):
        x = sa.malloc(n, a_stream)
        for _ in range(24):                      # ~2 ms of copies into x queued on A
            sa.lib.sideaware_memcpy(x, src1, n, dev, a_stream)
        sa.free(x, a_stream)
        y = sa.malloc(n, b_stream)
        assert y == x, "the freed block is the best fit for an equal request"
        sa.lib.sideaware_memcpy(y, src2, n, dev, b_stream)
        ch.check(ch.cudart().cudaStreamSynchronize(b_stream), "cudaStreamSynchronize")
        got = ch.d2h(y, n)
        ch.sync()
        assert np.array_equal(got, host2), f"attempt {attempt}: the other stream's queued copies ran after the new owner's"
        sa.free(y, b_stream)
    for p in (src1, src2):
        sa.free(p)
    destroy_streams([a_stream, b_stream])


def test_more_streams_than_rings_can_ever_be_made(sa):
    """1 100 streams, each used once: beyond 1 024 stream handles the rings are handed out afresh (after a
    device-wide wait, so no counter is in use).  Results stay exact and nothing is recorded as an error."""
    dev = 0
    errors_before = sa.error_count()
    n_streams = 1100
    piece = 64 << 10
    streams = make_streams(n_streams)
    src, host = device_bytes(sa, piece * n_streams, 6)
    dst = sa.malloc(piece * n_streams)
    ch.memset(dst, 0, piece * n_streams)
    ch.sync()
    for k, s in enumerate(streams):
        sa.lib.sideaware_memcpy(dst + k * piece, src + k * piece, piece, dev, s)
    ch.sync()
    assert sa.error_count() == errors_before, sa.last_error()
    assert np.array_equal(ch.d2h(dst, piece * n_streams), host)
    assert sa.stats()["kernel_wait_timeouts"] == 0
    for p in (src, dst):
        sa.free(p)
    destroy_streams(streams)


@pytest.mark.parametrize("engine", [1, 0])
def test_launches_recorded_in_a_cuda_graph_can_be_replayed(sa, engine):
    """A launch leaves its ticket counters as it found them (the last block to finish rewinds them), so kernels
    recorded in a CUDA graph give the right result every time the graph is replayed: a copy and an in-place RoPE
    captured once, replayed four times on fresh data."""
    import torch
    from oracle import oracle
    sa.lib.sideaware_set_memcpy_engine(engine)
    n = (40 << 20) + 4096 + 16
    src = torch.zeros(n, dtype=torch.uint8, device="cuda")
    dst = torch.zeros(n, dtype=torch.uint8, device="cuda")
    B, T, Nq, Nkv, HS = 2, 128, 8, 2, 64
    x_host = np.random.default_rng(5).uniform(-1, 1, size=(B, T, Nq + 2 * Nkv, HS)).astype(np.float32)
    table = oracle.freqs_cis(HS, T, 10000.0, 0)
    want = torch.from_numpy(oracle.rope_forward_f32(x_host, table, B, T, Nq, Nkv, HS)).cuda()
    x0 = torch.from_numpy(x_host).cuda()
    x = x0.clone()
    tab = torch.from_numpy(table).cuda()
    # once outside the capture: first use of a stream's counters and of the kernels' attributes
    sa.memcpy(dst, src)
    sa.rope_forward(x, tab, Nq, Nkv)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sa.memcpy(dst, src)
        sa.rope_forward(x, tab, Nq, Nkv)
    gen = torch.Generator(device="cuda").manual_seed(11)
    for _ in range(4):
        src.copy_(torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=gen))
        dst.zero_()
        x.copy_(x0)
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(dst, src)
        assert torch.equal(x, want)
    assert sa.error_count() == 0 or "ticket" not in sa.last_error()
