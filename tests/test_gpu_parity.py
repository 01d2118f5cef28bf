"""Parity of the CUDA path with the oracle, through the C ABI, on a B200.

memcpy: bit-exact against the source (the reference's own criterion, test.py:290-294),
over aligned/unaligned bases, ragged sizes, the reference's test shapes, every
placement mode, with canary pages around the destination.
RoPE: bit-exact against the C oracle (example_llmc_rope.cu:54-86 restated) for fp32
and bf16, MHA and grouped-query shapes, plus the golden vectors made by the compiled
reference.  Tolerances allowed by the task: 1e-6 relative (fp32), 1 bf16 ulp; the
kernels meet 0.
silu-mul functor: within 1 bf16 ulp of the oracle (expf differs between libm and GPU).
"""
import os

import numpy as np
import pytest

from oracle import oracle
from tests import cuda_helpers as ch

pytestmark = pytest.mark.gpu

PLACEMENTS = ["aware", "unaware", "wrong"]


@pytest.fixture(scope="module")
def sa():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import l2_torch_alloc_b200 as pkg
    s = pkg.SideAware()
    n, s0, s1, m, h = s.summary()
    assert n > 0
    yield s
    s.set_placement("aware")


def rng_bytes(seed, n):
    return np.random.default_rng(seed).integers(0, 256, size=n, dtype=np.uint8)


# ---------------------------------------------------------------------------
# memcpy
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("nbytes", [16, 48, 4096, 4112, 8192, 12432, 65536 + 16, (1 << 20) + 4096 + 32,
                                    1000 * 1000 * 2, 1000 * 1000 * 8, 10000 * 1000 * 4, (64 << 20)])
@pytest.mark.parametrize("placement", PLACEMENTS)
@pytest.mark.parametrize("engine", [0, 1])
def test_memcpy_bit_exact(sa, nbytes, placement, engine):
    """engine 0 = 128-bit vector loads/stores, 1 = bulk copies staged through shared memory"""
    sa.set_placement(placement)
    sa.lib.sideaware_set_memcpy_engine(engine)
    src_host = rng_bytes(0xB200 + 2, nbytes)
    src = ch.Guarded(sa, nbytes)
    dst = ch.Guarded(sa, nbytes)
    ch.h2d(src.ptr, src_host)
    ch.memset(dst.ptr, 0, dst.payload_bytes)
    sa.memcpy_ptr(dst.ptr, src.ptr, nbytes)
    ch.sync()
    got = ch.d2h(dst.ptr, dst.payload_bytes)
    assert np.array_equal(got[:nbytes], src_host)
    assert not got[nbytes:].any(), "bytes past the end of the copy were written"
    assert dst.canaries_intact() and src.canaries_intact()
    assert sa.stats()["kernel_wait_timeouts"] == 0
    sa.lib.sideaware_set_memcpy_engine(1)
    src.free()
    dst.free()


@pytest.mark.parametrize("src_off,dst_off", [(16, 16), (4096, 0), (4112, 8176), (0, 2 << 20), (8192 + 48, 32)])
def test_memcpy_unaligned_bases(sa, src_off, dst_off):
    """Offsets inside an allocation: chunks are anchored to absolute 8 KiB addresses of the source."""
    sa.set_placement("aware")
    nbytes = (3 << 20) + 4096 * 3 + 160
    src_host = rng_bytes(11, nbytes)
    src = ch.Guarded(sa, nbytes + (4 << 20))
    dst = ch.Guarded(sa, nbytes + (4 << 20))
    ch.memset(dst.ptr, 0, dst.payload_bytes)
    ch.h2d(src.ptr + src_off, src_host)
    sa.memcpy_ptr(dst.ptr + dst_off, src.ptr + src_off, nbytes)
    ch.sync()
    got = ch.d2h(dst.ptr, dst.payload_bytes)
    assert np.array_equal(got[dst_off:dst_off + nbytes], src_host)
    assert not got[:dst_off].any() and not got[dst_off + nbytes:].any()
    assert dst.canaries_intact()
    src.free()
    dst.free()


def test_memcpy_plain_cudamalloc_memory(sa):
    """Memory that did not come from the side-aware allocator: correct, just not placed."""
    nbytes = (5 << 20) + 16
    src_host = rng_bytes(5, nbytes)
    a, b = ch.cuda_malloc(nbytes + 256), ch.cuda_malloc(nbytes + 256)
    ch.h2d(a + 32, src_host)
    ch.memset(b, 0, nbytes + 256)
    sa.memcpy_ptr(b + 48, a + 32, nbytes)
    ch.sync()
    got = ch.d2h(b, nbytes + 256)
    assert np.array_equal(got[48:48 + nbytes], src_host)
    assert not got[:48].any() and not got[48 + nbytes:].any()
    ch.cuda_free(a)
    ch.cuda_free(b)


def test_memcpy_rejects_misuse_without_touching_memory(sa):
    dst = ch.Guarded(sa, 1 << 20)
    ch.memset(dst.ptr, 0, 1 << 20)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        sa.memcpy_ptr(dst.ptr, dst.ptr + 4096, 100)
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        sa.memcpy_ptr(dst.ptr + 8, dst.ptr + 4096, 160)
    sa.memcpy_ptr(dst.ptr, dst.ptr + 4096, 0)  # empty copy is a no-op (sideaware.cu:1366)
    ch.sync()
    assert not ch.d2h(dst.ptr, 1 << 20).any()
    dst.free()


@pytest.mark.parametrize("nbytes", [16, 4096, 4112, 12432, (1 << 20) + 4096 + 32, 10000 * 1000 * 4, (96 << 20) + 8192])
@pytest.mark.parametrize("placement", ["aware", "wrong"])
def test_memcpy_bulk_engine_bit_exact(sa, nbytes, placement):
    """Engine 1: bulk asynchronous copies staged through shared memory; same contract, same bytes."""
    sa.set_placement(placement)
    sa.lib.sideaware_set_memcpy_engine(1)
    try:
        src_host = rng_bytes(0xB200 + 7, nbytes)
        src = ch.Guarded(sa, nbytes + 8192)
        dst = ch.Guarded(sa, nbytes + 8192)
        for off in (0, 4096 + 16):
            ch.h2d(src.ptr + off, src_host)
            ch.memset(dst.ptr, 0, dst.payload_bytes)
            sa.memcpy_ptr(dst.ptr + off, src.ptr + off, nbytes)
            ch.sync()
            got = ch.d2h(dst.ptr, dst.payload_bytes)
            assert np.array_equal(got[off:off + nbytes], src_host)
            assert not got[:off].any() and not got[off + nbytes:].any()
        assert dst.canaries_intact() and src.canaries_intact()
        assert sa.stats()["kernel_wait_timeouts"] == 0
        src.free()
        dst.free()
    finally:
        sa.lib.sideaware_set_memcpy_engine(1)
        sa.set_placement("aware")


def test_memcpy_large_round_trip_property(sa):
    """1 GiB (the benchmark size): copy there and back, compare 64-bit checksums of 16 MiB slabs."""
    import torch
    nbytes = 1 << 30
    g = torch.Generator(device="cuda").manual_seed(0xB200 + 2)
    src_t = torch.randint(0, 2**31 - 1, (nbytes // 4,), dtype=torch.int32, device="cuda", generator=g)
    a = sa.malloc(nbytes)
    b = sa.malloc(nbytes)
    ch.memset(b, 0, nbytes)
    sa.memcpy_ptr(a, src_t.data_ptr(), nbytes)      # torch memory -> side-aware block
    sa.memcpy_ptr(b, a, nbytes)                      # side-aware -> side-aware (the benchmark copy)
    back = torch.empty_like(src_t)
    sa.memcpy_ptr(back.data_ptr(), b, nbytes)        # and back
    torch.cuda.synchronize()
    assert torch.equal(back, src_t)
    sums_src = src_t.view(-1, 4 << 20).to(torch.int64).sum(dim=1)
    sums_back = back.view(-1, 4 << 20).to(torch.int64).sum(dim=1)
    assert torch.equal(sums_src, sums_back)
    sa.free(a)
    sa.free(b)


# ---------------------------------------------------------------------------
# RoPE
# ---------------------------------------------------------------------------
def run_rope(sa, x_host, table, B, T, Nq, Nkv, HS, bf16, offset=0):
    nbytes = x_host.nbytes
    buf = ch.Guarded(sa, nbytes + offset)
    tab = ch.cuda_malloc(table.nbytes)
    ch.memset(buf.ptr, 0, buf.payload_bytes)
    ch.h2d(buf.ptr + offset, x_host)
    ch.h2d(tab, table)
    sa.rope_forward_ptr(buf.ptr + offset, tab, B, T, Nq, Nkv, HS, bf16)
    ch.sync()
    out = ch.d2h(buf.ptr + offset, nbytes, x_host.dtype).reshape(x_host.shape)
    assert buf.canaries_intact()
    tail = ch.d2h(buf.ptr, buf.payload_bytes)
    assert not tail[offset + nbytes:].any() and not tail[:offset].any()
    buf.free()
    ch.cuda_free(tab)
    return out


@pytest.fixture(params=[0, 1], ids=["vector", "bulk"])
def rope_engine(request, sa):
    """Both RoPE engines (registers / staged through shared memory by bulk copies) must give the same bits."""
    default = sa.lib.sideaware_get_rope_engine()
    sa.lib.sideaware_set_rope_engine(request.param)
    yield request.param
    sa.lib.sideaware_set_rope_engine(default)


ROPE_SHAPES = [  # B, T, Nq, Nkv, HS
    (4, 1024, 12, 12, 64),   # the CPU benchmark config of the reference function
    (2, 64, 32, 32, 128),    # the reference example's head geometry (example_llmc_rope.cu:246-249)
    (2, 160, 32, 8, 128),    # Llama-3-8B heads, short sequence
    (3, 33, 5, 2, 32),       # odd head counts, rows shorter than a 4 KiB chunk
    (1, 7, 1, 1, 8),         # tiny: several rows per chunk
    (2, 50, 6, 3, 48),       # head size that is not a power of two
    (2, 40, 20, 6, 48),      # the same with rows longer than a chunk (the staged engine's two-run case)
    (1, 300, 3, 1, 256),     # rows of exactly 5 KiB fp32 / 2.5 KiB bf16: run boundaries at odd places
]


@pytest.mark.parametrize("shape", ROPE_SHAPES)
@pytest.mark.parametrize("placement", ["aware", "wrong"])
def test_rope_f32_bit_exact(sa, shape, placement, rope_engine):
    sa.set_placement(placement)
    B, T, Nq, Nkv, HS = shape
    rng = np.random.default_rng(0xB200 + 1)
    x = rng.uniform(-1, 1, size=(B, T, Nq + 2 * Nkv, HS)).astype(np.float32)
    table = oracle.freqs_cis(HS, T, 10000.0, 1)
    want = oracle.rope_forward_f32(x, table, B, T, Nq, Nkv, HS)
    got = run_rope(sa, x, table, B, T, Nq, Nkv, HS, bf16=False)
    assert got.tobytes() == want.tobytes()
    # stated tolerance of the task, for the record: 1e-6 relative
    assert np.allclose(got, want, rtol=1e-6, atol=0)


@pytest.mark.parametrize("shape", ROPE_SHAPES)
def test_rope_bf16_bit_exact(sa, shape, rope_engine):
    sa.set_placement("aware")
    B, T, Nq, Nkv, HS = shape
    rng = np.random.default_rng(0xB200 + 3)
    x = oracle.f32_to_bf16(rng.standard_normal(size=(B, T, Nq + 2 * Nkv, HS)).astype(np.float32))
    table = oracle.freqs_cis(HS, T, 500000.0, 0)
    want = oracle.rope_forward_bf16(x, table, B, T, Nq, Nkv, HS)
    got = run_rope(sa, x, table, B, T, Nq, Nkv, HS, bf16=True)
    assert oracle.ulp_diff_bf16(got, want).max() <= 1  # the tolerance the task allows
    assert got.tobytes() == want.tobytes()              # and what the kernel achieves
    assert np.array_equal(got[:, :, Nq + Nkv:], x[:, :, Nq + Nkv:]), "V heads must be untouched"


def test_rope_unaligned_base(sa, rope_engine):
    for B, T, Nq, Nkv, HS in ((2, 96, 8, 2, 64), (2, 40, 16, 4, 128)):  # rows shorter and longer than a chunk
        rng = np.random.default_rng(3)
        x = rng.uniform(-1, 1, size=(B, T, Nq + 2 * Nkv, HS)).astype(np.float32)
        table = oracle.freqs_cis(HS, T, 10000.0, 0)
        want = oracle.rope_forward_f32(x, table, B, T, Nq, Nkv, HS)
        for off in (16, 4096 + 48, 8192 - 16):
            got = run_rope(sa, x, table, B, T, Nq, Nkv, HS, bf16=False, offset=off)
            assert got.tobytes() == want.tobytes()


def test_rope_matches_reference_golden_vectors(sa, golden_dir, rope_engine):
    g = np.load(os.path.join(golden_dir, "rope_small_f32.npz"))
    B, T, NH, HS = (int(v) for v in g["shape"])
    for scaled in (0, 1):
        got = run_rope(sa, g["inp"], g[f"table_s{scaled}"], B, T, NH, NH, HS, bf16=False)
        assert got.tobytes() == g[f"out_s{scaled}"].tobytes()
    g = np.load(os.path.join(golden_dir, "rope_gqa_bf16.npz"))
    B, T, Nq, Nkv, HS = (int(v) for v in g["shape"])
    got = run_rope(sa, g["inp_bf16"], g["table"], B, T, Nq, Nkv, HS, bf16=True)
    assert got.tobytes() == g["out_bf16"].tobytes()


@pytest.mark.parametrize("shape", [(2, 64, 32, 32, 128), (2, 160, 32, 8, 128), (3, 33, 5, 2, 32), (2, 50, 6, 3, 48)])
def test_rope_backward_matches_oracle(sa, shape, golden_dir, rope_engine):
    """In-place backward pass: equal to the oracle (example_llmc_rope.cu:166-195 restated); values compared
    as numbers because the reference adds into zeros, which turns -0 into +0."""
    B, T, Nq, Nkv, HS = shape
    rng = np.random.default_rng(0xB200 + 6)
    table = oracle.freqs_cis(HS, T, 10000.0, 1)
    g = rng.uniform(-1, 1, size=(B, T, Nq + 2 * Nkv, HS)).astype(np.float32)
    want = oracle.rope_backward_f32(g, table, B, T, Nq, Nkv, HS)
    nbytes = g.nbytes
    buf = ch.Guarded(sa, nbytes)
    tab = ch.cuda_malloc(table.nbytes)
    ch.h2d(buf.ptr, g)
    ch.h2d(tab, table)
    sa.rope_backward_ptr(buf.ptr, tab, B, T, Nq, Nkv, HS, False)
    ch.sync()
    got = ch.d2h(buf.ptr, nbytes, np.float32).reshape(g.shape)
    assert np.array_equal(got, want)
    # forward then backward is the identity up to rounding
    ch.h2d(buf.ptr, g)
    sa.rope_forward_ptr(buf.ptr, tab, B, T, Nq, Nkv, HS, False)
    sa.rope_backward_ptr(buf.ptr, tab, B, T, Nq, Nkv, HS, False)
    ch.sync()
    back = ch.d2h(buf.ptr, nbytes, np.float32).reshape(g.shape)
    assert np.allclose(back, g, rtol=0, atol=2e-6)
    # bf16 storage
    gb = oracle.f32_to_bf16(g)
    wantb = oracle.rope_backward_bf16(gb, table, B, T, Nq, Nkv, HS)
    ch.h2d(buf.ptr, gb)
    sa.rope_backward_ptr(buf.ptr, tab, B, T, Nq, Nkv, HS, True)
    ch.sync()
    gotb = ch.d2h(buf.ptr, gb.nbytes, np.uint16).reshape(gb.shape)
    assert np.array_equal(oracle.bf16_to_f32(gotb), oracle.bf16_to_f32(wantb))
    assert buf.canaries_intact()
    buf.free()
    ch.cuda_free(tab)
    # the reference's own backward output on its tiny case
    gold = np.load(os.path.join(golden_dir, "rope_small_f32.npz"))
    Bg, Tg, NHg, HSg = (int(v) for v in gold["shape"])
    buf = ch.Guarded(sa, gold["out_s1"].nbytes)
    tab = ch.cuda_malloc(gold["table_s1"].nbytes)
    ch.h2d(buf.ptr, gold["out_s1"])
    ch.h2d(tab, gold["table_s1"])
    sa.rope_backward_ptr(buf.ptr, tab, Bg, Tg, NHg, NHg, HSg, False)
    ch.sync()
    assert np.array_equal(ch.d2h(buf.ptr, gold["out_s1"].nbytes, np.float32).reshape(gold["dinp_s1"].shape), gold["dinp_s1"])
    buf.free()
    ch.cuda_free(tab)


@pytest.mark.parametrize("case", [(64, 1024, 10000.0, 0), (64, 1024, 10000.0, 1), (128, 8192, 500000.0, 0),
                                  (128, 8192, 500000.0, 1), (2, 5, 10000.0, 0), (48, 333, 1000000.0, 1)])
def test_rope_table_made_on_the_gpu(sa, case, golden_dir):
    """cos/sin table made on the GPU against precompute_freqs_cis (example_llmc_rope.cu:19-52, restated
    in the oracle and, for the golden case, as written out by the compiled reference).  Tolerance: 1 fp32
    ulp per entry (the task allows 1e-6 relative); the frequencies are bit-identical, the difference is
    fp64 sincos rounded once on the GPU against libm's cosf/sinf (within 0.56 ulp), seen in ~1 % of entries."""
    dim, end, theta, scaled = case
    want = np.asarray(oracle.freqs_cis(dim, end, theta, scaled), dtype=np.float32).reshape(-1)
    nbytes = want.nbytes
    tab = ch.cuda_malloc(nbytes + 256)
    ch.memset(tab, 0xEE, nbytes + 256)
    sa.rope_precompute_freqs_ptr(tab, dim, end, theta, bool(scaled))
    ch.sync()
    raw = ch.d2h(tab, nbytes + 256)
    ch.cuda_free(tab)
    assert (raw[nbytes:] == 0xEE).all(), "wrote past the end of the table"
    got = raw[:nbytes].view(np.float32)
    ulps = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
    # +0 / -0 and values straddling zero do not occur: cos and sin of these angles are never that small
    assert ulps.max() <= 1, f"max distance {ulps.max()} ulp"
    if got.size >= 10000:
        assert (ulps > 0).mean() <= 0.03
    assert got[0] == 1.0 and got[1] == 0.0  # t = 0


@pytest.mark.parametrize("scaled", [0, 1])
def test_rope_table_against_golden_table_of_the_compiled_reference(sa, scaled, golden_dir):
    g = np.load(os.path.join(golden_dir, "rope_small_f32.npz"))
    want = g[f"table_s{scaled}"].astype(np.float32).reshape(-1)  # dim 8, 5 positions, theta 10000
    tab = ch.cuda_malloc(want.nbytes)
    sa.rope_precompute_freqs_ptr(tab, 8, 5, 10000.0, bool(scaled))
    ch.sync()
    got = ch.d2h(tab, want.nbytes).view(np.float32)
    ch.cuda_free(tab)
    assert np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64)).max() <= 1


def test_rope_with_gpu_made_table_within_tolerance(sa):
    """The whole path on the GPU (table, then rotation) against the reference's CPU path with its own table:
    1e-6 relative to the magnitude of the pair, the tolerance the task states for fp32."""
    B, T, Nq, Nkv, HS = 2, 256, 8, 2, 64
    rng = np.random.default_rng(0xB200 + 7)
    x = rng.uniform(-1, 1, size=(B, T, Nq + 2 * Nkv, HS)).astype(np.float32)
    table = oracle.freqs_cis(HS, T, 10000.0, 0)
    want = oracle.rope_forward_f32(x, table, B, T, Nq, Nkv, HS)
    buf = ch.Guarded(sa, x.nbytes)
    tab = ch.cuda_malloc(table.nbytes)
    ch.h2d(buf.ptr, x)
    sa.rope_precompute_freqs_ptr(tab, HS, T, 10000.0, False)
    sa.rope_forward_ptr(buf.ptr, tab, B, T, Nq, Nkv, HS, False)
    ch.sync()
    got = ch.d2h(buf.ptr, x.nbytes).view(np.float32).reshape(x.shape)
    assert buf.canaries_intact()
    buf.free()
    ch.cuda_free(tab)
    pairs = x.reshape(B, T, -1, HS // 2, 2)
    mag = np.sqrt((pairs.astype(np.float64) ** 2).sum(-1, keepdims=True)).repeat(2, -1).reshape(x.shape)
    assert (np.abs(got.astype(np.float64) - want) <= 1e-6 * mag + 1e-12).all()
    # V heads untouched
    assert got[:, :, Nq + Nkv:].tobytes() == x[:, :, Nq + Nkv:].tobytes()


def test_rope_table_rejects_bad_arguments(sa):
    tab = ch.cuda_malloc(4096)
    before = sa.error_count()
    for dim, end, theta in [(0, 4, 1e4), (63, 4, 1e4), (2048, 4, 1e4), (64, 0, 1e4), (64, 4, 0.0)]:
        with pytest.raises(RuntimeError):
            sa.rope_precompute_freqs_ptr(tab, dim, end, theta, False)
    with pytest.raises(RuntimeError):
        sa.rope_precompute_freqs_ptr(0, 64, 4, 1e4, False)
    assert sa.error_count() == before + 6
    ch.cuda_free(tab)


def test_rope_rejects_bad_shapes(sa):
    buf = sa.malloc(8 << 20)
    with pytest.raises(RuntimeError):
        sa.rope_forward_ptr(buf, buf, 1, 4, 2, 2, 6, False)   # 6 floats are not whole 16-byte vectors
    with pytest.raises(RuntimeError):
        sa.rope_forward_ptr(buf, buf, 0, 4, 2, 2, 64, False)
    sa.free(buf)


def test_rope_llama3_shape_properties(sa, rope_engine):
    """Full benchmark shape B=8 T=8192 32q+8kv HS=128 bf16: one batch entry against the oracle,
    and every batch entry equal to it when all entries hold the same input (rotation depends on t, d only)."""
    import torch
    B, T, Nq, Nkv, HS = 8, 8192, 32, 8, 128
    H = Nq + 2 * Nkv
    rng = np.random.default_rng(0xB200 + 3)
    one = oracle.f32_to_bf16(rng.standard_normal(size=(1, T, H, HS)).astype(np.float32))
    table = oracle.freqs_cis(HS, T, 500000.0, 0)
    want = oracle.rope_forward_bf16(one, table, 1, T, Nq, Nkv, HS, threads=os.cpu_count() or 1)
    x = torch.from_numpy(one.view(np.int16)).cuda().repeat(B, 1, 1, 1).contiguous()
    nbytes = x.numel() * 2
    buf = sa.malloc(nbytes)
    tab = ch.cuda_malloc(table.nbytes)
    ch.h2d(tab, table)
    sa.memcpy_ptr(buf, x.data_ptr(), nbytes)
    sa.rope_forward_ptr(buf, tab, B, T, Nq, Nkv, HS, True)
    out = torch.empty_like(x)
    sa.memcpy_ptr(out.data_ptr(), buf, nbytes)
    torch.cuda.synchronize()
    want_t = torch.from_numpy(want.view(np.int16)).cuda()
    for b in range(B):
        assert torch.equal(out[b:b + 1], want_t), f"batch entry {b} differs from the oracle"
    sa.free(buf)
    ch.cuda_free(tab)


# ---------------------------------------------------------------------------
# silu-mul functor (ahead-of-time build)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("n", [8, 2048 + 8, (1 << 20) + 4096, 1 << 24])
def test_silu_mul_within_one_ulp(sa, n):
    rng = np.random.default_rng(0xB200 + 4)
    a = oracle.f32_to_bf16(rng.standard_normal(n).astype(np.float32))
    b = oracle.f32_to_bf16(rng.standard_normal(n).astype(np.float32))
    want = oracle.silu_mul_bf16(a, b, 0.5)
    bufs = [ch.Guarded(sa, 2 * n) for _ in range(3)]
    ch.h2d(bufs[0].ptr, a)
    ch.h2d(bufs[1].ptr, b)
    ch.memset(bufs[2].ptr, 0, bufs[2].payload_bytes)
    sa.silu_mul_ptr(bufs[2].ptr, bufs[0].ptr, bufs[1].ptr, 0.5, n)
    ch.sync()
    got = ch.d2h(bufs[2].ptr, 2 * n, np.uint16)
    assert oracle.ulp_diff_bf16(got, want).max() <= 1
    assert all(bf.canaries_intact() for bf in bufs)
    for bf in bufs:
        bf.free()
