"""The benchmark configurations at their FULL sizes, checked through size-independent properties and
sampled oracle comparisons (the oracle itself would take minutes on these sizes):
copies beyond the 32-bit byte and vector-index limits, the 2^30-element functor, both code paths."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sa():
    import torch
    assert torch.cuda.is_available()
    import l2_torch_alloc_b200 as pkg
    return pkg.SideAware()


@pytest.mark.parametrize("engine", [1, 0])
def test_memcpy_beyond_4_gib(sa, engine):
    """4 GiB + 40 KiB + 48 B: byte offsets need more than 32 bits.  Compared slab by slab against the source."""
    import torch
    n = (4 << 30) + 40 * 1024 + 48
    sa.lib.sideaware_set_memcpy_engine(engine)
    try:
        src = sa.malloc(n)
        dst = sa.malloc(n)
        slab = 256 << 20
        gen = torch.Generator(device="cuda").manual_seed(0xB200 + 8)
        pattern = torch.randint(0, 2**31 - 1, (slab // 4,), dtype=torch.int32, device="cuda", generator=gen)
        # the source is the pattern, XOR-ed with the slab number so that slabs differ
        for i, off in enumerate(range(0, n, slab)):
            size = min(slab, n - off)
            piece = (pattern ^ i)[: (size + 3) // 4].contiguous()
            sa.memcpy_ptr(src + off, piece.data_ptr(), size // 16 * 16)
            if size % 16:
                raise AssertionError("test sizes are multiples of 16")
        sa.memcpy_ptr(dst, src, n)
        out = torch.empty_like(pattern)
        for i, off in enumerate(range(0, n, slab)):
            size = min(slab, n - off)
            sa.memcpy_ptr(out.data_ptr(), dst + off, size)
            torch.cuda.synchronize()
            want = (pattern ^ i)[: size // 4]
            assert torch.equal(out[: size // 4], want), f"slab {i} differs"
        sa.free(src)
        sa.free(dst)
    finally:
        sa.lib.sideaware_set_memcpy_engine(1)


def test_functor_path_with_64_bit_indexing(sa):
    """An elementwise functor over 2.25 GiB (the NVRTC variant with 64-bit size_type, sideaware.cu:1386-1388)."""
    import torch
    from l2_torch_alloc_b200 import functors
    n_bytes = (2 << 30) + (256 << 20) + 4096 + 16
    src = torch.empty(n_bytes // 4, dtype=torch.int32, device="cuda")
    src.copy_(torch.arange(n_bytes // 4, dtype=torch.int64, device="cuda") % 2147483647)
    dst = torch.zeros_like(src)
    kid = sa.create_kernel(functors.MEMCPY + "// 64-bit indexing test\n")
    sa.one_to_one(kid, dst, src)
    torch.cuda.synchronize()
    assert torch.equal(dst, src)


def test_silu_mul_functor_at_2_pow_30_elements(sa):
    """out = bf16(a*sigmoid(a)*b*0.5) over 2^30 elements: NVRTC and ahead-of-time builds against each other
    everywhere (<= 1 bf16 ulp) and against the oracle on slices spread over the array."""
    import torch
    from l2_torch_alloc_b200 import functors
    n = 1 << 30
    gen = torch.Generator(device="cuda").manual_seed(0xB200 + 4)
    a = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    b = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    step = 1 << 27
    for off in range(0, n, step):
        a[off:off + step] = torch.randn(step, device="cuda", generator=gen).to(torch.bfloat16)
        b[off:off + step] = torch.randn(step, device="cuda", generator=gen).to(torch.bfloat16)
    out_jit = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    out_aot = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    kid = sa.create_kernel(functors.silu_mul_bf16())
    sa.elementwise(kid, out_jit, None, None, None, a, b, None, None, None, int(np.float32(0.5).view(np.int32)))
    sa.silu_mul(out_aot, a, b, 0.5)
    torch.cuda.synchronize()

    def ordered(t):  # bf16 bit patterns as monotonically ordered integers
        u = t.view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(u >= 0x8000, 0x8000 - u, u)

    for off in range(0, n, step):
        d = (ordered(out_jit[off:off + step]) - ordered(out_aot[off:off + step])).abs().max().item()
        assert d <= 1, f"NVRTC and ahead-of-time results differ by {d} ulp in slab at {off}"
    sl = 1 << 20
    for off in (0, 12345 * 8, n // 3 // 8 * 8, n - sl):
        au = a[off:off + sl].view(torch.int16).cpu().numpy().view(np.uint16)
        bu = b[off:off + sl].view(torch.int16).cpu().numpy().view(np.uint16)
        want = oracle.silu_mul_bf16(au, bu, 0.5)
        got = out_aot[off:off + sl].view(torch.int16).cpu().numpy().view(np.uint16)
        assert oracle.ulp_diff_bf16(got, want).max() <= 1


def test_mxfp8_functor_at_2_pow_30_elements(sa):
    """bf16 -> MXFP8 over 2^30 elements.  Size-independent property: a power-of-two factor on the input moves into the
    block scales and leaves every element byte as it was (x and 4x: same E4M3 bytes, scale bytes two higher).  And
    slices spread over the array equal the oracle bit for bit."""
    import torch
    n = 1 << 30
    gen = torch.Generator(device="cuda").manual_seed(0xB200 + 8)
    x = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    step = 1 << 27
    for off in range(0, n, step):
        x[off:off + step] = torch.randn(step, device="cuda", generator=gen).to(torch.bfloat16)
    el = torch.zeros(n, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(n // 32, dtype=torch.uint8, device="cuda")
    sa.mxfp8_quantize(el, sc, x)
    torch.cuda.synchronize()
    sl = 1 << 20
    for off in (0, 12345 * 32, n // 3 // 32 * 32, n - sl):
        xu = x[off:off + sl].view(torch.int16).cpu().numpy().view(np.uint16)
        want_el, want_sc = oracle.mxfp8_quantize_bf16(xu)
        assert np.array_equal(el[off:off + sl].cpu().numpy(), want_el)
        assert np.array_equal(sc[off // 32:(off + sl) // 32].cpu().numpy(), want_sc)
    el4 = torch.zeros(n, dtype=torch.uint8, device="cuda")
    sc4 = torch.zeros(n // 32, dtype=torch.uint8, device="cuda")
    for off in range(0, n, step):
        x[off:off + step] *= 4  # exact in bf16 (no value is near the top of the range)
    sa.mxfp8_quantize(el4, sc4, x)
    torch.cuda.synchronize()
    for off in range(0, n, step):
        assert torch.equal(el4[off:off + step], el[off:off + step])
    assert torch.equal(sc4.to(torch.int16), sc.to(torch.int16) + 2)
