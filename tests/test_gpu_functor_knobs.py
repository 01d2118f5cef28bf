"""The optional knobs of the functor-header contract (sideaware.cu:60-109, :170-184) on a B200:
UNROLLED, LAUNCH_BOUNDS with fewer groups, FORCE_WRONG_SIDE / FORCE_RANDOM_SIDE, DISCARD_INPUTS,
CUSTOM_VECTOR_OP with sideband memory, CUSTOM_IDX_FUNC with skipping.  Integer / exactly
representable data, so every comparison is exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

BASE = """
typedef int o0;
typedef int i0;
struct unused {};
typedef unused o1, o2, o3, i1, i2, i3;
constexpr bool reverse_order = %s;
constexpr bool input_evict[4] = {1, 0, 0, 0};
__device__ void elementwise_op(size_t idx, int sideband, o0 &out0, o1 &out1, o2 &out2, o3 &out3,
                               const i0 &in0, const i1 &in1, const i2 &in2, const i3 &in3) {
    out0 = in0 * 3 + sideband + (int)(idx & 7);
}
"""


@pytest.fixture(scope="module")
def sa():
    import torch
    assert torch.cuda.is_available()
    import l2_torch_alloc_b200 as pkg
    return pkg.SideAware()


def expected(src, sideband):
    import torch
    idx = torch.arange(src.numel(), device=src.device, dtype=torch.int64)
    return (src.to(torch.int64) * 3 + sideband + (idx & 7)).to(torch.int32)


@pytest.mark.parametrize("extra,groups", [
    ("", 0),
    ("#define UNROLLED 1\n", 0),
    ("#define UNROLLED 2\n", 0),
    ("#define UNROLLED 8\n#define LAUNCH_BOUNDS __launch_bounds__(512, 1)\n", 2),
    ("#define FORCE_WRONG_SIDE true\n", 0),
    ("#define FORCE_RANDOM_SIDE true\n", 0),
    ("#define DYNAMIC_INDEX_FOR_CONCURRENT_KERNELS\n", 1),
    ("#define DISCARD_INPUTS\nconstexpr bool input_discard[4] = {1, 0, 0, 0};\n", 0),
])
@pytest.mark.parametrize("reverse", ["false", "true"])
def test_knobs_keep_results_exact(sa, extra, groups, reverse):
    import torch
    n = 3 * 1000 * 1000 + 12  # ragged: not a multiple of a chunk
    src = torch.randint(-1000, 1000, (n,), dtype=torch.int32, device="cuda")
    want = expected(src, 5)
    kid = sa.create_kernel(extra + BASE % reverse)
    for big in (False, True):  # torch memory below the allocator threshold, then a side-aware block
        if big:
            n2 = 24 * 1024 * 1024
            src = torch.randint(-1000, 1000, (n2,), dtype=torch.int32, device="cuda")
            want = expected(src, 5)
        dst = torch.zeros_like(src)
        sa.elementwise(kid, dst, None, None, None, src, None, None, None, None, 5, groups, 0)
        torch.cuda.synchronize()
        assert torch.equal(dst, want)


VECTOR_OP = """
typedef float o0;
typedef float i0;
struct unused {};
typedef unused o1, o2, o3, i1, i2, i3;
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {1, 0, 0, 0};
#define CUSTOM_VECTOR_OP
// one scale per 16-byte vector (the micro-scaling pattern the contract mentions, sideaware.cu:81-83):
// out = in / absmax(vector), absmax written to the sideband array
__device__ void vector_op(size_type vec_idx, int n, o0 *out0, o1 *out1, o2 *out2, o3 *out3,
                          const i0 *in0, const i1 *in1, const i2 *in2, const i3 *in3, int *mem, int val) {
    float m = 0.0f;
    for (int e = 0; e < n; e++) m = fmaxf(m, fabsf(in0[e]));
    ((float*)mem)[vec_idx] = m;
    float scale = m > 0.0f ? __fdiv_rn(1.0f, m) : 0.0f;
    for (int e = 0; e < n; e++) out0[e] = __fmul_rn(in0[e], scale) + (float)val;
}
"""


def test_custom_vector_op_with_sideband_memory(sa):
    import torch
    n = 4 * (1 << 20) + 4 * 37
    # powers of two: absmax, reciprocal and products are exact
    exps = torch.randint(-8, 8, (n,), device="cuda")
    signs = torch.randint(0, 2, (n,), device="cuda") * 2 - 1
    x = (signs * torch.pow(2.0, exps.float())).float()
    out = torch.zeros_like(x)
    scales = torch.zeros(n // 4, dtype=torch.float32, device="cuda")
    kid = sa.create_kernel(VECTOR_OP)
    sa.elementwise(kid, out, None, None, None, x, None, None, None, scales.view(torch.int32), 2)
    torch.cuda.synchronize()
    m = x.view(-1, 4).abs().amax(dim=1)
    assert torch.equal(scales, m)
    assert torch.equal(out, (x.view(-1, 4) / m[:, None]).reshape(-1) + 2.0)


GATHER = """
typedef float o0;
typedef float i0;
typedef float i1;
struct unused {};
typedef unused o1, o2, o3, i2, i3;
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {1, 0, 0, 0};
__device__ void elementwise_op(size_t idx, int sideband, o0 &out0, o1 &out1, o2 &out2, o3 &out3,
                               const i0 &in0, const i1 &in1, const i2 &in2, const i3 &in3) {
    out0 = in0 + in1;
}
#define CUSTOM_IDX_FUNC
// in1 is a short row broadcast over the long array; every 5th row of 64 vectors is left untouched
__device__ bool indexing(size_type vec_idx, int n, size_type &idx_i0, size_type &idx_i1,
                         size_type &idx_i2, size_type &idx_i3, int *mem, int val) {
    idx_i0 = vec_idx;
    idx_i1 = vec_idx % val;
    return ((vec_idx / 64) % 5) == 4;
}
"""


def test_custom_index_function_broadcast_and_skip(sa):
    import torch
    rows, row_vecs, bias_vecs = 6000, 64, 48
    n = rows * row_vecs * 4
    x = torch.arange(n, dtype=torch.float32, device="cuda") % 1024
    bias = torch.arange(bias_vecs * 4, dtype=torch.float32, device="cuda") * 4
    out = x.clone()
    kid = sa.create_kernel(GATHER)
    sa.elementwise(kid, out, None, None, None, x, bias, None, None, None, bias_vecs)
    torch.cuda.synchronize()
    vec = torch.arange(n // 4, device="cuda")
    want = x.view(-1, 4) + bias.view(-1, 4)[vec % bias_vecs]
    keep = ((vec // 64) % 5) == 4
    want[keep] = x.view(-1, 4)[keep]
    assert torch.equal(out.view(-1, 4), want)


def test_mxfp8_quantize_matches_restatement(sa):
    """bf16 -> MXFP8 (blocks of 32, E4M3 elements, E8M0 scales in the sideband array): the use the reference names
    for custom vector functions (sideaware.cu:81-83).  Element bytes and scale bytes equal the numpy restatement of
    the OCP Microscaling v1.0 rules bit for bit, over magnitudes from bf16 subnormals to 3e38, zero blocks included."""
    import numpy as np
    import torch
    from oracle import oracle
    from l2_torch_alloc_b200 import functors
    blocks = (1 << 17) + 37
    n = blocks * 32
    rng = np.random.default_rng(0xB200 + 8)
    x = rng.standard_normal((blocks, 32)).astype(np.float32)
    x *= np.exp2(rng.integers(-60, 60, size=(blocks, 1))).astype(np.float32)
    x[5] = 0.0                                   # a block of zeros
    x[6] = 3.0e38 * np.sign(x[6] + 0.5)          # near the top of the range
    x[7] = 1.0e-40                               # bf16 subnormals
    x[8, :] = 0.0
    x[8, 3] = -448.0 * 2.0 ** 10                 # one element carries the block
    x_u16 = oracle.f32_to_bf16(x.reshape(-1))
    want_el, want_sc = oracle.mxfp8_quantize_bf16(x_u16)
    xin = torch.from_numpy(x_u16.view(np.int16)).cuda().view(torch.bfloat16)
    out = torch.zeros(n, dtype=torch.uint8, device="cuda")
    scales = torch.full(((blocks + 3) // 4 * 4,), 0xEE, dtype=torch.uint8, device="cuda")
    sa.mxfp8_quantize(out, scales, xin)
    torch.cuda.synchronize()
    got_el = out.cpu().numpy()
    got_sc = scales.cpu().numpy()
    assert np.array_equal(got_sc[:blocks], want_sc), np.nonzero(got_sc[:blocks] != want_sc)[0][:10]
    assert (got_sc[blocks:] == 0xEE).all(), "no scale byte is written past the last block"
    bad = np.nonzero(got_el != want_el)[0]
    assert bad.size == 0, (bad[:10], got_el[bad[:10]], want_el[bad[:10]])


@pytest.mark.parametrize("tail_vectors", [1, 2, 3])
def test_mxfp8_last_partial_block_is_scaled_by_the_elements_it_has(sa, tail_vectors):
    """Element counts that are not a multiple of 32: the last block has 8, 16 or 24 elements.  Its scale and its
    elements must be those of a block padded with zeros (zeros cannot raise the maximum)."""
    import torch
    from oracle import oracle
    blocks = 4099
    n = blocks * 32 + tail_vectors * 8
    rng = np.random.default_rng(0xB200 + 80 + tail_vectors)
    x = rng.standard_normal(n).astype(np.float32) * np.exp2(rng.integers(-20, 20, size=n)).astype(np.float32)
    x[-1] = 3.0e4  # the largest element of the partial block sits in its last vector
    x_u16 = oracle.f32_to_bf16(x)
    padded = np.concatenate([x_u16, np.zeros((blocks + 1) * 32 - n, dtype=np.uint16)])
    want_el, want_sc = oracle.mxfp8_quantize_bf16(padded)
    xin = torch.from_numpy(x_u16.view(np.int16)).cuda().view(torch.bfloat16)
    out = torch.full((n + 64,), 0xEE, dtype=torch.uint8, device="cuda")
    scales = torch.full(((blocks + 1 + 3) // 4 * 4 + 4,), 0xEE, dtype=torch.uint8, device="cuda")
    sa.mxfp8_quantize(out, scales, xin)
    torch.cuda.synchronize()
    got_el, got_sc = out.cpu().numpy(), scales.cpu().numpy()
    assert np.array_equal(got_sc[:blocks + 1], want_sc)
    assert (got_sc[blocks + 1:] == 0xEE).all()
    assert np.array_equal(got_el[:n], want_el[:n])
    assert (got_el[n:] == 0xEE).all(), "nothing is written behind the last element"


def test_mxfp8_helper_refuses_an_input_that_blocks_would_straddle(sa):
    import torch
    x = torch.zeros(4096 + 32, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(128, dtype=torch.uint8, device="cuda")
    with pytest.raises(AssertionError, match="64-byte boundary"):
        sa.mxfp8_quantize(out, scales, x[8:8 + 4096])  # 16 bytes in: legal for the kernel, wrong for the blocks
    with pytest.raises(AssertionError, match="multiple of 8"):
        sa.mxfp8_quantize(out, scales, x[:4092])


WIDE_AUX = """
#include <cuda_bf16.h>
typedef __nv_bfloat16 o0;
typedef __nv_bfloat16 i0;
typedef float i1;
struct unused {};
typedef unused o1, o2, o3, i2, i3;
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {1, 1, 0, 0};
__device__ void elementwise_op(size_t idx, int sideband, o0 &out0, o1 &out1, o2 &out2, o3 &out3,
                               const i0 &in0, const i1 &in1, const i2 &in2, const i3 &in3) {
    out0 = __float2bfloat16_rn(__bfloat162float(in0) + in1);
}
"""


def test_auxiliary_array_wider_than_the_tracked_one_does_not_widen_the_launch(sa):
    """in0 / out0 are bf16, in1 is fp32: in1 holds twice the bytes, but the number of 16-byte vectors follows
    in0 (sideaware.cu:127-129).  Canary bytes behind out0 and in0 show that nothing ran past their end."""
    import torch
    n = 3 * (1 << 20) + 8 * 11
    pad = 1 << 16
    a_all = torch.full((n + pad,), 7.0, dtype=torch.bfloat16, device="cuda")
    o_all = torch.full((n + pad,), -3.0, dtype=torch.bfloat16, device="cuda")
    a_all[:n] = torch.randint(-64, 64, (n,), device="cuda").to(torch.bfloat16)
    b = torch.randint(-64, 64, (n,), device="cuda").float()
    kid = sa.create_kernel(WIDE_AUX)
    sa.elementwise(kid, o_all[:n], None, None, None, a_all[:n], b, None, None)
    torch.cuda.synchronize()
    assert torch.equal(o_all[:n].float(), a_all[:n].float() + b)
    assert bool((o_all[n:] == -3.0).all()) and bool((a_all[n:] == 7.0).all())
