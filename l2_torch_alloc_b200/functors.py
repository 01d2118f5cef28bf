"""Functor headers for sideaware_create_kernel (the NVRTC path).

A header is CUDA source text that follows the contract of the reference's
functor headers (sideaware.cu:81-138; examples: sideaware.cu:33-48,
kernel_rope.cuh:1-60, test.py:191-216): element typedefs o0..o3 / i0..i3,
``elementwise_op``, ``reverse_order``, ``input_evict`` and optional macros.
These generators bake the shape into the text, so one header serves one shape
(the reference's RoPE header hard-codes T=1024, 32 heads, HS=128 the same way).
"""
from __future__ import annotations

MEMCPY = """
typedef int o0;
typedef int i0;
struct unused {};
typedef unused o1, o2, o3, i1, i2, i3;
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {1, 0, 0, 0};
__device__ void elementwise_op(size_t idx, int sideband, o0 &out0, o1 &out1, o2 &out2, o3 &out3,
                               const i0 &in0, const i1 &in1, const i2 &in2, const i3 &in3) {
    out0 = in0;
}
"""


def silu_mul_bf16() -> str:
    """out = bf16(a * sigmoid(a) * b * scale); scale travels as the bits of sideband_value."""
    return """
#include <cuda_bf16.h>
typedef __nv_bfloat16 o0;
typedef __nv_bfloat16 i0;
typedef __nv_bfloat16 i1;
struct unused {};
typedef unused o1, o2, o3, i2, i3;
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {1, 1, 0, 0};
__device__ void elementwise_op(size_t idx, int sideband, o0 &out0, o1 &out1, o2 &out2, o3 &out3,
                               const i0 &in0, const i1 &in1, const i2 &in2, const i3 &in3) {
    float a = __bfloat162float(in0), b = __bfloat162float(in1);
    float scale = __int_as_float(sideband);
    float sig = 1.0f / (1.0f + __expf(-a));
    out0 = __float2bfloat16_rn(((a * sig) * b) * scale);
}
"""


def rope_forward(T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, bf16: bool) -> str:
    """In-place forward RoPE on packed [B, T, Nq + 2 Nkv, HS]; in1 is the fp32 [T, HS/2, 2] table.
    One element = one (real, imag) pair; V heads are skipped by the index function."""
    pair_t = "__nv_bfloat162" if bf16 else "float2"
    to_f = ("float x = __low2float(in0), y = __high2float(in0);" if bf16 else "float x = in0.x, y = in0.y;")
    from_f = ("out0 = __floats2bfloat162_rn(re, im);" if bf16 else "out0.x = re; out0.y = im;")
    # bf16: a 16-byte data vector needs 32 bytes of table; four vectors with their entries in flight per lane need more
    # than the 64 registers of a 1024-thread block, so blocks of 768 threads.  fp32: the default shape is the fastest.
    launch = ("#define UNROLLED 4\n#define LAUNCH_BOUNDS __launch_bounds__(768, 1)" if bf16 else "#define UNROLLED 2")
    return f"""
#include <cuda_bf16.h>
typedef {pair_t} o0;
typedef {pair_t} i0;
typedef float2 i1;
struct unused {{}};
typedef unused o1, o2, o3, i2, i3;
{launch}
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {{1, 0, 0, 0}}; // the table is shared by all heads of a token: keep it cached
constexpr int rope_T = {T};
constexpr int rope_half = {head_dim // 2};
constexpr int rope_rotated = {n_q_heads + n_kv_heads};
constexpr int rope_heads = {n_q_heads + 2 * n_kv_heads};

__device__ void elementwise_op(size_t idx, int sideband, o0 &out0, o1 &out1, o2 &out2, o3 &out3,
                               const i0 &in0, const i1 &in1, const i2 &in2, const i3 &in3) {{
    {to_f}
    float re = __fsub_rn(__fmul_rn(x, in1.x), __fmul_rn(y, in1.y));
    float im = __fadd_rn(__fmul_rn(x, in1.y), __fmul_rn(y, in1.x));
    {from_f}
}}

#define CUSTOM_IDX_FUNC
__device__ bool indexing(size_type vec_idx, int n, size_type &idx_i0, size_type &idx_i1,
                         size_type &idx_i2, size_type &idx_i3, int *mem, int val) {{
    size_type pair = vec_idx * n;
    size_type row = pair / (rope_heads * rope_half);
    int in_row = (int)(pair - row * (rope_heads * rope_half));
    int token = (int)(row % rope_T);
    idx_i0 = vec_idx;
    idx_i1 = (size_type)(token * rope_half + in_row % rope_half) / n;
    return in_row >= rope_rotated * rope_half;
}}
"""


def mxfp8_quantize_bf16() -> str:
    """bf16 -> MXFP8 (OCP Microscaling Formats v1.0: blocks of 32 elements, elements FP8 E4M3, one shared
    power-of-two scale per block stored as E8M0), the use the reference names for custom vector functions
    (sideaware.cu:81-83).  out0 = the E4M3 bytes, the sideband array receives one scale byte per block
    (pass it as a uint8 tensor viewed as int32), sideband_value = the number of 16-byte input vectors
    (elements / 8; 0 = the element count is a multiple of 32).

    A lane holds 8 elements, so a block is the four vectors of a lane quad and the block maximum is a
    reduction over the quad.  Where the whole warp is present and every lane's block is whole, the quads
    exchange under the full-warp mask; otherwise which lanes of a quad take part is worked out from the vector
    index and the vector count: in the last, partial block of an array whose element count is not a multiple
    of 32 only the lanes that exist exchange values.  The input must
    start on a 64-byte boundary (then vector 4k..4k+3 of the array are lanes 4j..4j+3 of one warp
    instruction); SideAware.mxfp8_quantize checks that.  Only the exponent of the maximum matters, so it is
    taken on the bf16 bit patterns (two elements per instruction), and the scaling is one exact
    multiplication by a power of two.
    Scale: 2^(floor(log2(amax)) - 8), 8 being the largest E4M3 exponent; elements are rounded to nearest
    even and saturate at +-448.  A block of zeros gets the smallest scale (byte 0); bf16 subnormals count as zero
    (functor kernels are compiled with flush-to-zero)."""
    return """
#include <cuda_bf16.h>
#include <cuda_fp8.h>
typedef __nv_fp8_e4m3 o0;
typedef __nv_bfloat16 i0;
struct unused {};
typedef unused o1, o2, o3, i1, i2, i3;
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {1, 0, 0, 0};
#define LAUNCH_BOUNDS __launch_bounds__(768, 1) // 85 registers per thread: eight vectors in flight per lane without spills
__device__ __forceinline__ unsigned sa_max_u16x2(unsigned a, unsigned b) {
    unsigned d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); // one instruction on sm_90 and later
    return d;
}
// packed maximum over the lanes of a quad that are named in `quad`: arrays whose element count is not a
// multiple of 32, and the ragged chunks at the ends of an array (kept out of line, off the common path)
__device__ __noinline__ unsigned sa_partial_quad_max(unsigned m, unsigned quad, unsigned first) {
    unsigned r = m;
    for (unsigned i = 0; i < 4; i++)
        if ((quad >> (first + i)) & 1u) r = sa_max_u16x2(r, __shfl_sync(quad, m, first + i));
    return r;
}
#define CUSTOM_VECTOR_OP
__device__ void vector_op(size_type vec_idx, int n, o0 *out0, o1 *out1, o2 *out2, o3 *out3,
                          const i0 *in0, const i1 *in1, const i2 *in2, const i3 *in3, int *mem, int val) {
    const unsigned *w = (const unsigned *)in0; // 8 bf16 = 4 words
    // magnitudes order like their 15-bit patterns: maximum of two elements per instruction
    unsigned m = sa_max_u16x2(sa_max_u16x2(w[0] & 0x7fff7fffu, w[1] & 0x7fff7fffu),
                              sa_max_u16x2(w[2] & 0x7fff7fffu, w[3] & 0x7fff7fffu));
    const unsigned lane = threadIdx.x & 31u;
    // The whole warp is here together and every lane's block is whole (any chunk but a ragged first or last one,
    // any block but the last one of an array whose element count is not a multiple of 32): plain full-warp
    // exchanges, which cost a fraction of exchanges under a partial mask.
    bool whole_warp = __activemask() == 0xffffffffu;
    if (whole_warp && val > 0) whole_warp = __all_sync(0xffffffffu, (int)vec_idx - (int)(lane & 3u) + 4 <= val);
    if (whole_warp) {
        m = sa_max_u16x2(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = sa_max_u16x2(m, __shfl_xor_sync(0xffffffffu, m, 2));
    } else {
        const unsigned first = lane & ~3u;
        unsigned quad = 0xFu << first;
        if (val > 0) { // vectors of this block that exist: all four except in the array's last block
            const int left = val - ((int)vec_idx - (int)(lane & 3u)); // vector counts stay below 2^31
            if (left < 4) quad = ((1u << left) - 1u) << first;
        }
        m = sa_partial_quad_max(m, quad, first);
    }
    // floor(log2(amax)) is the exponent field of the larger half; bf16 subnormals have field 0 and get the
    // smallest scale, like zero.  E8M0 scale byte = shared exponent + 127 = max(field, 8) - 8; the multiplier
    // 2^-(shared exponent) has exponent field 254 - scale byte = 262 - max(field, 8): 2^-120 .. 2^127, a normal float.
    const int t = max(max((int)((m >> 7) & 0xffu), (int)(m >> 23)), 8);
    const float mult = __uint_as_float((unsigned)t * 0xFF800000u + (262u << 23)); // (262 - t) << 23 as one multiply-add
    unsigned packed[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const float a0 = __fmul_rn(__uint_as_float(w[2 * i] << 16), mult);
        const float a1 = __fmul_rn(__uint_as_float(w[2 * i] & 0xffff0000u), mult);
        const float b0 = __fmul_rn(__uint_as_float(w[2 * i + 1] << 16), mult);
        const float b1 = __fmul_rn(__uint_as_float(w[2 * i + 1] & 0xffff0000u), mult);
        // four floats to four E4M3 bytes (round to nearest even, saturating at +-448), first element in the lowest byte
        asm("{ .reg .b16 lo, hi; cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1; cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3; "
            "mov.b32 %0, {lo, hi}; }"
            : "=r"(packed[i]) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
    }
    *(uint2 *)out0 = make_uint2(packed[0], packed[1]);
    // all lanes of the quad hold the same scale and store it to the same byte (no branch; one of the four equal
    // writes lands); a lane of a partial last block stores for the block it belongs to as well
    ((unsigned char *)mem)[(size_t)vec_idx >> 2] = (unsigned char)(t - 8);
}
"""
