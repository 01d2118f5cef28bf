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
    return f"""
#include <cuda_bf16.h>
typedef {pair_t} o0;
typedef {pair_t} i0;
typedef float2 i1;
struct unused {{}};
typedef unused o1, o2, o3, i2, i3;
#define UNROLLED 2
constexpr bool reverse_order = false;
constexpr bool input_evict[4] = {{1, 0, 0, 0}};
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
