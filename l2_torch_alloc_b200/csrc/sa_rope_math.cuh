// Arithmetic of the rotary embedding shared by the RoPE kernels: the rotation of one (real, imaginary)
// pair, the cos/sin entries one 16-byte data vector needs, and the position of a vector in the packed
// [B, T, Nq + 2 Nkv, HS] tensor.  Matches kernel_rope.cuh:30-60 in what it computes and
// example_llmc_rope.cu:54-86 bit for bit.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "sa_kernels.hpp"

namespace { // internal linkage: this header is included by more than one translation unit

// streaming (evict-first) 128-bit load: the data is used once
__device__ __forceinline__ uint4 sa_ld_stream(const uint4* p) { return __ldcs(p); }

__device__ __forceinline__ void rotate(float x, float y, float c, float s, float& ox, float& oy) {
    // separate roundings, no fused multiply-add: identical to the host arithmetic of
    // example_llmc_rope.cu:80-81 compiled without contraction
    ox = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s));
    oy = __fadd_rn(__fmul_rn(x, s), __fmul_rn(y, c));
}

// cos/sin entries that one 16-byte data vector needs: bf16 = 4 pairs (two float4), fp32 = 2 pairs (one)
template <bool BF16>
struct RopeTab {
    float4 a, b;
};

// `inverse` flips the sign of the sine entries: x*c - y*(-s) = x*c + y*s and x*(-s) + y*c are,
// bit for bit, what the reference's backward pass computes (example_llmc_rope.cu:191-192).
template <bool BF16>
__device__ __forceinline__ RopeTab<BF16> rope_load_tab(const float4* p, bool inverse) {
    RopeTab<BF16> t;
    t.a = __ldg(p);
    if constexpr (BF16) t.b = __ldg(p + 1);
    if (inverse) {
        t.a.y = -t.a.y;
        t.a.w = -t.a.w;
        if constexpr (BF16) {
            t.b.y = -t.b.y;
            t.b.w = -t.b.w;
        }
    }
    return t;
}

template <bool BF16>
__device__ __forceinline__ uint4 rope_apply(uint4 in, const RopeTab<BF16>& t) {
    uint4 out;
    if constexpr (BF16) {
        auto pair = [](uint32_t w, float c, float s) {
            float x = __uint_as_float(w << 16), y = __uint_as_float(w & 0xffff0000u);
            float ox, oy;
            rotate(x, y, c, s, ox, oy);
            __nv_bfloat162 b = __floats2bfloat162_rn(ox, oy);
            return *reinterpret_cast<uint32_t*>(&b);
        };
        out.x = pair(in.x, t.a.x, t.a.y);
        out.y = pair(in.y, t.a.z, t.a.w);
        out.z = pair(in.z, t.b.x, t.b.y);
        out.w = pair(in.w, t.b.z, t.b.w);
    } else {
        float ox0, oy0, ox1, oy1;
        rotate(__uint_as_float(in.x), __uint_as_float(in.y), t.a.x, t.a.y, ox0, oy0);
        rotate(__uint_as_float(in.z), __uint_as_float(in.w), t.a.z, t.a.w, ox1, oy1);
        out = make_uint4(__float_as_uint(ox0), __float_as_uint(oy0), __float_as_uint(ox1), __float_as_uint(oy1));
    }
    return out;
}

template <bool BF16>
__device__ __forceinline__ uint4 rope_vec(uint4 in, const float4* tab, bool inverse) {
    return rope_apply<BF16>(in, rope_load_tab<BF16>(tab, inverse));
}

// Position of vector `e` (element index in 16-byte vectors): returns false for a V-head
// vector, else the float4 index into the table.
__device__ __forceinline__ bool rope_locate(const SaRopeShape& sh, uint64_t e, uint32_t* tab_idx) {
    uint64_t row = e / sh.vecs_per_row;
    uint32_t r = (uint32_t)(e - row * sh.vecs_per_row);
    if (r >= sh.rotated_vecs) return false;
    uint32_t tok = (uint32_t)(row % sh.T);
    uint32_t pos = r % sh.vecs_per_head;
    *tab_idx = tok * sh.tab_vecs_per_token + pos * sh.tab_vecs_per_vec;
    return true;
}

} // namespace
