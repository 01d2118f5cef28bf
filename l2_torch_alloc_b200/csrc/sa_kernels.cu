// Ahead-of-time side-aware kernels for sm_100a: memcpy, in-place forward RoPE
// (fp32 and bf16 storage) and the bf16 silu-mul example functor.
//
// Every kernel is a persistent grid of one 1024-thread block per SM.  A warp
// owns one 4 KiB chunk at a time: 32 lanes x 16 bytes per instruction, eight
// independent 128-bit loads in flight per lane, then the arithmetic, then
// eight 128-bit stores.  Which chunks a warp takes is decided by sa_sched.cuh.
// None of these paths is a contraction, so no tensor-core instructions appear;
// the bound is HBM bandwidth.
//
// Replaces the reference's JIT-ed template kernel for these functors:
// sideaware.cu:194-386 with the memcpy header sideaware.cu:33-48 and the RoPE
// header kernel_rope.cuh:1-60.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "sa_kernels.hpp"
#include "sa_rope_math.cuh"

namespace {

constexpr int kMaxThreads = 1024;


// ---------------------------------------------------------------------------
// memcpy
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kMaxThreads, 1)
sa_memcpy_kernel(const __grid_constant__ SaSched s, const __grid_constant__ SaSideTable sides,
                 uint4* __restrict__ dst, const uint4* __restrict__ src) {
    const uint32_t lane = sa_lane();
    sa_for_each_chunk(s, sides, [&](uint64_t first_vec) {
        if (first_vec >= s.lead && first_vec + SA_CHUNK_VECS <= s.end) {
            const uint64_t e = first_vec - s.lead + lane;
            const uint4* p = src + e;
            uint4 r[SA_VEC_PER_LANE];
#pragma unroll
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) r[k] = sa_ld_stream(p + k * 32);
            uint4* q = dst + e;
#pragma unroll
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) q[k * 32] = r[k];
        } else {
            // first or last chunk of the array: per-vector bounds
#pragma unroll 1
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                uint64_t v = first_vec + k * 32 + lane;
                if (v >= s.lead && v < s.end) dst[v - s.lead] = sa_ld_stream(src + (v - s.lead));
            }
        }
    });
}

// ---------------------------------------------------------------------------
// RoPE forward, in place on packed [B, T, Nq + 2 Nkv, HS]
// ---------------------------------------------------------------------------
template <bool BF16, int THREADS>
__global__ void __launch_bounds__(THREADS, 1)
sa_rope_kernel(const __grid_constant__ SaSched s, const __grid_constant__ SaSideTable sides,
               uint4* __restrict__ x, const float4* __restrict__ table,
               const __grid_constant__ SaRopeShape sh) {
    const uint32_t lane = sa_lane();
    sa_for_each_chunk(s, sides, [&](uint64_t first_vec) {
        if (first_vec >= s.lead && first_vec + SA_CHUNK_VECS <= s.end && sh.vecs_per_row >= SA_CHUNK_VECS) {
            // whole chunk: one 64-bit division per chunk, then 32-bit bookkeeping per vector
            const uint64_t e0 = first_vec - s.lead;
            const uint64_t row0 = e0 / sh.vecs_per_row;
            const uint32_t r0 = (uint32_t)(e0 - row0 * sh.vecs_per_row) + lane;
            const uint32_t tok0 = (uint32_t)(row0 % sh.T);
            uint4* p = x + e0 + lane;
            uint4 v[SA_VEC_PER_LANE];
            // position of vector k of this lane inside its token row; recomputed (not kept) for the
            // second loop to stay inside the 64-register budget of a 1024-thread block
            auto locate = [&](int k, uint32_t& r, uint32_t& tok) {
                r = r0 + k * 32;
                tok = tok0;
                if (r >= sh.vecs_per_row) { // a chunk is shorter than a row: at most one wrap
                    r -= sh.vecs_per_row;
                    tok = (tok + 1 == sh.T) ? 0 : tok + 1;
                }
            };
#pragma unroll
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                uint32_t r, tok;
                locate(k, r, tok);
                if (r < sh.rotated_vecs) v[k] = sa_ld_stream(p + k * 32);
            }
            // When a head is a power-of-two number of vectors that divides the 32-lane stride, every
            // vector of this lane sits at the same place in its head: the cos/sin entries only change
            // when the token changes (at most once inside a chunk), so they are fetched once and kept.
            const bool pos_fixed = sh.head_shift >= 0 && sh.vecs_per_head <= 32u;
            const uint32_t pos_lane = r0 & (sh.vecs_per_head - 1u);
            uint32_t have_tok = 0xffffffffu;
            RopeTab<BF16> tab;
#pragma unroll
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                uint32_t r, tok;
                locate(k, r, tok);
                if (r < sh.rotated_vecs) {
                    if (!pos_fixed || tok != have_tok) {
                        const uint32_t pos = pos_fixed ? pos_lane : (r % sh.vecs_per_head);
                        tab = rope_load_tab<BF16>(table + tok * sh.tab_vecs_per_token + pos * sh.tab_vecs_per_vec, sh.inverse != 0);
                        have_tok = tok;
                    }
                    p[k * 32] = rope_apply<BF16>(v[k], tab);
                }
            }
        } else {
#pragma unroll 1
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                uint64_t a = first_vec + k * 32 + lane;
                uint32_t ti;
                if (a >= s.lead && a < s.end && rope_locate(sh, a - s.lead, &ti)) {
                    uint4* p = x + (a - s.lead);
                    *p = rope_vec<BF16>(sa_ld_stream(p), table + ti, sh.inverse != 0);
                }
            }
        }
    });
}

// ---------------------------------------------------------------------------
// out = bf16(a * sigmoid(a) * b * scale)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t silu_mul_pair(uint32_t a, uint32_t b, float scale) {
    float a0 = __uint_as_float(a << 16), a1 = __uint_as_float(a & 0xffff0000u);
    float b0 = __uint_as_float(b << 16), b1 = __uint_as_float(b & 0xffff0000u);
    float s0 = __fdividef(1.0f, 1.0f + __expf(-a0)), s1 = __fdividef(1.0f, 1.0f + __expf(-a1));
    __nv_bfloat162 r = __floats2bfloat162_rn(((a0 * s0) * b0) * scale, ((a1 * s1) * b1) * scale);
    return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint4 silu_mul_vec(uint4 a, uint4 b, float scale) {
    return make_uint4(silu_mul_pair(a.x, b.x, scale), silu_mul_pair(a.y, b.y, scale),
                      silu_mul_pair(a.z, b.z, scale), silu_mul_pair(a.w, b.w, scale));
}

__global__ void __launch_bounds__(kMaxThreads, 1)
sa_silu_mul_kernel(const __grid_constant__ SaSched s, const __grid_constant__ SaSideTable sides,
                   uint4* __restrict__ out, const uint4* __restrict__ a,
                   const uint4* __restrict__ b, float scale) {
    const uint32_t lane = sa_lane();
    sa_for_each_chunk(s, sides, [&](uint64_t first_vec) {
        if (first_vec >= s.lead && first_vec + SA_CHUNK_VECS <= s.end) {
            const uint64_t e = first_vec - s.lead + lane;
#pragma unroll
            for (int h = 0; h < 2; ++h) { // two halves of four vectors: 8 loads in flight, 32 data registers
                uint4 ra[4], rb[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    ra[k] = sa_ld_stream(a + e + (h * 4 + k) * 32);
                    rb[k] = sa_ld_stream(b + e + (h * 4 + k) * 32);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) out[e + (h * 4 + k) * 32] = silu_mul_vec(ra[k], rb[k], scale);
            }
        } else {
#pragma unroll 1
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                uint64_t v = first_vec + k * 32 + lane;
                if (v >= s.lead && v < s.end)
                    out[v - s.lead] = silu_mul_vec(sa_ld_stream(a + (v - s.lead)), sa_ld_stream(b + (v - s.lead)), scale);
            }
        }
    });
}

} // namespace

bool sa_pdl_enabled() {
    static const bool pdl = [] { // on unless SIDEAWARE_PDL=0
        const char* e = std::getenv("SIDEAWARE_PDL");
        return !(e && std::atoi(e) == 0);
    }();
    return pdl;
}

SaLaunch::SaLaunch(const SaSched& s, int grid, int threads, size_t smem, cudaStream_t stream) {
    const bool pdl = sa_pdl_enabled();
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && s.overlap) ? 1 : 0;
}

cudaError_t sa_launch_memcpy(const SaSched& s, const SaSideTable& sides, int grid, int threads, void* dst, const void* src, cudaStream_t stream) {
    SaLaunch l(s, grid, threads, 0, stream);
    return cudaLaunchKernelEx(&l.cfg, sa_memcpy_kernel, s, sides, (uint4*)dst, (const uint4*)src);
}

cudaError_t sa_launch_rope(const SaSched& s, const SaSideTable& sides, int grid, int threads, void* x, const float* table,
                           const SaRopeShape& sh, bool bf16, cudaStream_t stream) {
    // at most 768 threads per block: that leaves 85 registers per thread (the bf16 rotation needs
    // ~72; a 1024-thread block would cap it at 64 and spill), and 24 warps x 4 KiB still keep
    // 96 KiB in flight per SM
    if (threads > 768) return cudaErrorInvalidConfiguration;
    SaLaunch l(s, grid, threads, 0, stream);
    if (bf16) return cudaLaunchKernelEx(&l.cfg, sa_rope_kernel<true, 768>, s, sides, (uint4*)x, (const float4*)table, sh);
    return cudaLaunchKernelEx(&l.cfg, sa_rope_kernel<false, 768>, s, sides, (uint4*)x, (const float4*)table, sh);
}

cudaError_t sa_launch_silu_mul(const SaSched& s, const SaSideTable& sides, int grid, int threads, void* out, const void* a, const void* b,
                               float scale, cudaStream_t stream) {
    SaLaunch l(s, grid, threads, 0, stream);
    return cudaLaunchKernelEx(&l.cfg, sa_silu_mul_kernel, s, sides, (uint4*)out, (const uint4*)a, (const uint4*)b, scale);
}

// ---------------------------------------------------------------------------
// cos/sin table of the rotary embedding
// ---------------------------------------------------------------------------
// table[t][i] = (cos(a), sin(a)) with a = (float)t * freq[i] rounded to fp32 as in
// example_llmc_rope.cu:46-50.  Cosine and sine are taken in fp64 and rounded once, which is the
// correctly rounded fp32 value except when the exact result lies within 2^-29 ulp of a rounding
// boundary; libm's cosf/sinf are within 0.56 ulp, so the two agree to 1 ulp.  The table is a few
// MiB and written once: a plain grid, no side awareness.
namespace {
struct SaRopeFreqs { float f[512]; };

__global__ void sa_rope_table_kernel(float2* __restrict__ table, const __grid_constant__ SaRopeFreqs freqs, int half, long long entries) {
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < entries; e += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(e / half), i = (int)(e % half);
        const float angle = __fmul_rn((float)t, freqs.f[i]);
        double s, c;
        sincos((double)angle, &s, &c);
        table[e] = make_float2((float)c, (float)s);
    }
}
} // namespace

cudaError_t sa_launch_rope_table(float* table, const float* freqs, int half, int end, cudaStream_t stream) {
    if (half <= 0 || half > 512 || end <= 0) return cudaErrorInvalidValue;
    SaRopeFreqs f;
    std::memset(&f, 0, sizeof(f));
    std::memcpy(f.f, freqs, sizeof(float) * (size_t)half);
    const long long entries = (long long)half * end;
    long long blocks = (entries + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    sa_rope_table_kernel<<<(unsigned)blocks, 256, 0, stream>>>((float2*)table, f, half, entries);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// memcpy for callers that must not allocate device memory
// ---------------------------------------------------------------------------
// The memcpy kernel needs three ticket counters in global memory.  Normally they come
// from a buffer the library allocated when the device was first used.  Here they live in
// a fixed 512-byte array that is part of the loaded module, so no allocation call is made;
// every GPU that loads the library carries these 512 bytes until the process exits.
#define SA_NOALLOC_SCRATCH_WORDS 128
static __device__ __align__(256) unsigned int sa_noalloc_scratch[SA_NOALLOC_SCRATCH_WORDS];

namespace {
constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned int* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
} // namespace

// `device` must be the current device.  The first call on a device looks up the device
// address of the array (in host code the array's name is only a handle, not an address a
// kernel could use) and keeps it.  Every call then zeroes the counters on `stream` before
// the kernel runs, because the array is shared by all calls and keeps whatever the last
// one left behind.
cudaError_t sa_launch_memcpy_noalloc(SaSched s, const SaSideTable& sides, int device, int grid, int threads, void* dst, const void* src,
                                     cudaStream_t stream) {
    if (device < 0 || device >= kNoAllocMaxDevices) return cudaErrorInvalidDevice;
    unsigned int* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (!g_noalloc_ptr[device]) {
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, sa_noalloc_scratch);
            if (e != cudaSuccess) return e;
            g_noalloc_ptr[device] = (unsigned int*)p;
        }
        scratch = g_noalloc_ptr[device];
    }
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(unsigned int) * SA_NOALLOC_SCRATCH_WORDS, stream);
    if (e != cudaSuccess) return e;
    s.tickets = scratch;
    sa_memcpy_kernel<<<grid, threads, 0, stream>>>(s, sides, (uint4*)dst, (const uint4*)src);
    return cudaGetLastError();
}
