// Generic side-aware elementwise kernel for user functors, compiled at run time
// with NVRTC for sm_100a.  The text of this file is embedded in the library and
// appended after (1) a small prefix generated per device and variant, (2) the
// user's functor header and (3) sa_sched.cuh.
//
// Functor header contract (kept from the reference, sideaware.cu:60-138):
//   typedef ... o0, o1, o2, o3, i0, i1, i2, i3;      unused slots are `unused` (struct unused {};)
//   constexpr bool reverse_order;                     walk the array from the end
//   constexpr bool input_evict[4];                    stream (evict-first) loads per input
//   __device__ void elementwise_op(size_t idx, int sideband, o0&, o1&, o2&, o3&,
//                                  const i0&, const i1&, const i2&, const i3&);
//   optional macros: UNROLLED, LAUNCH_BOUNDS, DISCARD_INPUTS (+ constexpr bool input_discard[4]),
//   CUSTOM_VECTOR_OP (+ vector_op), CUSTOM_IDX_FUNC (+ indexing), FORCE_WRONG_SIDE,
//   FORCE_RANDOM_SIDE, DYNAMIC_INDEX_FOR_CONCURRENT_KERNELS (accepted; work
//   assignment here is always dynamic).
// The prefix provides size_type, aligned_2MiB, MAX_SM and HASH as the reference does
// (sideaware.cu:786-795).
//
// The widest array (i0, or o0 if its element is larger) is moved as 16-byte
// vectors; the others move vec_size elements per vector with 16/8/4/2/1-byte
// accesses.  A warp owns one 4 KiB chunk of the widest array at a time and
// processes it in batches of vectors per lane (sa_batch below): all loads of a batch
// are issued before its arithmetic and stores.

#ifndef UNROLLED
#define UNROLLED 4
#endif
#ifndef LAUNCH_BOUNDS
#define LAUNCH_BOUNDS __launch_bounds__(1024, 1)
#endif
#ifndef DISCARD_INPUTS
constexpr bool input_discard[4] = {false, false, false, false};
#endif
#ifndef FORCE_WRONG_SIDE
#define FORCE_WRONG_SIDE false
#endif
#ifndef FORCE_RANDOM_SIDE
#define FORCE_RANDOM_SIDE false
#endif

constexpr bool sideaware_for_o0 = sizeof(o0) > sizeof(i0);
constexpr int vec_size = 16 / (int)(sideaware_for_o0 ? sizeof(o0) : sizeof(i0));

template <typename A, typename B> struct sa_same { static constexpr bool value = false; };
template <typename A> struct sa_same<A, A> { static constexpr bool value = true; };
template <typename T> constexpr bool sa_used = !sa_same<T, unused>::value;

// vec_size elements of T, aligned so one access moves them when the size allows it
template <typename T, int BYTES = (int)sizeof(T) * vec_size>
struct alignas(BYTES == 16 || BYTES == 8 || BYTES == 4 || BYTES == 2 ? BYTES : alignof(T)) sa_pack {
    T v[vec_size];
};

// Vectors each lane keeps in flight (loads issued before the arithmetic of the batch starts).
// UNROLLED is the header author's wish; on top of that the batch is widened while the inputs of
// a batch fit in about 32 registers, because bytes in flight are what hides HBM latency.  The
// library compiles this version first and falls back to the batch as written
// (SA_BATCH_AS_WRITTEN) if the compiler had to spill registers.
constexpr int sa_user_batch = (UNROLLED) >= 8 ? 8 : (UNROLLED) >= 4 ? 4 : (UNROLLED) >= 2 ? 2 : 1;
constexpr int sa_in_bytes = (sa_used<i0> ? (int)sizeof(sa_pack<i0>) : 0) + (sa_used<i1> ? (int)sizeof(sa_pack<i1>) : 0) +
                            (sa_used<i2> ? (int)sizeof(sa_pack<i2>) : 0) + (sa_used<i3> ? (int)sizeof(sa_pack<i3>) : 0);
constexpr int sa_auto_batch = sa_in_bytes <= 16 ? 8 : sa_in_bytes <= 32 ? 4 : sa_in_bytes <= 64 ? 2 : 1;
#ifdef SA_BATCH_AS_WRITTEN
constexpr int sa_batch = sa_user_batch;
#else
constexpr int sa_batch = sa_auto_batch > sa_user_batch ? sa_auto_batch : sa_user_batch;
#endif

#ifndef CUSTOM_VECTOR_OP
__device__ __forceinline__ void vector_op(size_type vec_idx, int n,
                                          o0* out0, o1* out1, o2* out2, o3* out3,
                                          const i0* in0, const i1* in1, const i2* in2, const i3* in3,
                                          int* sideband_memory, int sideband_value) {
#pragma unroll
    for (int e = 0; e < n; ++e)
        elementwise_op((size_t)vec_idx * n + e, sideband_value, out0[e], out1[e], out2[e], out3[e],
                       in0[e], in1[e], in2[e], in3[e]);
}
#endif

#ifndef CUSTOM_IDX_FUNC
__device__ __forceinline__ bool indexing(size_type vec_idx, int n, size_type& idx_i0, size_type& idx_i1,
                                         size_type& idx_i2, size_type& idx_i3, int* sideband_memory, int sideband_value) {
    idx_i0 = idx_i1 = idx_i2 = idx_i3 = vec_idx;
    return false;
}
#endif

// EVICT (input_evict[i] = 1): streaming load, the line is first in line for eviction (data used once).
// Otherwise an ordinary load that may stay in L1 and L2: what a functor wants for a table that many vectors share
// (a RoPE cos/sin row is read by every head of a token).  The reference uses ld.global.cg for these
// (sideaware.cu:140-168), which skips L1; the values loaded are the same.
template <bool EVICT, typename T>
__device__ __forceinline__ void sa_load(sa_pack<T>& dst, const sa_pack<T>* base, size_type idx) {
    if constexpr (sa_used<T>) {
        const sa_pack<T>* p = base + idx;
        if constexpr (sizeof(sa_pack<T>) == 32 || sizeof(sa_pack<T>) == 64) {
            // an array whose element is wider than the tracked one's (fp32 table beside bf16 data): 16-byte pieces
            // (every array starts on a 16-byte boundary, the launcher checks that)
#pragma unroll
            for (int k = 0; k < (int)sizeof(sa_pack<T>) / 16; ++k) {
                int4 r = EVICT ? __ldcs((const int4*)p + k) : *((const int4*)p + k);
                *((int4*)&dst + k) = r;
            }
        } else if constexpr (sizeof(sa_pack<T>) == 16) {
            int4 r = EVICT ? __ldcs((const int4*)p) : *(const int4*)p;
            *(int4*)&dst = r;
        } else if constexpr (sizeof(sa_pack<T>) == 8) {
            int2 r = EVICT ? __ldcs((const int2*)p) : *(const int2*)p;
            *(int2*)&dst = r;
        } else if constexpr (sizeof(sa_pack<T>) == 4) {
            int r = EVICT ? __ldcs((const int*)p) : *(const int*)p;
            *(int*)&dst = r;
        } else if constexpr (sizeof(sa_pack<T>) == 2) {
            short r = EVICT ? __ldcs((const short*)p) : *(const short*)p;
            *(short*)&dst = r;
        } else {
            dst = *p;
        }
    }
}

template <typename T>
__device__ __forceinline__ void sa_store(sa_pack<T>* base, size_type idx, const sa_pack<T>& v) {
    if constexpr (sa_used<T>) {
        sa_pack<T>* p = base + idx;
        if constexpr (sizeof(sa_pack<T>) == 16) *(int4*)p = *(const int4*)&v;
        else if constexpr (sizeof(sa_pack<T>) == 8) *(int2*)p = *(const int2*)&v;
        else if constexpr (sizeof(sa_pack<T>) == 4) *(int*)p = *(const int*)&v;
        else if constexpr (sizeof(sa_pack<T>) == 2) *(short*)p = *(const short*)&v;
        else *p = v;
    }
}

template <typename T>
__device__ __forceinline__ void sa_discard(const sa_pack<T>* base, size_type idx, bool enabled) {
    if constexpr (sa_used<T>) {
        const sa_pack<T>* p = base + idx;
        // drops a whole 128-byte line from L2 without writing it back: only lines the kernel has consumed
        if (enabled && ((unsigned long long)p & 127ull) == 0) asm volatile("discard.global.L2 [%0], 128;" ::"l"(p) : "memory");
    }
}

struct SaJitArgs {
    size_type num_vecs;
    void* out[4];
    const void* in[4];
    int* mem;
    int val;
};

struct SaJitArrays {
    sa_pack<o0>* po0;
    sa_pack<o1>* po1;
    sa_pack<o2>* po2;
    sa_pack<o3>* po3;
    const sa_pack<i0>* pi0;
    const sa_pack<i1>* pi1;
    const sa_pack<i2>* pi2;
    const sa_pack<i3>* pi3;
};

// One 4 KiB chunk.  `whole` (every vector of the chunk exists: all chunks but the array's first and last) is the
// same for the whole warp and short-cuts the per-vector range test; measured faster than a chunk-local range test.
__device__ __forceinline__ void sa_process_chunk(const SaSched& s, const SaJitArgs& a, const SaJitArrays& p,
                                                 sa_u64 first_vec, sa_u32 lane) {
    sa_pack<o0>* const po0 = p.po0;
    sa_pack<o1>* const po1 = p.po1;
    sa_pack<o2>* const po2 = p.po2;
    sa_pack<o3>* const po3 = p.po3;
    const sa_pack<i0>* const pi0 = p.pi0;
    const sa_pack<i1>* const pi1 = p.pi1;
    const sa_pack<i2>* const pi2 = p.pi2;
    const sa_pack<i3>* const pi3 = p.pi3;
    const size_type v0 = (size_type)(first_vec - s.lead) + (size_type)lane; // may be "negative" in the first chunk
    const bool whole = first_vec >= s.lead && first_vec + SA_CHUNK_VECS <= s.end;
#pragma unroll 1
    for (int b = 0; b < SA_VEC_PER_LANE / sa_batch; ++b) {
        bool live[sa_batch];
        sa_pack<i0> r0[sa_batch];
        sa_pack<i1> r1[sa_batch];
        sa_pack<i2> r2[sa_batch];
        sa_pack<i3> r3[sa_batch];
#pragma unroll
        for (int j = 0; j < sa_batch; ++j) {
            const size_type vidx = v0 + (size_type)((b * sa_batch + j) * 32);
            live[j] = whole || (first_vec + (sa_u64)((b * sa_batch + j) * 32) + lane >= s.lead &&
                                first_vec + (sa_u64)((b * sa_batch + j) * 32) + lane < s.end);
            if (live[j]) {
                size_type x0 = 0, x1 = 0, x2 = 0, x3 = 0;
                live[j] = !indexing(vidx, vec_size, x0, x1, x2, x3, a.mem, a.val);
                if (live[j]) {
                    sa_load<input_evict[0]>(r0[j], pi0, x0);
                    sa_load<input_evict[1]>(r1[j], pi1, x1);
                    sa_load<input_evict[2]>(r2[j], pi2, x2);
                    sa_load<input_evict[3]>(r3[j], pi3, x3);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < sa_batch; ++j) {
            if (live[j]) {
                const size_type vidx = v0 + (size_type)((b * sa_batch + j) * 32);
                sa_pack<o0> w0;
                sa_pack<o1> w1;
                sa_pack<o2> w2;
                sa_pack<o3> w3;
                vector_op(vidx, vec_size, w0.v, w1.v, w2.v, w3.v, r0[j].v, r1[j].v, r2[j].v, r3[j].v, a.mem, a.val);
                sa_store(po0, vidx, w0);
                sa_store(po1, vidx, w1);
                sa_store(po2, vidx, w2);
                sa_store(po3, vidx, w3);
            }
        }
#ifdef DISCARD_INPUTS
        // after the stores of the batch; the input positions are computed again rather than kept
#pragma unroll
        for (int j = 0; j < sa_batch; ++j) {
            if (live[j]) {
                const size_type vidx = v0 + (size_type)((b * sa_batch + j) * 32);
                size_type x0 = 0, x1 = 0, x2 = 0, x3 = 0;
                indexing(vidx, vec_size, x0, x1, x2, x3, a.mem, a.val);
                sa_discard(pi0, x0, input_discard[0]);
                sa_discard(pi1, x1, input_discard[1]);
                sa_discard(pi2, x2, input_discard[2]);
                sa_discard(pi3, x3, input_discard[3]);
            }
        }
#endif
    }
}

extern "C" __global__ LAUNCH_BOUNDS void sideaware_elementwise(const __grid_constant__ SaSched launch,
                                                               const __grid_constant__ SaSideTable sides,
                                                               const __grid_constant__ SaJitArgs a) {
    // geometry follows the array that is moved in 16-byte vectors
    SaSched s = launch;
    sa_sched_geometry(s, (sa_u64)(sideaware_for_o0 ? a.out[0] : a.in[0]), (sa_u64)a.num_vecs, 0);
    s.reverse = reverse_order ? 1u : 0u;
    if (FORCE_WRONG_SIDE && s.hash) s.placement = SA_PLACE_WRONG;
    if (FORCE_RANDOM_SIDE) s.placement = SA_PLACE_UNAWARE;

    const sa_u32 lane = sa_lane();

    SaJitArrays arrays;
    arrays.po0 = (sa_pack<o0>*)a.out[0];
    arrays.po1 = (sa_pack<o1>*)a.out[1];
    arrays.po2 = (sa_pack<o2>*)a.out[2];
    arrays.po3 = (sa_pack<o3>*)a.out[3];
    arrays.pi0 = (const sa_pack<i0>*)a.in[0];
    arrays.pi1 = (const sa_pack<i1>*)a.in[1];
    arrays.pi2 = (const sa_pack<i2>*)a.in[2];
    arrays.pi3 = (const sa_pack<i3>*)a.in[3];
    sa_for_each_chunk(s, sides, [&](sa_u64 first_vec) {
        sa_process_chunk(s, a, arrays, first_vec, lane);
    });
}
