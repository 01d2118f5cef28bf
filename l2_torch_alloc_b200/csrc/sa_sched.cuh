// Work scheduler shared by every side-aware kernel (ahead-of-time and NVRTC).
//
// Data is cut into 8 KiB "double chunks" anchored at absolute 8 KiB address
// boundaries of the side-tracking array; the two 4 KiB halves of a double chunk
// always lie on opposite L2 sides (address bit 12 is part of the side hash).
// For each side there is a ticket counter in global memory; a warp running on
// an SM of side s repeatedly claims a ticket (a run of consecutive double
// chunks) from counter s and processes the halves homed on side s.  When its
// own side is drained it claims from the other counter, so every half is
// processed exactly once whatever the placement of thread blocks on SMs.
// Speed depends on the side table, correctness never does.
//
// The reference assigns work statically from a per-SM ordinal and requires one
// resident block per SM (sideaware.cu:205-213, 264-272, 286-305); its opt-in
// dynamic ordinal is sideaware.cu:215-236.  The pairing of chunk halves and the
// parity-of-masked-address side rule are the behaviour kept (sideaware.cu:292-305).
#pragma once

// Fixed-width names of our own: the same text is compiled by NVRTC next to user
// headers, which may or may not bring in <cstdint>.
typedef unsigned char sa_u8;
typedef unsigned int sa_u32;
typedef unsigned long long sa_u64;

#if defined(__CUDACC__) || defined(__CUDACC_RTC__)
#define SA_HD __host__ __device__ __forceinline__
#define SA_D __device__ __forceinline__
#else
#define SA_HD inline
#endif

#define SA_MAX_SM 256            // size of the per-SM side table carried in kernel parameters
#define SA_CHUNK_VECS 256u       // 4 KiB chunk in 16-byte vectors
#define SA_DC_VECS 512u          // 8 KiB double chunk in 16-byte vectors
#define SA_VEC_PER_LANE 8        // 16-byte vectors each lane of a warp moves per chunk

enum { SA_PLACE_AWARE = 0, SA_PLACE_UNAWARE = 1, SA_PLACE_WRONG = 2 };

// Launch-constant scheduling state, passed by value as a kernel parameter.
struct SaSched {
    sa_u32* tickets;        // [0]: next ticket side 0, [32]: next ticket side 1, [64]: warps finished
    sa_u64 anchor;          // address of vector 0 rounded down to 8 KiB (side hashing uses its low 32 bits)
    sa_u64 lead;            // vectors between the anchor and element 0 (0..511)
    sa_u64 end;             // lead + number of 16-byte vectors
    sa_u64 num_dc;          // double chunks covering [0, end)
    sa_u32 num_tickets;     // tickets per side
    sa_u32 dc_per_ticket;   // double chunks per ticket
    sa_u32 hash;            // side hash over byte-address bits (includes bit 21); 0 = unknown
    sa_u32 placement;       // SA_PLACE_*
    sa_u32 reverse;         // walk double chunks from the end
    sa_u32 total_warps;     // warps of the whole grid (for resetting the tickets)
    sa_u8 side_of_sm[SA_MAX_SM]; // bit 0 = side of the SM
};

SA_HD sa_u32 sa_parity32(sa_u32 v) {
#if defined(__CUDA_ARCH__)
    return __popc(v) & 1u;
#else
    v ^= v >> 16; v ^= v >> 8; v ^= v >> 4; v ^= v >> 2; v ^= v >> 1;
    return v & 1u;
#endif
}

// Side on which the FIRST 4 KiB half of double chunk `dc` is homed (as far as the
// hash can tell).  Both sides evaluate the same pure function of (dc, launch
// constants), so they always pick complementary halves.
SA_HD sa_u32 sa_first_half_side(const SaSched& s, sa_u64 dc) {
    sa_u32 side = 0;
    if (s.placement != SA_PLACE_UNAWARE) {
        sa_u32 lo = (sa_u32)(s.anchor + dc * 8192ull);
        side = sa_parity32(lo & s.hash);
        if (s.placement == SA_PLACE_WRONG) side ^= 1u;
    }
    return side;
}

// First vector (in anchored index space) of the 4 KiB half of the d-th double
// chunk of ticket `t` that a worker acting for side `s` must process; returns
// false when the ticket has no d-th double chunk.
SA_HD bool sa_ticket_chunk(const SaSched& s, sa_u32 t, sa_u32 d, sa_u32 side, sa_u64* first_vec) {
    sa_u64 k = (sa_u64)t * s.dc_per_ticket + d;
    if (k >= s.num_dc) return false;
    sa_u64 dc = s.reverse ? (s.num_dc - 1 - k) : k;
    sa_u32 half = sa_first_half_side(s, dc) ^ side;
    *first_vec = dc * SA_DC_VECS + half * SA_CHUNK_VECS;
    return true;
}

// Host side: fill the geometry fields for an array of `num_vecs` 16-byte vectors at `addr`.
SA_HD void sa_sched_geometry(SaSched& s, sa_u64 addr, sa_u64 num_vecs, sa_u32 warps_per_side) {
    s.anchor = addr & ~8191ull;
    s.lead = (addr & 8191ull) >> 4;
    s.end = s.lead + num_vecs;
    s.num_dc = (s.end + SA_DC_VECS - 1) / SA_DC_VECS;
    // aim at >= 8 tickets per warp and side, 1..8 double chunks (8..64 KiB) per ticket;
    // a preset dc_per_ticket is kept (kernels that redo the geometry for another array)
    sa_u64 per = s.dc_per_ticket;
    if (per == 0) {
        per = warps_per_side ? s.num_dc / ((sa_u64)warps_per_side * 8u) : 1;
        if (per < 1) per = 1;
        if (per > 8) per = 8;
    }
    s.dc_per_ticket = (sa_u32)per;
    s.num_tickets = (sa_u32)((s.num_dc + per - 1) / per);
}

#if defined(__CUDACC__) || defined(__CUDACC_RTC__)

SA_D sa_u32 sa_smid() {
    sa_u32 v;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
    return v;
}

SA_D sa_u32 sa_lane() { return threadIdx.x & 31u; }

// One claim per warp: lane 0 takes the ticket, everybody gets it.
SA_D sa_u32 sa_claim(const SaSched& s, sa_u32 side) {
    sa_u32 t = 0;
    if (sa_lane() == 0) t = atomicAdd(s.tickets + side * 32u, 1u);
    return __shfl_sync(0xffffffffu, t, 0);
}

// Last warp out rewinds the counters for the next launch that uses this slot.
// Every other warp made its final claim before it incremented the finish
// counter, so nothing can touch the counters after the reset.
SA_D void sa_finish(const SaSched& s) {
    if (sa_lane() == 0) {
        sa_u32 done = atomicAdd(s.tickets + 64, 1u);
        if (done == s.total_warps - 1u) {
            s.tickets[0] = 0;
            s.tickets[32] = 0;
            __threadfence();
            s.tickets[64] = 0;
        }
    }
}

// Runs `body(first_vec)` for every 4 KiB half this warp is responsible for.
// `first_vec` is in anchored vector index space: element index = first_vec - lead;
// vectors outside [lead, end) do not exist (only possible in the first and last
// double chunk).  All 32 lanes call body together.
template <class Body>
SA_D void sa_for_each_chunk(const SaSched& s, Body&& body) {
    sa_u32 smid = sa_smid();
    sa_u32 my_side = (smid < SA_MAX_SM) ? (s.side_of_sm[smid] & 1u) : 0u;
#pragma unroll 1
    for (sa_u32 pass = 0; pass < 2; ++pass) {
        sa_u32 side = my_side ^ pass;
        sa_u32 t = sa_claim(s, side);
#pragma unroll 1
        while (t < s.num_tickets) {
            sa_u32 next = sa_claim(s, side); // in flight while this ticket is processed
#pragma unroll 1
            for (sa_u32 d = 0; d < s.dc_per_ticket; ++d) {
                sa_u64 first_vec;
                if (!sa_ticket_chunk(s, t, d, side, &first_vec)) break;
                if (first_vec < s.end && first_vec + SA_CHUNK_VECS > s.lead) body(first_vec);
            }
            t = next;
        }
    }
    sa_finish(s);
}

#endif // __CUDACC__
