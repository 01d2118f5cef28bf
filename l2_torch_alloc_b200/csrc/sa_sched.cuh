// Work scheduler shared by every side-aware kernel (ahead-of-time and NVRTC).
//
// Data is cut into 8 KiB "double chunks" anchored at absolute 8 KiB address
// boundaries of the side-tracking array; the two 4 KiB halves of a double chunk
// always lie on opposite L2 sides (address bit 12 is part of the side hash).
// For each side there is a ticket counter in global memory; a ticket is a run of
// consecutive double chunks, and whoever holds ticket t of side s processes, of each
// of its double chunks, the half homed on side s.  Blocks take tickets of their own
// SM's side first and sweep up the other side's leftovers at the end, so every half
// is processed exactly once whatever the placement of thread blocks on SMs.
// Speed depends on the side table, correctness never does.  How tickets are handed
// out with few atomics is described at sa_for_each_chunk.
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
#ifndef SA_STATIC_SHARE_PCT
#define SA_STATIC_SHARE_PCT 60   // large arrays: percentage of the tickets dealt out in the blocks' opening batches
#endif
#ifndef SA_DYNAMIC_FROM
#define SA_DYNAMIC_FROM 8        // per-warp claims are used from this many tickets per warp and side on (4 measured:
                                 // 48 MiB copies 9-13 % slower, nothing else faster)
#endif

enum { SA_PLACE_AWARE = 0, SA_PLACE_UNAWARE = 1, SA_PLACE_WRONG = 2 };

// Launch-constant scheduling state, passed by value as a kernel parameter.
struct SaSched {
    sa_u32* tickets;        // [0]: next ticket side 0, [32]: next ticket side 1, [64]: blocks finished
    sa_u64 anchor;          // address of vector 0 rounded down to 8 KiB (side hashing uses its low 32 bits)
    sa_u64 lead;            // vectors between the anchor and element 0 (0..511)
    sa_u64 end;             // lead + number of 16-byte vectors
    sa_u64 num_dc;          // double chunks covering [0, end)
    sa_u32 num_tickets;     // tickets per side
    sa_u32 dc_per_ticket;   // double chunks per ticket
    sa_u32 hash;            // side hash over byte-address bits (includes bit 21); 0 = unknown
    sa_u32 placement;       // SA_PLACE_*
    sa_u32 reverse;         // walk double chunks from the end
    sa_u32 total_blocks;    // blocks of the grid (the last one to finish rewinds the tickets)
    sa_u32 active_warps;    // warps per block that take part (small arrays do not need all of them)
    sa_u32 share;           // most tickets an active warp takes from its block's opening batch (no atomics)
    sa_u32 opening[2];      // tickets a block on side 0 / side 1 takes with its opening atomic (<= active_warps * share)
    sa_u32 dynamic;         // 1: after the share, warps claim single tickets for themselves (large arrays)
    sa_u32 overlap;         // host side only: 1 = the launch may begin while its predecessor on the stream drains
};

// Side of every SM (bit 0 of the byte), a kernel parameter of its own so that kernels which
// adjust a private copy of SaSched do not drag 256 bytes through local memory.
struct SaSideTable {
    sa_u8 side_of_sm[SA_MAX_SM];
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
    // Ticket length.  Short tickets keep the end of the kernel even (the last ticket of a warp is
    // time the other warps may sit idle), long tickets keep the claim rate down: at full HBM speed
    // one-double-chunk tickets would mean a same-address atomic every ~6 ns per side.  Aim at >= 24
    // tickets per warp and side, 1..8 double chunks (8..64 KiB) per ticket, and at least 2 once the
    // array is large enough for per-warp claims.  A preset dc_per_ticket is kept (kernels that redo
    // the geometry for another array).  (One-double-chunk tickets for all fully dealt arrays, which
    // deal out more evenly, were measured: nothing gained at 8-56 MiB, 2-8 % lost at 64-72 MiB.)
    sa_u64 per = s.dc_per_ticket;
    if (per == 0) {
        per = warps_per_side ? s.num_dc / ((sa_u64)warps_per_side * 24u) : 1;
        if (per < 1) per = 1;
        if (per > 8) per = 8;
        if (per < 2 && warps_per_side && s.num_dc >= 4ull * warps_per_side) per = 2;
    }
    s.dc_per_ticket = (sa_u32)per;
    s.num_tickets = (sa_u32)((s.num_dc + per - 1) / per);
}

// Host side: grid size and how the tickets are handed out, for a launch with `warps`
// warps per block on at most `max_blocks` blocks.
//  * large arrays (>= 8 tickets per warp and side): every warp of every block takes part;
//    about 60 % of the tickets are dealt out statically in each block's opening batch, the
//    rest is claimed ticket by ticket so faster SMs do more;
//  * small arrays: all tickets are dealt out in the opening batches (the per-ticket atomics
//    would cost more than the copy), spread over all blocks with only as many warps each as
//    there is work for; tiny ones get one block per ticket.
// Whatever an uneven SM split or a busy SM leaves over is swept up block-wide at the end.
SA_HD void sa_sched_grid(SaSched& s, int max_blocks, int warps, int* grid, int sms_side0 = -1, int sms_side1 = -1) {
    sa_u64 total = 2ull * s.num_tickets;
    int g = max_blocks < 1 ? 1 : max_blocks;
    if (total < (sa_u64)g) g = (int)(total ? total : 1);
    // blocks that will work for each side: the SM counts of the sides when the grid has one block per SM
    // (the two dies need not have equally many SMs), else half the grid each
    sa_u64 blocks[2] = {(sa_u64)(g + 1) / 2, (sa_u64)(g + 1) / 2};
    if (sms_side0 > 0 && sms_side1 > 0 && sms_side0 + sms_side1 == g) {
        blocks[0] = (sa_u64)sms_side0;
        blocks[1] = (sa_u64)sms_side1;
    }
    const sa_u64 fewer = blocks[0] < blocks[1] ? blocks[0] : blocks[1];
    const sa_u64 M = s.num_tickets;
    if (M >= (sa_u64)SA_DYNAMIC_FROM * fewer * (sa_u64)warps) {
        s.active_warps = (sa_u32)warps;
        const sa_u64 more = blocks[0] < blocks[1] ? blocks[1] : blocks[0];
        sa_u64 share = (M * SA_STATIC_SHARE_PCT / 100) / (more * (sa_u64)warps);
        s.share = (sa_u32)(share < 1 ? 1 : share);
        s.opening[0] = s.opening[1] = s.share * s.active_warps;
        s.dynamic = 1;
    } else {
        // everything is dealt out at the start: a block of side i takes its even share of that side's tickets
        sa_u64 per_block[2], most = 1;
        for (int i = 0; i < 2; ++i) {
            per_block[i] = (M + blocks[i] - 1) / blocks[i];
            if (per_block[i] < 1) per_block[i] = 1;
            if (per_block[i] > most) most = per_block[i];
        }
        sa_u64 active = most > (sa_u64)warps ? (sa_u64)warps : most;
        s.active_warps = (sa_u32)active;
        s.share = (sa_u32)((most + active - 1) / active);
        s.opening[0] = (sa_u32)per_block[0];
        s.opening[1] = (sa_u32)per_block[1];
        s.dynamic = 0;
    }
    s.total_blocks = (sa_u32)g;
    *grid = g;
}

#if defined(__CUDACC__) || defined(__CUDACC_RTC__)

SA_D sa_u32 sa_smid() {
    sa_u32 v;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
    return v;
}

SA_D sa_u32 sa_lane() { return threadIdx.x & 31u; }

// Runs `body(first_vec)` for every 4 KiB half this warp is responsible for.
// `first_vec` is in anchored vector index space: element index = first_vec - lead;
// vectors outside [lead, end) do not exist (only possible in the first and last
// double chunk).  All 32 lanes call body together; every thread of the block must
// call this function exactly once (it contains block-wide barriers).
//
// Same-address atomics are the scarce resource (an L2 slice retires one every few
// cycles), so they are kept few and off the critical path:
//  1. a block opens with ONE atomic that takes opening[side] tickets (at most share x active_warps);
//     warp w works on tickets base + w, base + w + active_warps, ... (neighbouring warps, neighbouring memory;
//     rotating the warps from round to round, against periodic patterns such as RoPE's V heads, was measured: no gain);
//  2. for large arrays each warp then claims single tickets for itself, always one ahead of
//     the ticket it is working on (the result is only looked at after that ticket is done);
//  3. leftovers of both sides (uneven SM split, a busy SM) are taken by the block as a whole,
//     one atomic per side per batch of active_warps tickets, both in flight together;
//     (putting the first sweep's claims in flight during a warp's last dealt ticket was measured: no gain);
//  4. one atomic per block counts finished blocks; the last one rewinds the counters, so a launch leaves its
//     slot as it found it (a kernel recorded in a CUDA graph can be replayed).
template <class Body>
SA_D void sa_for_each_chunk(const SaSched& s, const SaSideTable& sides, Body&& body) {
    __shared__ sa_u32 sa_batch;
    __shared__ sa_u32 sa_batch_other;
    __shared__ sa_u32 sa_drained;
    const sa_u32 smid = sa_smid();
    const sa_u32 my_side = (smid < SA_MAX_SM) ? (sides.side_of_sm[smid] & 1u) : 0u;
    const sa_u32 warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const bool active = warp < s.active_warps;
    const sa_u32 M = s.num_tickets;
    const sa_u32 none = 0xffffffffu;
    sa_u32* const own = s.tickets + my_side * 32u;
    sa_u32* const other = s.tickets + (my_side ^ 1u) * 32u;
    // lane 0 puts a claim in flight; nobody waits for it here
    auto claim_issue = [&]() -> sa_u32 {
        sa_u32 r = none;
        if (lane == 0 && !*(volatile sa_u32*)&sa_drained) r = atomicAdd(own, 1u);
        return r;
    };

    // Programmatic dependent launch: let the next kernel of the stream start its own prologue as
    // soon as this grid's blocks have all come this far, and do not touch data before the previous
    // kernel has completed and flushed.  Both are no-ops for launches without that attribute.  The
    // opening claim only touches this launch's own ticket slot, so it may precede the wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        sa_drained = 0u;
        sa_batch = atomicAdd(own, s.opening[my_side]);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    const sa_u32 base = sa_batch;
    // One loop with a single place where tickets are worked on (the body is inlined once):
    // phase 0 = tickets dealt from the opening batch, 1 = own claims, 2 = block-wide leftovers.
    sa_u32 phase = active ? 0u : 2u;
    sa_u32 dealt = 0, pending = none, second = none;
#pragma unroll 1
    for (;;) {
        sa_u32 t = none, side = my_side;
        if (phase == 0u) {
            const sa_u32 mine = dealt * s.active_warps + warp; // position in the block's opening batch
            if (dealt == s.share || mine >= s.opening[my_side]) {
                phase = s.dynamic ? 1u : 2u;
                continue;
            }
            t = base + mine;
            ++dealt;
            if (s.dynamic && dealt == s.share) pending = claim_issue(); // overlaps the last dealt ticket
        } else if (phase == 1u) {
            t = __shfl_sync(0xffffffffu, pending, 0);
            if (t >= M) {
                if (lane == 0 && t != none) *(volatile sa_u32*)&sa_drained = 1u; // spare the others the failing claim
                phase = 2u;
                continue;
            }
            pending = claim_issue(); // in flight while ticket t is worked on
        } else if (second != none) {
            t = second; // the other side's ticket of the current leftover batch
            side = my_side ^ 1u;
            second = none;
        } else {
            __syncthreads(); // everybody has finished with the previous batch numbers
            if (threadIdx.x == 0) {
                // the two claims travel together, so finding nothing left costs one round trip
                sa_u32 a = atomicAdd(own, s.active_warps);
                sa_u32 b = atomicAdd(other, s.active_warps);
                sa_batch = a;
                sa_batch_other = b;
            }
            __syncthreads();
            const sa_u32 base_own = sa_batch, base_other = sa_batch_other;
            if (base_own >= M && base_other >= M) break;
            if (active) {
                t = base_own + warp;
                if (base_other + warp < M) second = base_other + warp;
            }
        }
        if (t < M) {
#pragma unroll 1
            for (sa_u32 d = 0; d < s.dc_per_ticket; ++d) {
                sa_u64 first_vec;
                if (!sa_ticket_chunk(s, t, d, side, &first_vec)) break;
                if (first_vec < s.end && first_vec + SA_CHUNK_VECS > s.lead) body(first_vec);
            }
        }
    }
    // Thread 0 made this block's final claim above and no other thread claims any more, so
    // nothing can touch the counters after the last block's reset.
    if (threadIdx.x == 0) {
        sa_u32 done = atomicAdd(s.tickets + 64, 1u);
        if (done == s.total_blocks - 1u) {
            s.tickets[0] = 0;
            s.tickets[32] = 0;
            __threadfence();
            s.tickets[64] = 0;
        }
    }
}

#endif // __CUDACC__
