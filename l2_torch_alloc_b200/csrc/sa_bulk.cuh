// Bulk asynchronous copies (the TMA unit's untiled cp.async.bulk) between global memory and a
// block's own shared memory, and the bookkeeping of a per-warp ring of 4 KiB stages.
// Shared by the memcpy and RoPE kernels that stage chunks through shared memory.
//
// No copy here is a cluster multicast: every transfer is global <-> this block's shared memory.
// Every wait on an mbarrier is bounded.  What a warp does after a wait has run out is decided
// by SaStageRing below, which is plain arithmetic and is tested on the host.
#pragma once
#include "sa_sched.cuh"

// Ring of S stages owned by one warp.  Loads are issued into stage (issued % S) and retired in
// order.  A stage's mbarrier completes one phase per load; phase_bits holds, per stage, the
// parity the next wait on that stage expects.
//
// After the FIRST wait that runs out the ring is `failed`: no further load is issued (the
// caller moves the remaining chunks with ordinary loads and stores), every load still in
// flight gets one more bounded wait when it is retired, and a stage whose wait ran out is
// remembered in `lost`: its barrier never completed the phase, so its parity is not flipped
// and the barrier is never armed again; the chunk it held is done again by the caller.
struct SaStageRing {
    sa_u32 issued;
    sa_u32 retired;
    sa_u32 phase_bits;
    sa_u32 failed;  // 0 / 1
    sa_u32 lost;    // bit i: the load into stage i never arrived
};

SA_HD void sa_ring_reset(SaStageRing& r) { r.issued = r.retired = r.phase_bits = r.failed = r.lost = 0u; }
SA_HD bool sa_ring_may_issue(const SaStageRing& r) { return r.failed == 0u; }
SA_HD sa_u32 sa_ring_in_flight(const SaStageRing& r) { return r.issued - r.retired; }
// stage the next load goes into; the caller issues the load into it
SA_HD sa_u32 sa_ring_issue(SaStageRing& r, sa_u32 stages) {
    sa_u32 st = r.issued % stages;
    ++r.issued;
    return st;
}
SA_HD sa_u32 sa_ring_oldest(const SaStageRing& r, sa_u32 stages) { return r.retired % stages; }
SA_HD sa_u32 sa_ring_oldest_parity(const SaStageRing& r, sa_u32 stages) { return (r.phase_bits >> (r.retired % stages)) & 1u; }
// the oldest load has been waited for: `arrived` says whether its data is there
SA_HD void sa_ring_retire(SaStageRing& r, sa_u32 stages, bool arrived) {
    const sa_u32 st = r.retired % stages;
    if (arrived) {
        r.phase_bits ^= 1u << st;
    } else {
        r.failed = 1u;
        r.lost |= 1u << st;
    }
    ++r.retired;
}

#if defined(__CUDACC__) || defined(__CUDACC_RTC__)

#define SA_BULK_CHUNK_BYTES 4096u
#define SA_BULK_SPIN_LIMIT (1u << 18) // try_wait rounds (each may suspend for a while): about a second, not forever

SA_D sa_u32 sa_smem_addr(const void* p) { return (sa_u32)__cvta_generic_to_shared(p); }

SA_D void sa_mbar_init(sa_u32 bar, sa_u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
SA_D void sa_mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// announces `bytes` on the barrier; the loads that deliver them follow
SA_D void sa_mbar_expect(sa_u32 bar, sa_u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// global -> shared; completion is counted in bytes on `bar`.  16-byte aligned addresses, size a multiple of 16.
SA_D void sa_bulk_load(sa_u32 dst_smem, const void* src, sa_u32 bytes, sa_u32 bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// true when the phase with the given parity has completed within the limit
SA_D bool sa_mbar_wait(sa_u32 bar, sa_u32 parity) {
    for (sa_u32 spin = 0; spin < SA_BULK_SPIN_LIMIT; ++spin) {
        sa_u32 ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// shared -> global, one bulk group per call sequence ended by sa_bulk_commit
SA_D void sa_bulk_store(void* dst, sa_u32 src_smem, sa_u32 bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
SA_D void sa_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// at most N of the most recently committed store groups may still be READING shared memory
template <int N>
SA_D void sa_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

// orders this thread's ordinary shared-memory writes before later bulk (async proxy) reads of them
SA_D void sa_fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

#endif // __CUDACC__
