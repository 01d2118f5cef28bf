// memcpy engine 1: bulk asynchronous copies (the TMA unit's untiled cp.async.bulk) staged
// through shared memory.  A 4 KiB chunk is homed on one L2 side and is exactly one bulk copy:
// global -> shared (completion counted on an mbarrier), then shared -> global.  One lane per
// warp drives the copies, so the SM issues a handful of instructions per 4 KiB instead of the
// sixteen 128-bit loads and stores per lane of the vector engine.  No cluster multicast is
// used anywhere (every copy is global <-> this block's own shared memory).
//
// Shape: 8 warps per block, each with a ring of four 4 KiB stages (128 KiB of shared memory per
// SM).  A warp keeps two loads in flight: on chunk n it puts the load of chunk n in flight,
// then waits for chunk n-2 and sends it out; the fourth stage lets the newest store still
// read shared memory while the next load is issued.  Which chunks a warp takes is decided by
// sa_sched.cuh, as for every kernel.
//
// Every wait is bounded (sa_bulk.cuh).  When a wait runs out the warp counts it in the
// device's wait-error word (host-visible), issues no further bulk load, gives the loads it
// still has in flight one more bounded wait each, and moves every chunk whose data did not
// arrive, and all its later chunks, with ordinary loads and stores: the copy still completes.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "sa_bulk.cuh"
#include "sa_kernels.hpp"

namespace {

constexpr int kWarps = 8;
constexpr int kStages = 4;
constexpr uint32_t kLoadsInFlight = kStages - 2;

// plain copy of one whole or partial chunk by all lanes of the warp
__device__ __forceinline__ void copy_chunk_plain(const SaSched& s, uint4* dst, const uint4* src, uint64_t first_vec, uint32_t lane) {
#pragma unroll 1
    for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
        uint64_t v = first_vec + k * 32 + lane;
        if (v >= s.lead && v < s.end) dst[v - s.lead] = __ldcs(src + (v - s.lead));
    }
}

__global__ void __launch_bounds__(kWarps * 32, 1)
sa_memcpy_bulk_kernel(const __grid_constant__ SaSched s, const __grid_constant__ SaSideTable sides,
                      uint4* __restrict__ dst, const uint4* __restrict__ src, uint32_t* wait_errors) {
    constexpr uint32_t S = kStages;
    extern __shared__ __align__(128) unsigned char stage_mem[]; // [warps][stages][4 KiB]
    __shared__ __align__(8) unsigned long long bars[kWarps * S];
    __shared__ uint64_t chunk_of_stage[kWarps * S];              // anchored index of the chunk's first vector
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t my_stage0 = sa_smem_addr(stage_mem) + warp * S * SA_BULK_CHUNK_BYTES;
    const uint32_t my_bar0 = sa_smem_addr(&bars[warp * S]);
    uint64_t* const my_chunks = &chunk_of_stage[warp * S];
    if (lane == 0) {
        for (uint32_t i = 0; i < S; ++i) sa_mbar_init(my_bar0 + 8u * i, 1);
        sa_mbar_fence_init();
    }
    __syncwarp();

    SaStageRing ring; // meaningful in lane 0 only
    sa_ring_reset(ring);

    auto retire = [&]() { // lane 0: wait for the oldest chunk in flight and send it out
        const uint32_t st = sa_ring_oldest(ring, S);
        const bool arrived = sa_mbar_wait(my_bar0 + 8u * st, sa_ring_oldest_parity(ring, S));
        if (arrived) {
            sa_bulk_store(dst + (my_chunks[st] - s.lead), my_stage0 + st * SA_BULK_CHUNK_BYTES, SA_BULK_CHUNK_BYTES);
            sa_bulk_commit();
        } else {
            atomicAdd_system(wait_errors, 1u);
        }
        sa_ring_retire(ring, S, arrived);
    };

    sa_for_each_chunk(s, sides, [&](uint64_t first_vec) {
        const bool whole = first_vec >= s.lead && first_vec + SA_CHUNK_VECS <= s.end;
        const bool bulk = whole && __shfl_sync(0xffffffffu, ring.failed, 0) == 0u;
        if (bulk) {
            if (lane == 0) {
                // the store that last used this stage (S chunks ago) must have read it
                sa_bulk_wait_read<1>();
                const uint32_t st = sa_ring_issue(ring, S);
                const uint32_t bar = my_bar0 + 8u * st;
                sa_mbar_expect(bar, SA_BULK_CHUNK_BYTES);
                sa_bulk_load(my_stage0 + st * SA_BULK_CHUNK_BYTES, src + (first_vec - s.lead), SA_BULK_CHUNK_BYTES, bar);
                my_chunks[st] = first_vec;
                while (sa_ring_in_flight(ring) > kLoadsInFlight) retire(); // older chunks go out while newer ones come in
            }
        } else {
            // first or last chunk of the array, or this warp has given up on bulk copies
            copy_chunk_plain(s, dst, src, first_vec, lane);
        }
    });
    if (lane == 0) {
        while (sa_ring_in_flight(ring) > 0) retire();
        sa_bulk_wait_read<0>(); // shared memory must stay valid until the last store has read it
    }
    // chunks whose data never arrived (only after a wait ran out): all lanes redo them
    const uint32_t lost = __shfl_sync(0xffffffffu, ring.lost, 0);
    if (lost) {
        __syncwarp();
        for (uint32_t st = 0; st < S; ++st)
            if ((lost >> st) & 1u) copy_chunk_plain(s, dst, src, my_chunks[st], lane);
    }
}

} // namespace

cudaError_t sa_launch_memcpy_bulk(const SaSched& s, const SaSideTable& sides, int grid, void* dst, const void* src,
                                  uint32_t* wait_errors, cudaStream_t stream) {
    constexpr int smem = kWarps * kStages * (int)SA_BULK_CHUNK_BYTES;
    // once per device: the attribute belongs to the current device's copy of the function
    static std::atomic<bool> opted_in[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !opted_in[dev].load(std::memory_order_acquire)) {
        cudaError_t attr = cudaFuncSetAttribute(sa_memcpy_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (attr != cudaSuccess) return attr;
        if (dev >= 0 && dev < 64) opted_in[dev].store(true, std::memory_order_release);
    }
    SaLaunch l(s, grid, kWarps * 32, smem, stream);
    return cudaLaunchKernelEx(&l.cfg, sa_memcpy_bulk_kernel, s, sides, (uint4*)dst, (const uint4*)src, wait_errors);
}

int sa_memcpy_bulk_warps() { return kWarps; }
