// memcpy engine 1: bulk asynchronous copies (the TMA unit's untiled cp.async.bulk) staged
// through shared memory.  A 4 KiB chunk is homed on one L2 side and is exactly one bulk copy:
// global -> shared (completion counted on an mbarrier), then shared -> global.  One lane per
// warp drives the copies, so the SM issues a handful of instructions per 4 KiB instead of the
// sixteen 128-bit loads and stores per lane of the vector engine.  No cluster multicast is
// used anywhere (every copy is global <-> this block's own shared memory).
//
// Pipeline per warp: two 4 KiB stages.  On chunk n the warp first puts the load of chunk n
// in flight, then waits for chunk n-1, and sends it out; 16 warps keep up to 128 KiB per SM
// in flight.  Which chunks a warp takes is decided by sa_sched.cuh, as for every kernel.
//
// Every wait is bounded: if an mbarrier does not complete within the limit the warp records
// it in the launch's error word (4th line of the ticket slot), skips that store and carries on.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdlib>

#include "sa_kernels.hpp"

namespace {

constexpr uint32_t kChunkBytes = 4096;
constexpr uint32_t kSpinLimit = 1u << 18; // try_wait rounds (each may suspend for a while): about a second, not forever

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// hinted = true: the line is marked evict-first in L2 (streamed data is not read again)
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar, bool hinted,
                                          uint64_t policy) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    if (hinted)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                     ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
                     : "memory");
    else
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
                     : "memory");
}

// true when the phase with the given parity has completed
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t ok;
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

__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes, bool hinted, uint64_t policy) {
    if (hinted)
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
                     ::"l"(dst), "r"(src_smem), "r"(bytes), "l"(policy)
                     : "memory");
    else
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// at most N of the most recently committed stores may still be READING shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

// WARPS warps per block, S stages of 4 KiB per warp.  A warp keeps L = S - 2 loads in flight
// (1 when S == 2); the spare stage lets the newest store still read shared memory while the
// next load is issued.
template <int WARPS, int S>
__global__ void __launch_bounds__(WARPS * 32, 1)
sa_memcpy_bulk_kernel(const __grid_constant__ SaSched s, const __grid_constant__ SaSideTable sides,
                      uint4* __restrict__ dst, const uint4* __restrict__ src, int hints) {
    const uint64_t policy = l2_evict_first_policy();
    const bool hint_load = hints & 1, hint_store = hints & 2;
    constexpr uint32_t L = S >= 3 ? S - 2 : 1;
    extern __shared__ __align__(128) unsigned char stage_mem[]; // [warps][stages][4 KiB]
    __shared__ __align__(8) unsigned long long bars[WARPS * S];
    __shared__ uint4* dsts[WARPS * S];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t my_stage0 = smem_addr(stage_mem) + warp * S * kChunkBytes;
    const uint32_t my_bar0 = smem_addr(&bars[warp * S]);
    uint4** const my_dsts = &dsts[warp * S];
    if (lane == 0) {
        for (int i = 0; i < S; ++i) mbar_init(my_bar0 + 8u * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // pipeline state of lane 0
    uint32_t issued = 0, retired = 0;
    uint32_t phase_bits = 0; // bit i = parity the next wait on stage i expects

    auto retire = [&]() { // wait for the oldest chunk in flight and send it out
        const uint32_t st = retired % S;
        if (mbar_wait(my_bar0 + 8u * st, (phase_bits >> st) & 1u)) {
            bulk_store(my_dsts[st], my_stage0 + st * kChunkBytes, kChunkBytes, hint_store, policy);
        } else {
            atomicAdd(s.tickets + 96, 1u); // reported by the host; the copy is incomplete
        }
        phase_bits ^= 1u << st;
        ++retired;
    };

    sa_for_each_chunk(s, sides, [&](uint64_t first_vec) {
        if (first_vec >= s.lead && first_vec + SA_CHUNK_VECS <= s.end) {
            if (lane == 0) {
                const uint64_t e = first_vec - s.lead;
                const uint32_t st = issued % S;
                // the store that last used this stage (S chunks ago) must have read it
                bulk_wait_read<(S >= 3 ? 1 : 0)>();
                bulk_load(my_stage0 + st * kChunkBytes, src + e, kChunkBytes, my_bar0 + 8u * st, hint_load, policy);
                my_dsts[st] = dst + e;
                ++issued;
                while (issued - retired > L) retire(); // older chunks go out while newer ones come in
            }
        } else {
            // first or last chunk of the array: plain per-vector copy by the whole warp
#pragma unroll 1
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                uint64_t v = first_vec + k * 32 + lane;
                if (v >= s.lead && v < s.end) dst[v - s.lead] = __ldcs(src + (v - s.lead));
            }
        }
    });
    if (lane == 0) {
        while (retired < issued) retire();
        bulk_wait_read<0>(); // shared memory must stay valid until the last store has read it
    }
}

template <int WARPS, int S>
cudaError_t launch_cfg(const SaSched& s, const SaSideTable& sides, int grid, void* dst, const void* src, cudaStream_t stream) {
    constexpr int smem = WARPS * S * (int)kChunkBytes;
    // once per device: the attribute belongs to the current device's copy of the function
    static std::atomic<bool> opted_in[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !opted_in[dev].load(std::memory_order_acquire)) {
        cudaError_t attr = cudaFuncSetAttribute(sa_memcpy_bulk_kernel<WARPS, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (attr != cudaSuccess) return attr;
        if (dev >= 0 && dev < 64) opted_in[dev].store(true, std::memory_order_release);
    }
    static const int hints = [] { // tuning aid: SIDEAWARE_BULK_HINTS bit 0 = evict-first loads, bit 1 = evict-first stores
        const char* e = std::getenv("SIDEAWARE_BULK_HINTS");
        return e ? std::atoi(e) & 3 : 0;
    }();
    SaLaunch l(s, grid, WARPS * 32, smem, stream);
    return cudaLaunchKernelEx(&l.cfg, sa_memcpy_bulk_kernel<WARPS, S>, s, sides, (uint4*)dst, (const uint4*)src, hints);
}

// default shape; SIDEAWARE_BULK_CFG=<n> picks another one for tuning
struct BulkCfg { int warps, stages; };
const BulkCfg kCfgs[] = {{8, 4}, {16, 3}, {16, 2}, {8, 6}, {24, 2}, {12, 4}, {8, 7}};
int chosen_cfg() {
    static const int c = [] {
        const char* e = std::getenv("SIDEAWARE_BULK_CFG");
        int v = e ? std::atoi(e) : 0;
        return (v >= 0 && v < 7) ? v : 0;
    }();
    return c;
}

} // namespace

cudaError_t sa_launch_memcpy_bulk(const SaSched& s, const SaSideTable& sides, int grid, void* dst, const void* src,
                                  cudaStream_t stream) {
    switch (chosen_cfg()) {
        case 1: return launch_cfg<16, 3>(s, sides, grid, dst, src, stream);
        case 2: return launch_cfg<16, 2>(s, sides, grid, dst, src, stream);
        case 3: return launch_cfg<8, 6>(s, sides, grid, dst, src, stream);
        case 4: return launch_cfg<24, 2>(s, sides, grid, dst, src, stream);
        case 5: return launch_cfg<12, 4>(s, sides, grid, dst, src, stream);
        case 6: return launch_cfg<8, 7>(s, sides, grid, dst, src, stream);
        default: return launch_cfg<8, 4>(s, sides, grid, dst, src, stream); // best balance over 16 MiB .. 4 GiB in the sweep
    }
}

int sa_memcpy_bulk_warps() { return kCfgs[chosen_cfg()].warps; }
