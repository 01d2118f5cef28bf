// RoPE engine 1: the in-place rotation staged through shared memory with bulk asynchronous
// copies (the TMA unit's untiled cp.async.bulk; no cluster multicast anywhere).
//
// A 4 KiB chunk of the packed [B, T, Nq + 2 Nkv, HS] tensor is homed on one L2 side.  Of each
// chunk only the Q and K parts are brought in: with rows of at least 4 KiB a chunk touches at
// most two token rows, so its rotated vectors are at most two contiguous runs, "A" in the row
// the chunk starts in and "B" at the start of the next row; V vectors are neither loaded nor
// stored, and a chunk that holds only V is skipped.  Per chunk the warp
//   1. lane 0: announces the bytes on the stage's mbarrier and issues one bulk load per run,
//   2. later, all lanes: wait for the barrier (bounded), rotate the vectors in shared memory
//      with 128-bit ld.shared / st.shared (cos/sin from the table through the read-only path),
//   3. lane 0: one bulk store per run back to the same global addresses.
// Every warp has a ring of S stages and keeps S - 2 loads in flight ahead of the chunk it rotates.
// Which chunks a warp takes is decided by sa_sched.cuh, as for every kernel.
//
// Chunks at the ends of the array, shapes whose rows are shorter than a chunk, and everything
// after a wait that ran out (sa_bulk.cuh) go through ordinary loads and stores.
//
// Same arithmetic as the vector kernel (sa_rope_math.cuh): bit-identical results.
// Replaces the reference's JIT-ed template with kernel_rope.cuh:1-60.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "sa_bulk.cuh"
#include "sa_kernels.hpp"
#include "sa_rope_math.cuh"

#ifndef SA_ROPE_BULK_WARPS
#define SA_ROPE_BULK_WARPS 16
#endif
#ifndef SA_ROPE_BULK_STAGES
#define SA_ROPE_BULK_STAGES 3
#endif

namespace {

constexpr int kWarps = SA_ROPE_BULK_WARPS;
constexpr int kStages = SA_ROPE_BULK_STAGES;
constexpr uint32_t kLoadsInFlight = kStages - 2 > 0 ? kStages - 2 : 1;
// store groups committed after the one that last read a stage, when that stage is loaded into again
constexpr int kPendingStoreGroups = kStages - 1 - (int)kLoadsInFlight;

// where a chunk lies in its token row, kept per stage between the load and the rotation
struct StageInfo {
    uint64_t first_vec; // anchored index of the chunk's first vector
    uint32_t r0;        // position of that vector in its row, in vectors
    uint32_t tok0;      // token of that row
};

// the two runs of rotated vectors of a chunk that starts at row position r0 (chunk-local, in vectors)
struct Runs {
    uint32_t a_end;          // A = [0, a_end)
    uint32_t b_begin, b_end; // B = [b_begin, b_end); empty when b_begin >= b_end
};

__device__ __forceinline__ Runs chunk_runs(const SaRopeShape& sh, uint32_t r0) {
    Runs r;
    const uint32_t left = sh.rotated_vecs > r0 ? sh.rotated_vecs - r0 : 0u;
    r.a_end = left < SA_CHUNK_VECS ? left : SA_CHUNK_VECS;
    r.b_begin = sh.vecs_per_row - r0; // > 0; >= 256 when the chunk stays inside its row
    const uint32_t b_end = r.b_begin + sh.rotated_vecs;
    r.b_end = b_end < SA_CHUNK_VECS ? b_end : SA_CHUNK_VECS;
    if (r.b_begin > SA_CHUNK_VECS) r.b_begin = SA_CHUNK_VECS;
    return r;
}

// one chunk with ordinary loads and stores (array ends, short rows, after a wait ran out)
template <bool BF16>
__device__ __forceinline__ void rope_chunk_plain(const SaSched& s, const SaRopeShape& sh, uint4* x, const float4* table,
                                                 uint64_t first_vec, uint32_t lane) {
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

template <bool BF16>
__global__ void __launch_bounds__(kWarps * 32, 1)
sa_rope_bulk_kernel(const __grid_constant__ SaSched s, const __grid_constant__ SaSideTable sides,
                    uint4* __restrict__ x, const float4* __restrict__ table,
                    const __grid_constant__ SaRopeShape sh, uint32_t* wait_errors) {
    constexpr uint32_t S = kStages;
    extern __shared__ __align__(128) unsigned char stage_mem[]; // [warps][stages][4 KiB]
    __shared__ __align__(8) unsigned long long bars[kWarps * S];
    __shared__ StageInfo infos[kWarps * S];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t my_stage0 = sa_smem_addr(stage_mem) + warp * S * SA_BULK_CHUNK_BYTES;
    const uint32_t my_bar0 = sa_smem_addr(&bars[warp * S]);
    StageInfo* const my_infos = &infos[warp * S];
    if (lane == 0) {
        for (uint32_t i = 0; i < S; ++i) sa_mbar_init(my_bar0 + 8u * i, 1);
        sa_mbar_fence_init();
    }
    __syncwarp();

    // All lanes run the same sequence of issues and retirements (wait results are agreed on by
    // vote), so every lane keeps the same ring state and no broadcast is needed.
    SaStageRing ring;
    sa_ring_reset(ring);
    const bool staged_shape = sh.vecs_per_row >= SA_CHUNK_VECS;
    // cos/sin position of this lane's vectors inside a head: fixed when a head is a power-of-two
    // number of vectors that divides the 32-lane stride (rows are whole heads, so it survives a row change)
    const bool pos_fixed = sh.head_shift >= 0 && sh.vecs_per_head <= 32u;
    // In that case the cos/sin entries of a chunk (its row's token and the next one) are fetched when the chunk's
    // load is issued and wait in registers, in the order of the ring, until the chunk is rotated: their latency
    // is hidden behind the data's.  Slot 0 belongs to the oldest chunk in flight.
    constexpr int kQueue = (int)kLoadsInFlight + 1;
    RopeTab<BF16> tabs[kQueue][2] = {};

    // wait for the oldest chunk in flight, rotate it in shared memory, send it back
    auto retire = [&]() {
        const uint32_t st = sa_ring_oldest(ring, S);
        const bool arrived = __all_sync(0xffffffffu, sa_mbar_wait(my_bar0 + 8u * st, sa_ring_oldest_parity(ring, S)));
        if (arrived) {
            const StageInfo info = my_infos[st];
            const Runs runs = chunk_runs(sh, info.r0);
            const uint32_t stage = my_stage0 + st * SA_BULK_CHUNK_BYTES;
            const uint32_t tok1 = info.tok0 + 1u == sh.T ? 0u : info.tok0 + 1u;
            // ordinary shared-memory accesses, 16 bytes per lane: the eight loads first, then arithmetic and stores
            uint4* const sp = reinterpret_cast<uint4*>(stage_mem + (size_t)(warp * S + st) * SA_BULK_CHUNK_BYTES) + lane;
            uint4 v[SA_VEC_PER_LANE];
#pragma unroll
            for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                const uint32_t i = lane + 32u * k;
                if (i < runs.a_end || (i >= runs.b_begin && i < runs.b_end)) v[k] = sp[32 * k];
            }
            if (pos_fixed) {
                const RopeTab<BF16> ta = tabs[0][0], tb = tabs[0][1];
                if (runs.b_begin >= runs.b_end) { // the usual case: the chunk lies inside one row
#pragma unroll
                    for (int k = 0; k < SA_VEC_PER_LANE; ++k)
                        if (lane + 32u * k < runs.a_end) sp[32 * k] = rope_apply<BF16>(v[k], ta);
                } else {
#pragma unroll
                    for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                        const uint32_t i = lane + 32u * k;
                        if (i < runs.a_end) sp[32 * k] = rope_apply<BF16>(v[k], ta);
                        else if (i >= runs.b_begin && i < runs.b_end) sp[32 * k] = rope_apply<BF16>(v[k], tb);
                    }
                }
            } else {
                uint32_t have = 0xffffffffu;
                RopeTab<BF16> tab;
#pragma unroll
                for (int k = 0; k < SA_VEC_PER_LANE; ++k) {
                    const uint32_t i = lane + 32u * k;
                    const bool in_a = i < runs.a_end;
                    const bool in_b = i >= runs.b_begin && i < runs.b_end;
                    if (in_a || in_b) {
                        const uint32_t tok = in_a ? info.tok0 : tok1;
                        const uint32_t r = in_a ? info.r0 + i : i - runs.b_begin;
                        const uint32_t idx = tok * sh.tab_vecs_per_token + (r % sh.vecs_per_head) * sh.tab_vecs_per_vec;
                        if (idx != have) {
                            tab = rope_load_tab<BF16>(table + idx, sh.inverse != 0);
                            have = idx;
                        }
                        sp[32 * k] = rope_apply<BF16>(v[k], tab);
                    }
                }
            }
            sa_fence_async_shared(); // this lane's shared-memory writes, before the bulk store reads them
            __syncwarp();
            if (lane == 0) {
                uint4* const g = x + (info.first_vec - s.lead);
                if (runs.a_end) sa_bulk_store(g, stage, runs.a_end * 16u);
                if (runs.b_begin < runs.b_end) sa_bulk_store(g + runs.b_begin, stage + runs.b_begin * 16u, (runs.b_end - runs.b_begin) * 16u);
                sa_bulk_commit();
            }
        } else if (lane == 0) {
            atomicAdd_system(wait_errors, 1u);
        }
        sa_ring_retire(ring, S, arrived);
#pragma unroll
        for (int i = 0; i + 1 < kQueue; ++i) {
            tabs[i][0] = tabs[i + 1][0];
            tabs[i][1] = tabs[i + 1][1];
        }
    };

    sa_for_each_chunk(s, sides, [&](uint64_t first_vec) {
        const bool whole = first_vec >= s.lead && first_vec + SA_CHUNK_VECS <= s.end;
        if (whole && staged_shape && sa_ring_may_issue(ring)) {
            const uint64_t e0 = first_vec - s.lead;
            const uint64_t row0 = e0 / sh.vecs_per_row;
            const uint32_t r0 = (uint32_t)(e0 - row0 * sh.vecs_per_row);
            const Runs runs = chunk_runs(sh, r0);
            const uint32_t vecs = runs.a_end + (runs.b_end - runs.b_begin);
            if (vecs == 0u) return; // nothing but V heads in this chunk
            const uint32_t slot = sa_ring_in_flight(ring); // chunks ahead of this one in the ring
            const uint32_t tok0 = (uint32_t)(row0 % sh.T);
            if (pos_fixed) {
                const uint32_t pos = ((r0 + lane) & (sh.vecs_per_head - 1u)) * sh.tab_vecs_per_vec;
                const uint32_t tok1 = tok0 + 1u == sh.T ? 0u : tok0 + 1u;
                const RopeTab<BF16> ta = rope_load_tab<BF16>(table + tok0 * sh.tab_vecs_per_token + pos, sh.inverse != 0);
                const RopeTab<BF16> tb = rope_load_tab<BF16>(table + tok1 * sh.tab_vecs_per_token + pos, sh.inverse != 0);
#pragma unroll
                for (int i = 0; i < kQueue; ++i)
                    if ((uint32_t)i == slot) {
                        tabs[i][0] = ta;
                        tabs[i][1] = tb;
                    }
            }
            const uint32_t st = sa_ring_issue(ring, S);
            if (lane == 0) {
                // the store that last used this stage (S chunks ago) must have read it
                sa_bulk_wait_read<kPendingStoreGroups>();
                const uint32_t stage = my_stage0 + st * SA_BULK_CHUNK_BYTES, bar = my_bar0 + 8u * st;
                sa_mbar_expect(bar, vecs * 16u);
                if (runs.a_end) sa_bulk_load(stage, x + e0, runs.a_end * 16u, bar);
                if (runs.b_begin < runs.b_end) sa_bulk_load(stage + runs.b_begin * 16u, x + e0 + runs.b_begin, (runs.b_end - runs.b_begin) * 16u, bar);
                StageInfo info;
                info.first_vec = first_vec;
                info.r0 = r0;
                info.tok0 = tok0;
                my_infos[st] = info;
            }
            __syncwarp(); // the stage's info is visible to the lanes that will rotate it
            while (sa_ring_in_flight(ring) > kLoadsInFlight) retire(); // older chunks are rotated while newer ones come in
        } else {
            rope_chunk_plain<BF16>(s, sh, x, table, first_vec, lane);
        }
    });
    while (sa_ring_in_flight(ring) > 0) retire();
    if (lane == 0) sa_bulk_wait_read<0>(); // shared memory must stay valid until the last store has read it
    // chunks whose data never arrived (only after a wait ran out): nothing of them was stored, so they are still
    // unrotated in global memory and are done again with ordinary loads and stores
    if (ring.lost) {
        __syncwarp();
        for (uint32_t st = 0; st < S; ++st)
            if ((ring.lost >> st) & 1u) rope_chunk_plain<BF16>(s, sh, x, table, my_infos[st].first_vec, lane);
    }
}

template <bool BF16>
cudaError_t launch(const SaSched& s, const SaSideTable& sides, int grid, void* x, const float* table, const SaRopeShape& sh,
                   uint32_t* wait_errors, cudaStream_t stream) {
    constexpr int smem = kWarps * kStages * (int)SA_BULK_CHUNK_BYTES;
    // once per device: the attribute belongs to the current device's copy of the function
    static std::atomic<bool> opted_in[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !opted_in[dev].load(std::memory_order_acquire)) {
        cudaError_t attr = cudaFuncSetAttribute(sa_rope_bulk_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (attr != cudaSuccess) return attr;
        if (dev >= 0 && dev < 64) opted_in[dev].store(true, std::memory_order_release);
    }
    SaLaunch l(s, grid, kWarps * 32, smem, stream);
    return cudaLaunchKernelEx(&l.cfg, sa_rope_bulk_kernel<BF16>, s, sides, (uint4*)x, (const float4*)table, sh, wait_errors);
}

} // namespace

cudaError_t sa_launch_rope_bulk(const SaSched& s, const SaSideTable& sides, int grid, void* x, const float* table,
                                const SaRopeShape& sh, bool bf16, uint32_t* wait_errors, cudaStream_t stream) {
    return bf16 ? launch<true>(s, sides, grid, x, table, sh, wait_errors, stream)
                : launch<false>(s, sides, grid, x, table, sh, wait_errors, stream);
}

int sa_rope_bulk_warps() { return kWarps; }
