// Launch interface of the ahead-of-time kernels (sa_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "sa_sched.cuh"

// Geometry of a packed [B, T, Nq + 2 Nkv, HS] tensor in 16-byte vectors.
struct SaRopeShape {
    uint32_t vecs_per_head;      // HS * elem_size / 16
    uint32_t vecs_per_row;       // (Nq + 2 Nkv) * vecs_per_head
    uint32_t rotated_vecs;       // (Nq + Nkv) * vecs_per_head: Q and K heads come first in a row
    uint32_t T;
    uint32_t tab_vecs_per_token; // float4 entries of the cos/sin table per token = HS / 4
    uint32_t tab_vecs_per_vec;   // float4 table entries consumed per data vector (bf16: 2, fp32: 1)
    int32_t head_shift;          // log2(vecs_per_head) if it is a power of two, else -1
    int32_t inverse;             // 1: rotate by the opposite angle (the backward pass)
};

cudaError_t sa_launch_memcpy(const SaSched& s, const SaSideTable& sides, int grid, int threads, void* dst, const void* src, cudaStream_t stream);
cudaError_t sa_launch_rope(const SaSched& s, const SaSideTable& sides, int grid, int threads, void* x, const float* table,
                           const SaRopeShape& sh, bool bf16, cudaStream_t stream);
cudaError_t sa_launch_silu_mul(const SaSched& s, const SaSideTable& sides, int grid, int threads, void* out, const void* a, const void* b,
                               float scale, cudaStream_t stream);
// cos/sin table [end][half][2] from `half` frequencies (host memory, half <= 512)
cudaError_t sa_launch_rope_table(float* table, const float* freqs, int half, int end, cudaStream_t stream);
// Same kernel as sa_launch_memcpy with its ticket counters in a static device array (no allocation).
cudaError_t sa_launch_memcpy_noalloc(SaSched s, const SaSideTable& sides, int device, int grid, int threads, void* dst, const void* src,
                                     cudaStream_t stream);
// memcpy through bulk asynchronous copies staged in shared memory (sa_memcpy_bulk.cu); the block
// size is fixed: sa_memcpy_bulk_warps() warps.  `wait_errors`: device-visible word that counts waits that ran out.
cudaError_t sa_launch_memcpy_bulk(const SaSched& s, const SaSideTable& sides, int grid, void* dst, const void* src,
                                  uint32_t* wait_errors, cudaStream_t stream);
int sa_memcpy_bulk_warps();
// RoPE staged through shared memory with bulk copies (sa_rope_bulk.cu); fixed block size of sa_rope_bulk_warps() warps.
cudaError_t sa_launch_rope_bulk(const SaSched& s, const SaSideTable& sides, int grid, void* x, const float* table,
                                const SaRopeShape& sh, bool bf16, uint32_t* wait_errors, cudaStream_t stream);
int sa_rope_bulk_warps();

// Launch configuration shared by the ahead-of-time kernels.  Unless SIDEAWARE_PDL=0 the launch carries the
// programmatic-stream-serialization attribute: when two of this library's kernels follow each other on a
// stream, the second one's launch and prologue overlap the first one's tail; it touches data only after the
// first has completed (griddepcontrol.wait in sa_for_each_chunk).  Measured: +3 % at 256 MiB, +1 % at 1 GiB.
// Launches whose SaSched says overlap == 0 go without the attribute (every 32nd launch of a stream: that
// bounds how many launches of a stream can be under way at once, see the ticket rings in sa_probe.cu).
bool sa_pdl_enabled(); // false when SIDEAWARE_PDL=0
struct SaLaunch {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    SaLaunch(const SaSched& s, int grid, int threads, size_t smem, cudaStream_t stream);
};
