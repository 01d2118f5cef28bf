// extern "C" surface of sideaware.so (declarations and reference citations: include/sideaware.h).
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <random>

#include "../../include/sideaware.h"
#include "sa_context.hpp"
#ifndef SIDEAWARE_ALLOC_ONLY
#include "sa_jit.hpp"
#include "sa_kernels.hpp"
#endif

#define SA_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t kChunkBytes = 4096;

size_t threshold_now() {
    std::lock_guard<std::mutex> lock(sa_config().mu);
    return sa_config().threshold;
}

SaAllocConfig alloc_config_now() {
    std::lock_guard<std::mutex> lock(sa_config().mu);
    return sa_config().alloc;
}

void* malloc_large(SaDevice* dev, size_t size, cudaStream_t stream) {
    SaScopedDevice guard(dev->id);
    uint64_t p = dev->alloc->malloc(size, (void*)stream, alloc_config_now());
    if (!p) sa_set_error("device %d: out of memory allocating %zu bytes side-aware", dev->id, size);
    return (void*)p;
}

// Unknown pointers are handed to the runtime's pool, as the reference does (sideaware.cu:1258-1261).
cudaError_t free_large(SaDevice* dev, void* ptr, cudaStream_t stream) {
    if (!ptr) return cudaSuccess;
    if (dev->alloc->free((uint64_t)ptr, (void*)stream)) {
        // free-time upkeep (sideaware_prealloc_config): nothing but a flag test unless the last request ran the
        // free memory at hand down below extra_required
        const SaAllocConfig cfg = alloc_config_now();
        if (cfg.extra_alloc > 0 && cfg.extra_required > 0) {
            SaScopedDevice guard(dev->id);
            dev->alloc->top_up((void*)stream, cfg);
        }
        return cudaSuccess;
    }
    SaScopedDevice guard(dev->id);
    return cudaFreeAsync(ptr, stream);
}

#ifndef SIDEAWARE_ALLOC_ONLY
bool check_launch_args(const char* what, size_t num_bytes, const void* const* ptrs, int n) {
    if (num_bytes % 16 != 0) {
        sa_set_error("%s: num_bytes (%zu) must be a multiple of 16", what, num_bytes);
        return false;
    }
    for (int i = 0; i < n; ++i)
        if (((uintptr_t)ptrs[i] & 15u) != 0) {
            sa_set_error("%s: pointer %p is not 16-byte aligned", what, ptrs[i]);
            return false;
        }
    return true;
}
#endif

} // namespace

// ---------------------------------------------------------------------------
// allocation
// ---------------------------------------------------------------------------
SA_API sideaware_status_t sideaware_malloc_async(void** dev_ptr, size_t size, sideaware_stream_t stream) {
    if (!dev_ptr) return cudaErrorInvalidValue;
    *dev_ptr = nullptr;
    SaDevice* dev = sa_device(-1);
    if (!dev) return cudaErrorInitializationError;
    *dev_ptr = malloc_large(dev, size, (cudaStream_t)stream);
    return *dev_ptr ? cudaSuccess : cudaErrorMemoryAllocation;
}

SA_API sideaware_status_t sideaware_free_async(void* ptr, sideaware_stream_t stream) {
    SaDevice* dev = sa_device(-1);
    if (!dev) return cudaErrorInitializationError;
    return free_large(dev, ptr, (cudaStream_t)stream);
}

SA_API sideaware_status_t sideaware_malloc(void** dev_ptr, size_t size) {
    if (!dev_ptr) return cudaErrorInvalidValue;
    *dev_ptr = nullptr;
    SaDevice* dev = sa_device(-1);
    if (!dev) return cudaErrorInitializationError;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        sa_set_error("sideaware_malloc: earlier asynchronous error: %s", cudaGetErrorString(e));
        return e;
    }
    *dev_ptr = malloc_large(dev, size, nullptr);
    return *dev_ptr ? cudaSuccess : cudaErrorMemoryAllocation;
}

SA_API sideaware_status_t sideaware_free(void* ptr) {
    SaDevice* dev = sa_device(-1);
    if (!dev) return cudaErrorInitializationError;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        sa_set_error("sideaware_free: earlier asynchronous error: %s", cudaGetErrorString(e));
        return e;
    }
    return free_large(dev, ptr, nullptr);
}

SA_API sideaware_status_t sideaware_prealloc(size_t bytes, int device) {
    if (bytes == 0) return cudaSuccess;
    SaDevice* dev = sa_device(device);
    if (!dev) return cudaErrorInitializationError;
    SaScopedDevice guard(dev->id);
    if (!dev->alloc->prealloc(bytes, alloc_config_now())) {
        sa_set_error("device %d: out of memory mapping %zu bytes ahead of need", dev->id, bytes);
        return cudaErrorMemoryAllocation;
    }
    return cudaSuccess;
}

SA_API size_t sideaware_release_unused(void) {
    size_t total = 0;
    for (SaDevice* dev : sa_initialised_devices()) {
        SaScopedDevice guard(dev->id);
        total += dev->alloc->release_unused();
    }
    return total;
}

SA_API void* sideaware_malloc_auto(size_t size, int device, sideaware_stream_t stream) {
    SaDevice* dev = sa_device(device);
    if (!dev) return nullptr;
    if (size >= threshold_now()) return malloc_large(dev, size, (cudaStream_t)stream);
    SaScopedDevice guard(dev->id);
    void* p = nullptr;
    cudaError_t e = cudaMallocAsync(&p, size, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        dev->alloc->trim(0, 0); // cached side-aware blocks may be holding the memory (sideaware.cu:1334)
        e = cudaMallocAsync(&p, size, (cudaStream_t)stream);
        if (e != cudaSuccess) {
            cudaGetLastError();
            dev->alloc->release_unused();
            e = cudaMallocAsync(&p, size, (cudaStream_t)stream);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            sa_set_error("device %d: cudaMallocAsync(%zu): %s", dev->id, size, cudaGetErrorString(e));
            return nullptr;
        }
    }
    dev->small_allocs.fetch_add(1);
    return p;
}

SA_API void sideaware_free_auto(void* ptr, size_t size, int device, sideaware_stream_t stream) {
    (void)size;
    if (!ptr) return;
    SaDevice* dev = sa_device(device);
    if (!dev) return;
    cudaError_t e = free_large(dev, ptr, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        sa_set_error("device %d: freeing %p: %s", dev->id, ptr, cudaGetErrorString(e));
    }
}

#ifndef SIDEAWARE_ALLOC_ONLY // the allocator-only build has no kernels and no functor compiler
// ---------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------
SA_API void sideaware_elementwise(int kernel_id, size_t num_bytes,
                                  void* out0, void* out1, void* out2, void* out3,
                                  const void* in0, const void* in1, const void* in2, const void* in3,
                                  void* sideband_memory, int sideband_value,
                                  int parallel_groups, int forced_per_side,
                                  int device, sideaware_stream_t stream) {
    if (num_bytes == 0 || (out0 == nullptr && in0 == nullptr)) return;
    SaDevice* dev = sa_device(device);
    if (!dev) return;
    const void* ptrs[8] = {out0, out1, out2, out3, in0, in1, in2, in3};
    if (!check_launch_args("sideaware_elementwise", num_bytes, ptrs, 8)) return;
    if (kernel_id < 0 || kernel_id >= sa_jit_num_kernels()) {
        sa_set_error("sideaware_elementwise: unknown kernel id %d", kernel_id);
        return;
    }
    if (forced_per_side < 0 || forced_per_side > dev->topo.min_per_side) forced_per_side = 0;
    SaScopedDevice guard(dev->id);
    const uint64_t num_vecs = num_bytes / 16;
    SaSched s;
    int grid = 0, threads = 0;
    cudaError_t e;
    if (kernel_id == 0) {
        if (!out0 || !in0) {
            sa_set_error("sideaware_memcpy: null pointer");
            return;
        }
        if (sa_config().memcpy_engine.load() == 1) {
            if (!sa_prepare_launch(dev, stream, (uint64_t)in0, num_vecs, 0, forced_per_side, false, &s, &grid, &threads, sa_memcpy_bulk_warps())) return;
            sa_report_wait_timeouts(dev, "sideaware_memcpy");
            e = sa_launch_memcpy_bulk(s, dev->side_table, grid, out0, in0, sa_probe_wait_error_word(dev->probe), (cudaStream_t)stream);
            if (e != cudaSuccess) sa_set_error("sideaware_memcpy (bulk engine) launch: %s", cudaGetErrorString(e));
            return;
        }
        if (!sa_prepare_launch(dev, stream, (uint64_t)in0, num_vecs, parallel_groups, forced_per_side, false, &s, &grid, &threads)) return;
        e = sa_launch_memcpy(s, dev->side_table, grid, threads, out0, in0, (cudaStream_t)stream);
        if (e != cudaSuccess) sa_set_error("sideaware_memcpy launch: %s", cudaGetErrorString(e));
        return;
    }
    int groups = parallel_groups > 0 ? parallel_groups : sa_jit_default_groups(kernel_id);
    bool misaligned = ((uintptr_t)in0 % kSaPageBytes) || ((uintptr_t)out0 % kSaPageBytes);
    bool wide = misaligned || num_bytes >= (2ull << 30); // same rule as sideaware.cu:1386-1388
    std::string why;
    // a header may bound its block size (LAUNCH_BOUNDS) below the four 256-thread groups of the default launch
    const int max_threads = sa_jit_max_threads(dev, kernel_id, wide, &why);
    if (max_threads < 256) {
        sa_set_error("sideaware_elementwise(kernel %d): %s", kernel_id, why.empty() ? "the functor cannot run 256 threads per block" : why.c_str());
        return;
    }
    if (groups > max_threads / 256) groups = max_threads / 256;
    // geometry is redone inside the kernel for whichever array it moves as 16-byte vectors;
    // the host only needs the size to pick grid and ticket length
    const void* track = in0 ? in0 : out0;
    if (!sa_prepare_launch(dev, stream, (uint64_t)track, num_vecs, groups, forced_per_side, false, &s, &grid, &threads)) return;
    void* outs[4] = {out0, out1, out2, out3};
    const void* ins[4] = {in0, in1, in2, in3};
    e = sa_jit_launch(dev, kernel_id, wide, s, grid, threads, num_vecs, outs, ins, sideband_memory, sideband_value,
                      (cudaStream_t)stream, &why);
    if (e != cudaSuccess) sa_set_error("sideaware_elementwise(kernel %d): %s", kernel_id, why.c_str());
}

SA_API void sideaware_one_to_one(int kernel_id, size_t num_bytes, void* out0, const void* in0,
                                 int device, sideaware_stream_t stream) {
    sideaware_elementwise(kernel_id, num_bytes, out0, nullptr, nullptr, nullptr, in0, nullptr, nullptr, nullptr,
                          nullptr, 0, 0, 0, device, stream);
}

SA_API void sideaware_memcpy(void* out, const void* in, size_t num_bytes, int device, sideaware_stream_t stream) {
    sideaware_elementwise(0, num_bytes, out, nullptr, nullptr, nullptr, in, nullptr, nullptr, nullptr,
                          nullptr, 0, 0, 0, device, stream);
}

static sideaware_status_t rope_launch(void* qkv, const float* freqs_cis, int B, int T, int Nq, int Nkv, int HS, int dtype,
                                      int device, sideaware_stream_t stream, bool inverse);

SA_API sideaware_status_t sideaware_rope_forward(void* qkv, const float* freqs_cis, int B, int T, int Nq, int Nkv,
                                                 int HS, int dtype, int device, sideaware_stream_t stream) {
    return rope_launch(qkv, freqs_cis, B, T, Nq, Nkv, HS, dtype, device, stream, false);
}

SA_API sideaware_status_t sideaware_rope_backward(void* dqkv, const float* freqs_cis, int B, int T, int Nq, int Nkv,
                                                  int HS, int dtype, int device, sideaware_stream_t stream) {
    return rope_launch(dqkv, freqs_cis, B, T, Nq, Nkv, HS, dtype, device, stream, true);
}

static sideaware_status_t rope_launch(void* qkv, const float* freqs_cis, int B, int T, int Nq, int Nkv, int HS, int dtype,
                                      int device, sideaware_stream_t stream, bool inverse) {
    if (B <= 0 || T <= 0 || Nq < 0 || Nkv < 0 || Nq + Nkv <= 0 || HS <= 0 || (dtype != 0 && dtype != 1) || !qkv || !freqs_cis) {
        sa_set_error("sideaware_rope_forward: invalid argument");
        return cudaErrorInvalidValue;
    }
    const int esize = dtype == 1 ? 2 : 4;
    if ((HS * esize) % 16 != 0 || HS % 4 != 0) {
        sa_set_error("sideaware_rope_forward: head size %d with %d-byte elements is not a whole number of 16-byte vectors", HS, esize);
        return cudaErrorInvalidValue;
    }
    const void* ptrs[2] = {qkv, freqs_cis};
    if (!check_launch_args("sideaware_rope_forward", 16, ptrs, 2)) return cudaErrorInvalidValue;
    SaDevice* dev = sa_device(device);
    if (!dev) return cudaErrorInitializationError;
    SaScopedDevice guard(dev->id);
    SaRopeShape sh;
    sh.vecs_per_head = (uint32_t)(HS * esize / 16);
    sh.vecs_per_row = (uint32_t)(Nq + 2 * Nkv) * sh.vecs_per_head;
    sh.rotated_vecs = (uint32_t)(Nq + Nkv) * sh.vecs_per_head;
    sh.T = (uint32_t)T;
    sh.tab_vecs_per_token = (uint32_t)HS / 4;
    sh.tab_vecs_per_vec = dtype == 1 ? 2 : 1;
    sh.head_shift = -1;
    sh.inverse = inverse ? 1 : 0;
    for (int b = 0; b < 31; ++b)
        if ((1u << b) == sh.vecs_per_head) sh.head_shift = b;
    const uint64_t num_vecs = (uint64_t)B * T * sh.vecs_per_row;
    SaSched s;
    int grid = 0, threads = 0;
    cudaError_t e;
    if (sa_config().rope_engine.load() == 1) {
        if (!sa_prepare_launch(dev, stream, (uint64_t)qkv, num_vecs, 0, 0, false, &s, &grid, &threads, sa_rope_bulk_warps())) return cudaErrorMemoryAllocation;
        sa_report_wait_timeouts(dev, "sideaware_rope_forward");
        e = sa_launch_rope_bulk(s, dev->side_table, grid, qkv, freqs_cis, sh, dtype == 1, sa_probe_wait_error_word(dev->probe), (cudaStream_t)stream);
    } else {
        // 768 threads per block: the rotation needs ~70 registers, measured faster than 1024 threads with spills
        if (!sa_prepare_launch(dev, stream, (uint64_t)qkv, num_vecs, 3, 0, false, &s, &grid, &threads)) return cudaErrorMemoryAllocation;
        e = sa_launch_rope(s, dev->side_table, grid, threads, qkv, freqs_cis, sh, dtype == 1, (cudaStream_t)stream);
    }
    if (e != cudaSuccess) sa_set_error("sideaware_rope_forward launch: %s", cudaGetErrorString(e));
    return e;
}

// Frequency of pair i: theta^(-2i/dim) in fp32, then the llama-3 context-extension rule
// (wavelengths above the original 8192-token context slowed 8x, those below a quarter of it
// kept, a linear blend in between).  Same fp32/fp64 mix, operation by operation, as
// precompute_freqs_cis (example_llmc_rope.cu:24-43), so the values are the reference's bit for bit.
static float rope_pair_frequency(int i, int dim, float theta, bool use_scaled) {
    float freq = 1.0f / powf(theta, (float)(2 * i) / dim);
    if (!use_scaled) return freq;
    const float slow_down = 8.0f, long_wave = 8192.0f, short_wave = 8192.0f / 4.0f;
    const float wavelen = (float)((double)2.0f * 3.14159265358979323846 / (double)freq);
    if (wavelen < short_wave) return freq;
    if (wavelen > long_wave) return freq / slow_down;
    const float blend = (8192.0f / wavelen - 1.0f) / 3.0f;
    const float kept = blend * freq;
    return (1.0f - blend) * freq / slow_down + kept;
}

SA_API sideaware_status_t sideaware_rope_precompute_freqs(float* freqs_cis, int dim, int end, float theta,
                                                          int use_scaled, int device, sideaware_stream_t stream) {
    if (!freqs_cis || dim < 2 || dim > 1024 || (dim & 1) || end <= 0 || !(theta > 0.0f)) {
        sa_set_error("sideaware_rope_precompute_freqs: invalid argument (dim %d, end %d, theta %g)", dim, end, (double)theta);
        return cudaErrorInvalidValue;
    }
    const void* ptrs[1] = {freqs_cis};
    if (!check_launch_args("sideaware_rope_precompute_freqs", 16, ptrs, 1)) return cudaErrorInvalidValue;
    SaDevice* dev = sa_device(device);
    if (!dev) return cudaErrorInitializationError;
    SaScopedDevice guard(dev->id);
    float freqs[512];
    for (int i = 0; i < dim / 2; ++i) freqs[i] = rope_pair_frequency(i, dim, theta, use_scaled != 0);
    cudaError_t e = sa_launch_rope_table(freqs_cis, freqs, dim / 2, end, (cudaStream_t)stream);
    if (e != cudaSuccess) sa_set_error("sideaware_rope_precompute_freqs launch: %s", cudaGetErrorString(e));
    return e;
}

SA_API sideaware_status_t sideaware_silu_mul_bf16(void* out, const void* a, const void* b, float scale, size_t n,
                                                  int device, sideaware_stream_t stream) {
    if (n == 0) return cudaSuccess;
    if (!out || !a || !b || n % 8 != 0) {
        sa_set_error("sideaware_silu_mul_bf16: null pointer or element count %zu not a multiple of 8", n);
        return cudaErrorInvalidValue;
    }
    const void* ptrs[3] = {out, a, b};
    if (!check_launch_args("sideaware_silu_mul_bf16", 16, ptrs, 3)) return cudaErrorInvalidValue;
    SaDevice* dev = sa_device(device);
    if (!dev) return cudaErrorInitializationError;
    SaScopedDevice guard(dev->id);
    SaSched s;
    int grid = 0, threads = 0;
    if (!sa_prepare_launch(dev, stream, (uint64_t)a, n / 8, 0, 0, false, &s, &grid, &threads)) return cudaErrorMemoryAllocation;
    cudaError_t e = sa_launch_silu_mul(s, dev->side_table, grid, threads, out, a, b, scale, (cudaStream_t)stream);
    if (e != cudaSuccess) sa_set_error("sideaware_silu_mul_bf16 launch: %s", cudaGetErrorString(e));
    return e;
}

// ---------------------------------------------------------------------------
// functors
// ---------------------------------------------------------------------------
SA_API int sideaware_create_kernel_advanced(const char* header, bool precompile, int default_num_groups) {
    if (!header || !*header) return 0;
    int id = sa_jit_register(header, default_num_groups);
    if (precompile) {
        SaDevice* dev = sa_device(-1);
        std::string why;
        if (!dev || !sa_jit_precompile(dev, id, &why)) {
            sa_set_error("sideaware_create_kernel: %s", why.c_str());
            return -1;
        }
    }
    return id;
}

SA_API int sideaware_compile_check(const char* header, int wide, char* log_out, size_t log_capacity) {
    std::string why;
    bool ok = sa_jit_compile_only(header, wide != 0, &why);
    const std::string warn = sa_jit_contract_warnings(header); // reported with the log, whether or not the header compiles
    if (!warn.empty()) why = why.empty() ? warn : warn + "\n" + why;
    if (log_out && log_capacity) {
        std::strncpy(log_out, why.c_str(), log_capacity - 1);
        log_out[log_capacity - 1] = 0;
    }
    return ok ? 0 : 1;
}

SA_API int sideaware_create_kernel(const char* header) { return sideaware_create_kernel_advanced(header, false, 4); }

#endif // SIDEAWARE_ALLOC_ONLY

// ---------------------------------------------------------------------------
// configuration
// ---------------------------------------------------------------------------
SA_API void sideaware_compression(bool enable) {
    std::lock_guard<std::mutex> lock(sa_config().mu);
    sa_config().alloc.compression = enable;
}
SA_API void sideaware_alloc_threshold(size_t threshold) {
    std::lock_guard<std::mutex> lock(sa_config().mu);
    sa_config().threshold = threshold;
}
SA_API void sideaware_prealloc_config(int extra_required, int extra_alloc) {
    std::lock_guard<std::mutex> lock(sa_config().mu);
    sa_config().alloc.extra_required = extra_required;
    sa_config().alloc.extra_alloc = extra_alloc;
}
SA_API void sideaware_free_mapped_thresholds(size_t start_threshold, size_t end_threshold) {
    std::lock_guard<std::mutex> lock(sa_config().mu);
    sa_config().alloc.trim_start = start_threshold;
    sa_config().alloc.trim_end = end_threshold;
    sa_config().alloc.trim_scaled = false; // the caller's numbers, whatever the device's size
}
#ifndef SIDEAWARE_ALLOC_ONLY
SA_API void sideaware_write_sass(const char* filename) {
    std::lock_guard<std::mutex> lock(sa_config().mu);
    sa_config().log_file = filename ? filename : "";
}
#endif
#ifndef SIDEAWARE_ALLOC_ONLY
SA_API void sideaware_set_placement(int mode) {
    if (mode < 0 || mode > 2) mode = 0;
    sa_config().placement.store(mode);
}
SA_API int sideaware_get_placement(void) { return sa_config().placement.load(); }
SA_API void sideaware_set_memcpy_engine(int engine) { sa_config().memcpy_engine.store(engine == 0 ? 0 : 1); }
SA_API int sideaware_get_memcpy_engine(void) { return sa_config().memcpy_engine.load(); }
SA_API void sideaware_set_rope_engine(int engine) { sa_config().rope_engine.store(engine == 0 ? 0 : 1); }
SA_API int sideaware_get_rope_engine(void) { return sa_config().rope_engine.load(); }
#endif

// ---------------------------------------------------------------------------
// queries
// ---------------------------------------------------------------------------
SA_API void sideaware_fill_side_index(unsigned char* gpu_array) {
    SaDevice* dev = sa_device(-1);
    if (!dev || !gpu_array) return;
    cudaError_t e = cudaMemcpy(gpu_array, sa_probe_gpu_side_index(dev->probe), dev->topo.num_sms, cudaMemcpyDeviceToDevice);
    if (e != cudaSuccess) sa_set_error("sideaware_fill_side_index: %s", cudaGetErrorString(e));
}
SA_API const char* sideaware_gpu_side_index(void) {
    SaDevice* dev = sa_device(-1);
    return dev ? (const char*)sa_probe_gpu_side_index(dev->probe) : nullptr;
}
SA_API const char* sideaware_cpu_side_index(void) {
    SaDevice* dev = sa_device(-1);
    return dev ? (const char*)dev->topo.side_index : nullptr;
}
SA_API const int* sideaware_sm_side_summary(void) {
    static const int none[5] = {0, 0, 0, 0, 0};
    SaDevice* dev = sa_device(-1);
    return dev ? dev->summary : none;
}
SA_API int sideaware_num_sms(void) { SaDevice* d = sa_device(-1); return d ? d->summary[0] : 0; }
SA_API int sideaware_num_sm_side0(void) { SaDevice* d = sa_device(-1); return d ? d->summary[1] : 0; }
SA_API int sideaware_num_sm_side1(void) { SaDevice* d = sa_device(-1); return d ? d->summary[2] : 0; }
SA_API int sideaware_min_sm_per_side(void) { SaDevice* d = sa_device(-1); return d ? d->summary[3] : 0; }
SA_API int sideaware_hash_mask(void) { SaDevice* d = sa_device(-1); return d ? d->summary[4] : 0; }

SA_API const char* sideaware_last_error(void) { return sa_last_error_text(); }
SA_API unsigned long long sideaware_error_count(void) { return sa_error_total(); }

SA_API size_t sideaware_chunk_sides(const void* ptr, size_t num_bytes, unsigned char* host_out) {
    SaDevice* dev = sa_device(-1);
    if (!dev || !host_out) return 0;
    const uint64_t first = (uint64_t)ptr & ~(uint64_t)(kChunkBytes - 1);
    const uint64_t last = (uint64_t)ptr + num_bytes;
    size_t n = 0;
    const uint32_t hash = dev->topo.hash | (1u << kSaSideBit);
    for (uint64_t a = first; a < last; a += kChunkBytes) host_out[n++] = (unsigned char)sa_parity32((uint32_t)a & hash);
    return n;
}

SA_API int sideaware_verify_chunk_sides(const void* ptr, size_t num_bytes, int samples, unsigned seed) {
    SaDevice* dev = sa_device(-1);
    if (!dev || !ptr || num_bytes < kChunkBytes || samples <= 0) return -1;
    SaScopedDevice guard(dev->id);
    const uint64_t first = ((uint64_t)ptr + kChunkBytes - 1) & ~(uint64_t)(kChunkBytes - 1);
    const uint64_t chunks = ((uint64_t)ptr + num_bytes - first) / kChunkBytes;
    if (chunks == 0) return -1;
    std::mt19937_64 rng(seed);
    std::vector<uint64_t> addrs(samples);
    for (int i = 0; i < samples; ++i) addrs[i] = first + (rng() % chunks) * kChunkBytes;
    std::vector<uint8_t> measured(samples);
    int ambiguous = 0;
    cudaError_t e = sa_probe_sides(dev->probe, dev->topo, addrs.data(), samples, measured.data(), dev->probe_stream, &ambiguous);
    if (e != cudaSuccess) {
        sa_set_error("sideaware_verify_chunk_sides: %s", cudaGetErrorString(e));
        return -1;
    }
    const uint32_t hash = dev->topo.hash | (1u << kSaSideBit);
    int mismatches = 0;
    for (int i = 0; i < samples; ++i) mismatches += measured[i] != sa_parity32((uint32_t)addrs[i] & hash);
    return mismatches;
}

SA_API void sideaware_get_stats(sideaware_stats_t* out) {
    if (!out) return;
    std::memset(out, 0, sizeof(*out));
    SaDevice* dev = sa_device(-1);
    if (!dev) return;
    SaAllocStats st = dev->alloc->stats();
    out->bytes_mapped_live = st.bytes_live;
    out->bytes_mapped_cached = st.bytes_cached;
    out->pages_pool_side0 = st.pages_pool[0];
    out->pages_pool_side1 = st.pages_pool[1];
    out->pages_created = st.pages_created;
    out->cross_side_pages = st.cross_side_pages;
    out->reuse_hits = st.reuse_hits;
    out->large_allocs = st.large_allocs;
    out->small_allocs = dev->small_allocs.load();
    out->trims = st.trims;
    out->handles_created = st.handles_created;
    out->handles_discarded = st.handles_discarded;
    out->extensions = st.extensions;
    out->hole_refills = st.hole_refills;
    out->headroom_pages = st.headroom_pages;
    out->top_ups = st.top_ups;
    out->jit_compiles = dev->jit_compiles.load();
    out->kernel_launches = dev->launches.load();
    out->probe_confidence_ppm = (unsigned long long)(dev->topo.confidence > 0 ? dev->topo.confidence * 1e6 : 0);
    out->hash_validation_errors = (unsigned long long)dev->topo.validation_errors;
    {
        SaScopedDevice guard(dev->id);
        out->kernel_wait_timeouts = sa_probe_wait_timeouts(dev->probe);
    }
}

SA_API void sideaware_driver_call_times(unsigned long long ns_out[8], unsigned long long calls_out[8]) {
    if (ns_out && calls_out) sa_backend_times(ns_out, calls_out);
}

SA_API const char* sideaware_topology_json(void) {
    SaDevice* dev = sa_device(-1);
    return dev ? dev->topo.json.c_str() : "{}";
}

#ifndef SIDEAWARE_ALLOC_ONLY
// ---------------------------------------------------------------------------
// memcpy without any device-memory allocation
// ---------------------------------------------------------------------------
SA_API sideaware_status_t sideaware_memcpy_noalloc(void* out, const void* in, size_t num_bytes, int device,
                                                   sideaware_stream_t stream) {
    if (num_bytes == 0) return cudaSuccess;
    if (!out || !in) {
        sa_set_error("sideaware_memcpy_noalloc: null pointer");
        return cudaErrorInvalidValue;
    }
    if (num_bytes > SIDEAWARE_NOALLOC_MAX_BYTES) {
        sa_set_error("sideaware_memcpy_noalloc: %zu bytes is more than this entry point accepts (%llu); split the copy",
                     num_bytes, (unsigned long long)SIDEAWARE_NOALLOC_MAX_BYTES);
        return cudaErrorInvalidValue;
    }
    const void* ptrs[2] = {out, in};
    if (!check_launch_args("sideaware_memcpy_noalloc", num_bytes, ptrs, 2)) return cudaErrorInvalidValue;
    if (device < 0 && cudaGetDevice(&device) != cudaSuccess) {
        sa_set_error("sideaware_memcpy_noalloc: no CUDA device");
        return cudaErrorNoDevice;
    }
    SaScopedDevice guard(device);
    int num_sms = 0;
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || num_sms <= 0) {
        sa_set_error("sideaware_memcpy_noalloc: cannot query device %d", device);
        return cudaErrorInvalidDevice;
    }
    // The SM side table exists only if some earlier call set this device up (that set-up
    // allocates, so it is not done here).  Without it the copy runs side-unaware.
    SaDevice* dev = sa_device_if_ready(device);
    SaSched s;
    std::memset(&s, 0, sizeof(s));
    const int warps = 32;
    sa_sched_geometry(s, (uint64_t)in, num_bytes / 16, (uint32_t)(num_sms * warps / 2));
    int grid = num_sms;
    sa_sched_grid(s, num_sms, warps, &grid);
    s.placement = SA_PLACE_UNAWARE;
    SaSideTable sides;
    std::memset(&sides, 0, sizeof(sides));
    if (dev && dev->full_hash) {
        s.hash = dev->full_hash;
        s.placement = (uint32_t)sa_config().placement.load();
        sides = dev->side_table;
    }
    cudaError_t e = sa_launch_memcpy_noalloc(s, sides, device, grid, warps * 32, out, in, (cudaStream_t)stream);
    if (e != cudaSuccess) sa_set_error("sideaware_memcpy_noalloc: %s", cudaGetErrorString(e));
    return e;
}
#endif // SIDEAWARE_ALLOC_ONLY
