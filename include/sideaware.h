/*
 * sideaware.h - C ABI of sideaware.so, the B200 (sm_100a) side-aware allocator
 * and elementwise-kernel library.
 *
 * Every entry point of the first section keeps the name, argument meaning and
 * error behaviour of the corresponding `extern "C"` function of the reference
 * project (ademeure/l2_torch_alloc, file sideaware.cu; the line each one
 * replaces is cited).  Streams are passed as opaque pointers (a cudaStream_t),
 * status codes are CUDA runtime error numbers (0 = success, 2 = out of memory).
 * No C++ or torch types cross this boundary.
 *
 * Thread safety: all entry points may be called from any host thread; state is
 * guarded per device.  Launchers enqueue on the given stream and return.
 */
#ifndef SIDEAWARE_H
#define SIDEAWARE_H

#include <stddef.h>
#include <stdint.h>
#ifndef __cplusplus
#include <stdbool.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef void* sideaware_stream_t; /* cudaStream_t */
typedef int sideaware_status_t;   /* cudaError_t value */

/* ---- allocation (replaces sideaware.cu:1280-1352) ------------------------- */
/* Side-aware block on the current device: 2 MiB granular, VA bit 21 of every
 * page equals the L2 side its physical page is homed on, same size => same
 * bit-21 phase.  Replaces sideaware_malloc_async, sideaware.cu:1280. */
sideaware_status_t sideaware_malloc_async(void** dev_ptr, size_t size, sideaware_stream_t stream);
/* Returns the block to the (still mapped) reuse cache.  sideaware.cu:1286. */
sideaware_status_t sideaware_free_async(void* ptr, sideaware_stream_t stream);
/* Same, after a device synchronisation.  sideaware.cu:1292, :1301. */
sideaware_status_t sideaware_malloc(void** dev_ptr, size_t size);
sideaware_status_t sideaware_free(void* ptr);
/* Unmaps every cached block and releases all pooled physical pages on every
 * initialised device; returns the bytes released.  sideaware.cu:1307. */
size_t sideaware_release_unused(void);
/* PyTorch CUDAPluggableAllocator entry points.  size >= threshold (8 MiB by
 * default) is served side-aware, smaller sizes by cudaMallocAsync; NULL on
 * failure.  sideaware.cu:1320, :1343. */
void* sideaware_malloc_auto(size_t size, int device, sideaware_stream_t stream);
void sideaware_free_auto(void* ptr, size_t size, int device, sideaware_stream_t stream);

/* ---- kernels (replaces sideaware.cu:1358-1416) ---------------------------- */
/* Up to 4 outputs / 4 inputs, num_bytes = byte size of the widest array
 * (multiple of 16; pointers 16-byte aligned).  kernel_id 0 is memcpy.
 * parallel_groups: 256-thread groups per SM (0 = default), forced_per_side:
 * limit the SMs used per side (0 = all).  sideaware.cu:1358. */
void sideaware_elementwise(int kernel_id, size_t num_bytes,
                           void* out0, void* out1, void* out2, void* out3,
                           const void* in0, const void* in1, const void* in2, const void* in3,
                           void* sideband_memory, int sideband_value,
                           int parallel_groups, int forced_per_side,
                           int device, sideaware_stream_t stream);
/* sideaware.cu:1410 */
void sideaware_one_to_one(int kernel_id, size_t num_bytes, void* out0, const void* in0,
                          int device, sideaware_stream_t stream);
/* sideaware.cu:1414 */
void sideaware_memcpy(void* out, const void* in, size_t num_bytes, int device, sideaware_stream_t stream);

/* ---- user functors (replaces sideaware.cu:1421-1462) ---------------------- */
/* Registers a functor header (source text following the reference's header
 * contract, sideaware.cu:81-138) and returns its id; NULL/"" -> 0 (memcpy);
 * the same text always returns the same id.  Compiled with NVRTC for sm_100a
 * on first use per device, or immediately when precompile is set.
 * Returns -1 on a compile error (see sideaware_last_error). */
int sideaware_create_kernel_advanced(const char* header, bool precompile, int default_num_groups);
int sideaware_create_kernel(const char* header);

/* ---- configuration (replaces sideaware.cu:1467-1487) ---------------------- */
void sideaware_compression(bool enable);
void sideaware_alloc_threshold(size_t threshold);
/* In 2 MiB pages (sideaware.cu:1475-1478, top-up rule :1066-1080).  extra_alloc: whenever the mapped set has to
 * grow, that many pages more than asked for are mapped, as a free run behind the new block.  extra_required: if a
 * request leaves fewer free pages than this at hand (mapped-and-free or pooled), the next free call maps
 * extra_alloc more.  Defaults 1 and 10, the reference's.  0 for extra_alloc switches both off. */
void sideaware_prealloc_config(int extra_required, int extra_alloc);
/* Maps `bytes` of side-placed memory now, as one free run on `device` (< 0: the current one), so that later
 * requests up to that size find their pages mapped (about 2 us instead of about 80 us per 2 MiB page).
 * No counterpart in the reference, whose preallocation (sideaware.cu:934-1034) runs only inside a request. */
sideaware_status_t sideaware_prealloc(size_t bytes, int device);
/* When the mapped set has to grow and more than start_threshold bytes are mapped but free, free blocks are unmapped,
 * least recently freed first, down to end_threshold (sideaware.cu:1479-1483; the reference's defaults are 16 GiB and
 * 2 GiB).  Until this is called the two are at least a half and a quarter of the device's memory: 16 GiB is a ninth
 * of a B200, and a growing program that crosses it unmaps and maps the same memory again and again. */
void sideaware_free_mapped_thresholds(size_t start_threshold, size_t end_threshold);
/* The reference appends a disassembly of each JIT-ed kernel to this file; this
 * library appends the NVRTC log and the generated source instead. */
void sideaware_write_sass(const char* filename);

/* ---- queries (replaces sideaware.cu:1492-1522) ---------------------------- */
void sideaware_fill_side_index(unsigned char* gpu_array); /* num_sms bytes, device to device */
const char* sideaware_gpu_side_index(void);               /* device pointer, library owned */
const char* sideaware_cpu_side_index(void);               /* host pointer: byte = side | ordinal<<1 */
const int* sideaware_sm_side_summary(void);               /* {num_sms, side0, side1, min, hash|1<<21} */
int sideaware_num_sms(void);
int sideaware_num_sm_side0(void);
int sideaware_num_sm_side1(void);
int sideaware_min_sm_per_side(void);
int sideaware_hash_mask(void);

/* =========================================================================
 * Additions (no counterpart in the reference unless noted).
 * ========================================================================= */

/* Last error text recorded on the calling thread's most recent failing call
 * ("" if none).  The reference reports misuse through assert() only
 * (sideaware.cu:1371-1375); the launchers here stay void and record instead. */
const char* sideaware_last_error(void);
/* Number of errors recorded since load (all threads). */
unsigned long long sideaware_error_count(void);

/* In-place forward RoPE over a packed [B, T, Nq + 2*Nkv, HS] tensor with an
 * fp32 [T, HS/2, 2] cos/sin table; V heads are not touched.  dtype: 0 = fp32,
 * 1 = bf16 (fp32 math, one round-to-nearest-even).  Generalises the reference's
 * fixed-shape functor kernel_rope.cuh:19-60 (MHA, fp32, T=1024) to runtime
 * shapes; arithmetic is that of example_llmc_rope.cu:54-86 without FMA
 * contraction.  Returns 0 or a CUDA error number. */
sideaware_status_t sideaware_rope_forward(void* qkv, const float* freqs_cis,
                                          int B, int T, int Nq, int Nkv, int HS, int dtype,
                                          int device, sideaware_stream_t stream);

/* Backward pass of the same operator, in place on the gradient of the packed tensor:
 * rotation by the opposite angle, V-head gradients untouched.  Arithmetic of the
 * reference's apply_rotary_emb_backward / rope_backward_inplace_kernel1
 * (example_llmc_rope.cu:166-228). */
sideaware_status_t sideaware_rope_backward(void* dqkv, const float* freqs_cis,
                                           int B, int T, int Nq, int Nkv, int HS, int dtype,
                                           int device, sideaware_stream_t stream);

/* Fills the cos/sin table the two calls above read, freqs_cis[end][dim/2][2] fp32, in
 * device memory.  Takes the place of the host function precompute_freqs_cis
 * (example_llmc_rope.cu:19-52): the dim/2 frequencies (with the llama-3 wavelength
 * rescale when use_scaled != 0) are computed on the host with the reference's fp32
 * expression, the end * dim/2 angles t * freq in fp32 on the GPU, their cosine and sine
 * in fp64 rounded once to fp32 (within 1 fp32 ulp of the reference's cosf/sinf, equal
 * in nearly every entry).  dim even, 2 <= dim <= 1024. */
sideaware_status_t sideaware_rope_precompute_freqs(float* freqs_cis, int dim, int end, float theta,
                                                   int use_scaled, int device, sideaware_stream_t stream);

/* out = bf16(a * sigmoid(a) * b * scale), n elements (multiple of 8), the
 * ahead-of-time build of the benchmark's example functor. */
sideaware_status_t sideaware_silu_mul_bf16(void* out, const void* a, const void* b, float scale,
                                           size_t n, int device, sideaware_stream_t stream);

/* Compiles a functor header with NVRTC for sm_100a without loading it, so headers
 * can be checked on a machine without a GPU.  wide != 0 selects the 64-bit index
 * variant.  Returns 0 on success; the compiler log is copied to log_out.  A header that
 * uses threadIdx.y, blockDim.y or a block-wide barrier gets a warning line in log_out even
 * when it compiles: blocks are one-dimensional here and a warp, not a 256-thread group, owns
 * a chunk (the reference launches (256, groups) blocks, sideaware.cu:1407). */
int sideaware_compile_check(const char* header, int wide, char* log_out, size_t log_capacity);

/* Kernel placement policy for all launchers: 0 = side-aware (default),
 * 1 = side-unaware (same kernel, chunk halves chosen without looking at the
 * address), 2 = forced wrong side.  For A/B measurements; the reference offers
 * the same through the FORCE_WRONG_SIDE / FORCE_RANDOM_SIDE functor macros
 * (sideaware.cu:70-75). */
void sideaware_set_placement(int mode);
int sideaware_get_placement(void);
/* memcpy engine: 1 (default) = bulk asynchronous copies (TMA unit) staged through
 * shared memory, 4 KiB per copy; 0 = 128-bit vector loads/stores.  Same results. */
void sideaware_set_memcpy_engine(int engine);
int sideaware_get_memcpy_engine(void);
/* The same choice for sideaware_rope_forward / _backward: 1 = the chunk is brought into
 * shared memory by bulk copies, rotated there and sent back (V heads are never moved),
 * 0 = 128-bit vector loads/stores from registers.  Bit-identical results.  Replaces the
 * reference's JIT-ed kernel with kernel_rope.cuh:1-60 either way. */
void sideaware_set_rope_engine(int engine);
int sideaware_get_rope_engine(void);

/* Per-chunk side map: writes one byte (0/1) per 4 KiB chunk of
 * [ptr, ptr + num_bytes) to host memory, as predicted from the address hash
 * and VA bit 21.  Returns the number of chunks written. */
size_t sideaware_chunk_sides(const void* ptr, size_t num_bytes, unsigned char* host_out);
/* Re-measures, by L2 latency probing on the GPU, the side of `samples` randomly
 * chosen chunks of a live allocation and compares with the prediction.
 * Contents are not modified (atomic add of zero).  Returns the number of
 * mismatches, or -1 on error. */
int sideaware_verify_chunk_sides(const void* ptr, size_t num_bytes, int samples, unsigned seed);

/* Counters of the current device, for tests and monitoring. */
#ifndef SIDEAWARE_STATS_T
#define SIDEAWARE_STATS_T
typedef struct sideaware_stats_t {
    unsigned long long bytes_mapped_live;   /* side-aware blocks handed out */
    unsigned long long bytes_mapped_cached; /* freed but still mapped */
    unsigned long long pages_pool_side0;    /* unmapped physical pages */
    unsigned long long pages_pool_side1;
    unsigned long long pages_created;       /* cuMemCreate successes since start */
    unsigned long long cross_side_pages;    /* pages mapped against their side */
    unsigned long long reuse_hits;
    unsigned long long large_allocs;
    unsigned long long small_allocs;        /* served by cudaMallocAsync */
    unsigned long long trims;               /* threshold/OOM unmap passes */
    unsigned long long jit_compiles;
    unsigned long long kernel_launches;
    unsigned long long probe_confidence_ppm; /* min SM signature margin, 1e6 = perfect */
    unsigned long long hash_validation_errors; /* mispredicted validation offsets at init */
    unsigned long long kernel_wait_timeouts;   /* bounded waits inside kernels that ran out (0 in a healthy run) */
    unsigned long long handles_created;        /* cuMemCreate calls; pages_created counts the 2 MiB pages they hold */
    unsigned long long handles_discarded;      /* handles given back because their pages' sides did not alternate */
    unsigned long long extensions;             /* blocks made of a segment's last free run plus newly mapped pages */
    unsigned long long hole_refills;           /* blocks mapped into a hole that a trim had left inside a segment */
    unsigned long long headroom_pages;         /* pages mapped beyond what requests asked for (sideaware_prealloc_config) */
    unsigned long long top_ups;                /* free calls that mapped extra_alloc pages */
} sideaware_stats_t;
#endif
void sideaware_get_stats(sideaware_stats_t* out);

/* Host time (ns) and call counts the allocator has spent in driver calls since load, by kind:
 * [0] cuMemCreate [1] cuMemRelease [2] cuMemAddressReserve/Free [3] cuMemMap [4] cuMemUnmap
 * [5] cuMemSetAccess [6] side probing [7] synchronisation.  For allocator tuning. */
void sideaware_driver_call_times(unsigned long long ns_out[8], unsigned long long calls_out[8]);

/* Raw discovery data of the current device (latency matrix etc.) as JSON text
 * owned by the library; for diagnostics. */
const char* sideaware_topology_json(void);

/* Copy for callers that cannot allocate device memory.  (No counterpart in the
 * reference.)  Some users of a GPU library run where a cudaMalloc is not an
 * option: a server that handed all of HBM to its own pool at start-up, so any
 * further allocation fails; code that runs inside another allocator's callback
 * and must not re-enter allocation; a shutdown or error path that copies state
 * out after an out-of-memory condition.  sideaware_memcpy cannot serve them on a
 * device it has not seen yet, because its first use of a device allocates probe
 * and bookkeeping buffers.  This entry point never calls cudaMalloc, cudaFree or
 * any allocating routine: the three work counters the copy kernel needs sit in a
 * fixed 512-byte array inside the loaded module (each GPU that loads the library
 * holds those 512 bytes until the process ends).
 *   - num_bytes: multiple of 16, at most SIDEAWARE_NOALLOC_MAX_BYTES (the work
 *     counters are 32 bits wide; the cap keeps them far from wrapping); larger
 *     requests are refused with cudaErrorInvalidValue (1) and a message in
 *     sideaware_last_error().  out/in: 16-byte aligned device pointers.
 *   - The first call on a device looks up the array's device address (a lookup,
 *     not an allocation) with that device made current; make that first call
 *     before starting any stream capture.
 *   - The array is shared by every call and keeps the last call's contents, so
 *     each call first zeroes it on `stream`.  Two calls whose kernels overlap on
 *     the GPU (different streams, or different threads) race on it and may skip
 *     or repeat data: issue these copies on one stream, or order them yourself.
 *   - Side placement is used only if an earlier, allocating call has already
 *     set the device up; otherwise the copy is side-unaware (same result,
 *     slower).  The result is bit-identical to sideaware_memcpy either way. */
#define SIDEAWARE_NOALLOC_MAX_BYTES (1ull << 36) /* 64 GiB per call */
sideaware_status_t sideaware_memcpy_noalloc(void* out, const void* in, size_t num_bytes, int device,
                                            sideaware_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SIDEAWARE_H */
