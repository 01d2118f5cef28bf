/* sideaware_alloc.h — the allocator and the topology queries on their own.
 *
 * For CUDA projects that bring their own kernels and only want memory whose L2 side is known:
 * link or dlopen `sideaware_alloc.so` (python -m l2_torch_alloc_b200.build --alloc-only), which
 * holds no elementwise kernels, no functor compiler and never loads NVRTC.  It takes the place
 * of the reference's single-file subset sideaware_alloc.cu (its extern "C" block, lines
 * 692-762) and exports the same entry points with the same meaning, plus the torch entry
 * points and the diagnostics of the full library.  Every declaration below is identical to
 * the one in sideaware.h; a program may include either header, not both libraries.
 *
 * What a kernel needs to know: side(address) = parity(address & sideaware_hash_mask()) for any
 * address inside a block returned by this allocator (4 KiB granularity; bit 21 of the virtual
 * address stands for the side of the 2 MiB page), and side(SM) = sideaware_cpu_side_index()[smid] & 1.
 */
#ifndef SIDEAWARE_ALLOC_H
#define SIDEAWARE_ALLOC_H

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

/* ---- allocation (sideaware_alloc.cu:694-722, sideaware.cu:1280-1352) ------- */
sideaware_status_t sideaware_malloc_async(void** dev_ptr, size_t size, sideaware_stream_t stream);
sideaware_status_t sideaware_free_async(void* ptr, sideaware_stream_t stream);
sideaware_status_t sideaware_malloc(void** dev_ptr, size_t size); /* waits for the device first */
sideaware_status_t sideaware_free(void* ptr);                     /* waits for the device first */
size_t sideaware_release_unused(void);                            /* bytes given back, all devices */
void* sideaware_malloc_auto(size_t size, int device, sideaware_stream_t stream);   /* NULL on failure */
void sideaware_free_auto(void* ptr, size_t size, int device, sideaware_stream_t stream);

/* ---- configuration (sideaware_alloc.cu:724-734) ---------------------------- */
void sideaware_compression(bool enable);
void sideaware_alloc_threshold(size_t threshold); /* smaller requests of the *_auto calls go to cudaMallocAsync */
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

/* ---- queries (sideaware_alloc.cu:736-762) ----------------------------------- */
void sideaware_fill_side_index(unsigned char* gpu_array); /* num_sms bytes, device to device */
const char* sideaware_gpu_side_index(void);               /* device pointer, library owned */
const char* sideaware_cpu_side_index(void);               /* host pointer: byte = side | ordinal<<1 */
const int* sideaware_sm_side_summary(void);               /* {num_sms, side0, side1, min, hash|1<<21} */
int sideaware_num_sms(void);
int sideaware_num_sm_side0(void);
int sideaware_num_sm_side1(void);
int sideaware_min_sm_per_side(void);
int sideaware_hash_mask(void);

/* ---- additions (no counterpart in the reference) ---------------------------- */
/* Text of the calling thread's last error, "" if none; number of errors recorded since load. */
const char* sideaware_last_error(void);
unsigned long long sideaware_error_count(void);
/* One byte (0/1) per 4 KiB chunk of [ptr, ptr + num_bytes), as predicted from the address. */
size_t sideaware_chunk_sides(const void* ptr, size_t num_bytes, unsigned char* host_out);
/* Re-measures `samples` random chunks of a live allocation by latency probing (contents are not
 * modified) and returns how many are not on the predicted side, -1 on error. */
int sideaware_verify_chunk_sides(const void* ptr, size_t num_bytes, int samples, unsigned seed);

#ifndef SIDEAWARE_STATS_T
#define SIDEAWARE_STATS_T
/* Counters of the current device (the kernel-related ones stay 0 in the allocator-only library). */
typedef struct sideaware_stats_t {
    unsigned long long bytes_mapped_live;   /* side-aware blocks handed out */
    unsigned long long bytes_mapped_cached; /* freed but still mapped */
    unsigned long long pages_pool_side0;    /* unmapped physical pages */
    unsigned long long pages_pool_side1;
    unsigned long long pages_created;       /* 2 MiB pages created since start */
    unsigned long long cross_side_pages;    /* pages mapped against their side */
    unsigned long long reuse_hits;
    unsigned long long large_allocs;
    unsigned long long small_allocs;        /* served by cudaMallocAsync */
    unsigned long long trims;               /* threshold/OOM unmap passes */
    unsigned long long jit_compiles;
    unsigned long long kernel_launches;
    unsigned long long probe_confidence_ppm;   /* min SM signature margin, 1e6 = perfect */
    unsigned long long hash_validation_errors; /* mispredicted validation offsets at init */
    unsigned long long kernel_wait_timeouts;
    unsigned long long handles_created;        /* cuMemCreate calls */
    unsigned long long handles_discarded;      /* handles given back because their pages' sides did not alternate */
    unsigned long long extensions;             /* blocks placed behind the last page of an existing segment */
    unsigned long long hole_refills;           /* blocks mapped into a hole that a trim had left inside a segment */
    unsigned long long headroom_pages;         /* pages mapped beyond what requests asked for (sideaware_prealloc_config) */
    unsigned long long top_ups;                /* free calls that mapped extra_alloc pages */
} sideaware_stats_t;
#endif
void sideaware_get_stats(sideaware_stats_t* out);
/* Host time (ns) and call counts spent in driver calls since load: [0] cuMemCreate [1] cuMemRelease
 * [2] cuMemAddressReserve/Free [3] cuMemMap [4] cuMemUnmap [5] cuMemSetAccess [6] side probing [7] waits. */
void sideaware_driver_call_times(unsigned long long ns_out[8], unsigned long long calls_out[8]);
/* Raw discovery data of the current device as JSON text owned by the library. */
const char* sideaware_topology_json(void);

#ifdef __cplusplus
}
#endif
#endif /* SIDEAWARE_ALLOC_H */
