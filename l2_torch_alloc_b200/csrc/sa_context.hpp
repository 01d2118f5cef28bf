// Per-device state of the library and the process-wide configuration.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "sa_alloc.hpp"
#include "sa_driver.hpp"
#include "sa_probe.hpp"

struct SaJitDeviceCache; // sa_jit.cpp

struct SaConfig {
    std::mutex mu;
    SaAllocConfig alloc;
    size_t threshold = 8ull << 20; // sizes below go to cudaMallocAsync in the *_auto entry points
    std::string log_file;          // JIT log destination ("" = none)
    std::atomic<int> placement{0};
    std::atomic<int> memcpy_engine{1}; // 0 = vector loads/stores, 1 = bulk copies through shared memory
    std::atomic<int> rope_engine{0};   // the same choice for the RoPE kernels
};
SaConfig& sa_config();

struct SaDevice {
    int id = -1;
    std::mutex mu;
    std::atomic<bool> ready{false}; // set last by the set-up, read without the lock by sa_device_if_ready
    bool failed = false;
    std::string fail_why;
    const SaDriver* drv = nullptr;
    SaTopology topo;
    SaProbeDevice* probe = nullptr;
    uint64_t probe_page_va = 0;
    unsigned long long probe_page_handle = 0;
    cudaStream_t probe_stream = nullptr;
    bool compression_supported = false;
    std::unique_ptr<SaBackend> backend;
    std::unique_ptr<SaAllocator> alloc;
    int summary[5] = {0, 0, 0, 0, 0};
    uint32_t full_hash = 0; // hash | 1 << 21 when usable, else 0
    SaSideTable side_table; // bit 0 of each byte = side of the SM; passed to every kernel
    std::atomic<unsigned long long> small_allocs{0}, launches{0}, jit_compiles{0};
    std::atomic<unsigned long long> wait_timeouts_reported{0}; // of the device's wait-error word, how much has been reported
    SaJitDeviceCache* jit = nullptr;
    std::mutex jit_mu;
    ~SaDevice();
};

// Device `device` (< 0: the calling thread's current device), initialised on first use.
// nullptr after recording an error when the device cannot be set up.
SaDevice* sa_device(int device);
// Every device that has been initialised so far.
std::vector<SaDevice*> sa_initialised_devices();

// Makes `device` current for the lifetime of the object, then restores the previous one.
class SaScopedDevice {
public:
    explicit SaScopedDevice(int device);
    ~SaScopedDevice();
private:
    int prev_ = -1;
    bool switched_ = false;
};

// Error channel: text kept per thread, count kept per process, line written to stderr.
void sa_set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
const char* sa_last_error_text();
unsigned long long sa_error_total();

// Fills the launch-constant scheduling state for an array of `num_vecs` 16-byte vectors
// whose side-tracking array starts at `track_addr`, and picks grid and block size.  The ticket
// slot comes from the ring of `stream`.  False (error recorded) if no slot could be had.
bool sa_prepare_launch(SaDevice* dev, void* stream, uint64_t track_addr, uint64_t num_vecs, int parallel_groups,
                       int forced_per_side, bool reverse, SaSched* s, int* grid, int* threads,
                       int exact_warps = 0); // exact_warps > 0: that many warps per block, whatever the groups say

// Records an error (once per new occurrence) if kernels launched earlier on this device counted waits that
// ran out; called by the launchers of the kernels that have such waits.  Reads host memory only.
void sa_report_wait_timeouts(SaDevice* dev, const char* what);

// The device's state if some earlier call has already set it up, else nullptr.  Never
// initialises anything (so it never allocates).
SaDevice* sa_device_if_ready(int device);

// Time spent in driver calls by kind: create, release, reserve/free VA, map, unmap, set access, probe, sync.
void sa_backend_times(unsigned long long ns_out[8], unsigned long long calls_out[8]);
