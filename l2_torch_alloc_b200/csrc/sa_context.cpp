#include "sa_context.hpp"

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#ifndef SIDEAWARE_ALLOC_ONLY
#include "sa_jit.hpp"
#endif

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
namespace {
thread_local std::string t_last_error;
std::atomic<unsigned long long> g_error_total{0};
} // namespace

void sa_set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
    g_error_total.fetch_add(1);
    std::fprintf(stderr, "sideaware: %s\n", buf);
}
const char* sa_last_error_text() { return t_last_error.c_str(); }
unsigned long long sa_error_total() { return g_error_total.load(); }

SaConfig& sa_config() {
    static SaConfig c;
    return c;
}

// ---------------------------------------------------------------------------
// device guard
// ---------------------------------------------------------------------------
SaScopedDevice::SaScopedDevice(int device) {
    if (device < 0) return;
    if (cudaGetDevice(&prev_) != cudaSuccess) return;
    if (prev_ != device) switched_ = cudaSetDevice(device) == cudaSuccess;
}
SaScopedDevice::~SaScopedDevice() {
    if (switched_) cudaSetDevice(prev_);
}

// ---------------------------------------------------------------------------
// CUDA backend of the allocator: driver virtual-memory-management calls
// (the calls the reference makes in sideaware.cu:947-1019 and :1093-1181)
// ---------------------------------------------------------------------------
namespace {

// nanoseconds spent in each kind of backend call (SIDEAWARE_VERBOSE prints them at exit; also in the stats)
struct BackendTimes {
    std::atomic<unsigned long long> ns[8];
    std::atomic<unsigned long long> calls[8];
};
BackendTimes g_times;
enum { T_CREATE, T_RELEASE, T_RESERVE, T_MAP, T_UNMAP, T_ACCESS, T_PROBE, T_SYNC };
struct ScopedTime {
    int k;
    std::chrono::steady_clock::time_point t0;
    explicit ScopedTime(int kind) : k(kind), t0(std::chrono::steady_clock::now()) {}
    ~ScopedTime() {
        g_times.ns[k] += (unsigned long long)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
        g_times.calls[k]++;
    }
};

class CudaBackend : public SaBackend {
public:
    explicit CudaBackend(SaDevice* dev) : dev_(dev), d_(dev->drv) {}

    int create_chunk(uint64_t* handle, int pages, bool compressed) override {
        ScopedTime st(T_CREATE);
        CUmemAllocationProp prop;
        std::memset(&prop, 0, sizeof(prop));
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = dev_->id;
        prop.allocFlags.compressionType = compressed ? CU_MEM_ALLOCATION_COMP_GENERIC : 0;
        CUmemGenericAllocationHandle h = 0;
        CUresult r = d_->MemCreate(&h, (size_t)pages * kSaPageBytes, &prop, 0);
        *handle = (uint64_t)h;
        return (int)r;
    }
    void release_chunk(uint64_t handle) override {
        ScopedTime st(T_RELEASE);
        d_->MemRelease((CUmemGenericAllocationHandle)handle);
    }
    int reserve_va(uint64_t* va, size_t bytes) override {
        ScopedTime st(T_RESERVE);
        CUdeviceptr p = 0;
        CUresult r = d_->MemAddressReserve(&p, bytes, kSaPageBytes, 0, 0);
        *va = (uint64_t)p;
        return (int)r;
    }
    void free_va(uint64_t va, size_t bytes) override {
        ScopedTime st(T_RESERVE);
        d_->MemAddressFree((CUdeviceptr)va, bytes);
    }
    int map_chunk(uint64_t va, uint64_t handle, int pages) override {
        ScopedTime st(T_MAP);
        return (int)d_->MemMap((CUdeviceptr)va, (size_t)pages * kSaPageBytes, 0, (CUmemGenericAllocationHandle)handle, 0);
    }
    void unmap_chunk(uint64_t va, int pages) override {
        ScopedTime st(T_UNMAP);
        d_->MemUnmap((CUdeviceptr)va, (size_t)pages * kSaPageBytes);
    }
    int set_access(uint64_t va, size_t bytes) override {
        ScopedTime st(T_ACCESS);
        CUmemAccessDesc acc;
        std::memset(&acc, 0, sizeof(acc));
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = dev_->id;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        return (int)d_->MemSetAccess((CUdeviceptr)va, bytes, &acc, 1);
    }
    int probe_pages(const uint64_t* vas, int n, uint8_t* sides, void* /*stream*/) override {
        ScopedTime st(T_PROBE);
        // fresh pages have no pending work: probe on the library's own stream so the
        // caller's stream is not drained
        int ambiguous = 0;
        cudaError_t e = sa_probe_sides(dev_->probe, dev_->topo, vas, n, sides, dev_->probe_stream, &ambiguous);
        return e == cudaSuccess ? 0 : 1000 + (int)e;
    }
    void device_sync() override {
        ScopedTime st(T_SYNC);
        cudaDeviceSynchronize();
    }
    // An event recorded on `earlier` now stands for all work queued there so far; `later` waits for it on
    // the device.  Called under the allocator's lock, so one event per device is enough (a wait refers to
    // the record that preceded it, recording again later does not change it).  If the stream that used
    // the memory is gone, or anything else fails, the whole device is waited for instead.
    void order_after(void* earlier, void* later) override {
        ScopedTime st(T_SYNC);
        if (!order_event_ && cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming) != cudaSuccess) order_event_ = nullptr;
        if (order_event_ && cudaEventRecord(order_event_, (cudaStream_t)earlier) == cudaSuccess &&
            cudaStreamWaitEvent((cudaStream_t)later, order_event_, 0) == cudaSuccess)
            return;
        cudaGetLastError(); // the failed call's error must not stick to the caller's next launch
        cudaDeviceSynchronize();
    }

private:
    SaDevice* dev_;
    const SaDriver* d_;
    cudaEvent_t order_event_ = nullptr;
};

std::mutex g_devices_mu;
std::vector<std::unique_ptr<SaDevice>> g_devices;

bool init_device(SaDevice* dev) {
    SaScopedDevice guard(dev->id);
    auto fail = [&](const std::string& why) {
        dev->failed = true;
        dev->fail_why = why;
        sa_set_error("device %d: %s", dev->id, why.c_str());
        return false;
    };
    cudaError_t e = cudaFree(nullptr); // creates / binds the primary context
    if (e != cudaSuccess) return fail(std::string("cannot initialise CUDA: ") + cudaGetErrorString(e));
    std::string why;
    dev->drv = sa_driver(&why);
    if (!dev->drv) return fail(why);

    int major = 0, minor = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev->id);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev->id);
    if (major != 10)
        return fail("compute capability " + std::to_string(major) + "." + std::to_string(minor) +
                    " is not supported: this library is built for sm_100a (B200) only");

    // physical allocation granularity must be the 2 MiB page the side map is kept at (sideaware.cu:826-834)
    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev->id;
    size_t gran = 0;
    CUresult r = dev->drv->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
    if (r != CUDA_SUCCESS) return fail("cuMemGetAllocationGranularity: " + sa_cu_error(dev->drv, r));
    if (gran != kSaPageBytes) return fail("allocation granularity is " + std::to_string(gran) + " bytes, expected 2 MiB");
    int comp = 0;
    dev->drv->DeviceGetAttribute(&comp, CU_DEVICE_ATTRIBUTE_GENERIC_COMPRESSION_SUPPORTED, dev->id);
    dev->compression_supported = comp != 0;

    // a dedicated physical page for discovery (the reference probes inside its metadata page, sideaware.cu:844-853)
    CUmemGenericAllocationHandle h = 0;
    if ((r = dev->drv->MemCreate(&h, kSaPageBytes, &prop, 0)) != CUDA_SUCCESS) return fail("cuMemCreate(probe page): " + sa_cu_error(dev->drv, r));
    CUdeviceptr va = 0;
    if ((r = dev->drv->MemAddressReserve(&va, kSaPageBytes, kSaPageBytes, 0, 0)) != CUDA_SUCCESS) {
        dev->drv->MemRelease(h);
        return fail("cuMemAddressReserve(probe page): " + sa_cu_error(dev->drv, r));
    }
    CUmemAccessDesc acc;
    std::memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev->id;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if ((r = dev->drv->MemMap(va, kSaPageBytes, 0, h, 0)) != CUDA_SUCCESS ||
        (r = dev->drv->MemSetAccess(va, kSaPageBytes, &acc, 1)) != CUDA_SUCCESS) {
        dev->drv->MemAddressFree(va, kSaPageBytes);
        dev->drv->MemRelease(h);
        return fail("mapping the probe page: " + sa_cu_error(dev->drv, r));
    }
    dev->probe_page_va = (uint64_t)va;
    dev->probe_page_handle = (unsigned long long)h;
    if ((e = cudaMemset((void*)va, 0, kSaPageBytes)) != cudaSuccess) return fail(std::string("cudaMemset(probe page): ") + cudaGetErrorString(e));
    if ((e = cudaStreamCreateWithFlags(&dev->probe_stream, cudaStreamNonBlocking)) != cudaSuccess)
        return fail(std::string("cudaStreamCreate: ") + cudaGetErrorString(e));

    if ((e = sa_probe_create(dev->id, dev->probe_page_va, &dev->probe, &dev->topo, &why)) != cudaSuccess) return fail(why);

    // SIDEAWARE_FORCE_HASH overrides the detected hash (the reference has a compile-time FORCED_HASH, sideaware.cu:401)
    if (const char* fh = std::getenv("SIDEAWARE_FORCE_HASH")) {
        unsigned long v = std::strtoul(fh, nullptr, 0);
        if (v) { dev->topo.hash = (uint32_t)v & 0x1FFFF0u; dev->topo.hash_usable = (v & 4096u) && !(v & 4095u); }
    }
    dev->full_hash = dev->topo.hash_usable ? (dev->topo.hash | (1u << kSaSideBit)) : 0u;
    if (!dev->topo.hash_usable)
        std::fprintf(stderr, "sideaware: device %d: no usable side hash found (hash 0x%x, %d validation errors, confidence %.2f); "
                             "kernels run side-unaware\n", dev->id, dev->topo.hash, dev->topo.validation_errors, dev->topo.confidence);
    std::memcpy(dev->side_table.side_of_sm, dev->topo.side_index, SA_MAX_SM);
    dev->summary[0] = dev->topo.num_sms;
    dev->summary[1] = dev->topo.count[0];
    dev->summary[2] = dev->topo.count[1];
    dev->summary[3] = dev->topo.min_per_side;
    dev->summary[4] = (int)(dev->topo.hash | (1u << kSaSideBit));

    dev->backend.reset(new CudaBackend(dev));
    size_t free_bytes = 0, total_bytes = 0;
    cudaMemGetInfo(&free_bytes, &total_bytes);
    dev->alloc.reset(new SaAllocator(dev->backend.get(), dev->compression_supported, total_bytes));
#ifndef SIDEAWARE_ALLOC_ONLY
    dev->jit = sa_jit_new_device_cache();
#endif
    if (const char* dump = std::getenv("SIDEAWARE_DUMP_TOPOLOGY")) {
        std::string path = std::string(dump) + "." + std::to_string(dev->id) + ".json";
        if (FILE* f = std::fopen(path.c_str(), "w")) { std::fputs(dev->topo.json.c_str(), f); std::fclose(f); }
    }
    dev->ready.store(true, std::memory_order_release);
    return true;
}

} // namespace

SaDevice::~SaDevice() {}

SaDevice* sa_device(int device) {
    if (device < 0) {
        if (cudaGetDevice(&device) != cudaSuccess) {
            sa_set_error("no CUDA device available (this library has no CPU path)");
            return nullptr;
        }
    }
    SaDevice* dev = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_devices_mu);
        if (g_devices.empty()) {
            int count = 0;
            if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
                sa_set_error("no CUDA device available (this library has no CPU path)");
                return nullptr;
            }
            g_devices.resize(count);
        }
        if (device >= (int)g_devices.size()) {
            sa_set_error("device %d out of range (%zu devices)", device, g_devices.size());
            return nullptr;
        }
        if (!g_devices[device]) {
            g_devices[device].reset(new SaDevice());
            g_devices[device]->id = device;
        }
        dev = g_devices[device].get();
    }
    std::lock_guard<std::mutex> lock(dev->mu);
    if (dev->ready) return dev;
    if (dev->failed) {
        sa_set_error("device %d unusable: %s", device, dev->fail_why.c_str());
        return nullptr;
    }
    return init_device(dev) ? dev : nullptr;
}

std::vector<SaDevice*> sa_initialised_devices() {
    std::lock_guard<std::mutex> lock(g_devices_mu);
    std::vector<SaDevice*> out;
    for (auto& d : g_devices)
        if (d && d->ready) out.push_back(d.get());
    return out;
}

bool sa_prepare_launch(SaDevice* dev, void* stream, uint64_t track_addr, uint64_t num_vecs, int parallel_groups,
                       int forced_per_side, bool reverse, SaSched* s, int* grid, int* threads, int exact_warps) {
    std::memset(s, 0, sizeof(*s));
    int groups = parallel_groups > 0 ? parallel_groups : 4;
    if (groups > 4) groups = 4;
    int warps = exact_warps > 0 ? exact_warps : groups * 8;
    int g = dev->topo.num_sms;
    if (forced_per_side > 0 && 2 * forced_per_side < g) g = 2 * forced_per_side;
    s->dc_per_ticket = 0;
    sa_sched_geometry(*s, track_addr, num_vecs, (uint32_t)(g * warps / 2));
    sa_sched_grid(*s, g, warps, &g, dev->topo.count[0], dev->topo.count[1]);
    bool overlap = false;
    s->tickets = sa_probe_ticket_slot(dev->probe, stream, &overlap);
    if (!s->tickets) {
        sa_set_error("no ticket slot for stream %p on device %d (device memory exhausted, or a new stream first used while capturing)", stream, dev->id);
        return false;
    }
    s->overlap = overlap ? 1u : 0u;
    s->hash = dev->full_hash;
    int placement = sa_config().placement.load();
    s->placement = dev->full_hash ? (uint32_t)placement : (uint32_t)SA_PLACE_UNAWARE;
    s->reverse = reverse ? 1u : 0u;
    *grid = g;
    *threads = warps * 32;
    dev->launches.fetch_add(1);
    return true;
}

void sa_report_wait_timeouts(SaDevice* dev, const char* what) {
    const unsigned long long now = sa_probe_wait_timeouts(dev->probe);
    unsigned long long seen = dev->wait_timeouts_reported.load();
    if (now > seen && dev->wait_timeouts_reported.compare_exchange_strong(seen, now))
        sa_set_error("%s: %llu bounded waits ran out in bulk-copy kernels launched earlier on device %d; the chunks concerned "
                     "were moved with ordinary loads and stores instead", what, now - seen, dev->id);
}

SaDevice* sa_device_if_ready(int device) {
    std::lock_guard<std::mutex> lock(g_devices_mu);
    if (device < 0 || device >= (int)g_devices.size() || !g_devices[device]) return nullptr;
    SaDevice* dev = g_devices[device].get();
    return dev->ready.load(std::memory_order_acquire) ? dev : nullptr;
}

void sa_backend_times(unsigned long long ns_out[8], unsigned long long calls_out[8]) {
    for (int i = 0; i < 8; ++i) {
        ns_out[i] = g_times.ns[i].load();
        calls_out[i] = g_times.calls[i].load();
    }
}
