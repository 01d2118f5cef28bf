// Side-aware block allocator for one device: physical 2 MiB pages sorted by the
// L2 side they are homed on, mapped into virtual address ranges so that bit 21
// of a page's virtual address equals its side, with an exact-size reuse cache
// of still-mapped blocks and a staged out-of-memory ladder.
//
// All device interaction goes through SaBackend, so the state machine is plain
// C++ and runs against a simulated driver in the CPU tests.
//
// Behaviour follows the reference's allocator (sideaware.cu:873-926 unmap and
// release, :934-1034 page pool, :1036-1197 mapping, :1199-1273 cache, ladder
// and free).  Deliberate differences: per-device lock; the address range is
// released with the size it was reserved with (the reference reserves size+1
// page and frees size+2 pages, :1094 vs :896); a page mapped against its side
// for lack of matching pages goes back to the pool of its TRUE side (the
// reference records the wanted side, :1148-1150); compressed and plain pages
// are pooled separately; the cache is trimmed least-recently-freed first.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>
#include <vector>

constexpr size_t kSaPageBytes = 2u << 20;
constexpr int kSaSideBit = 21;

// Result codes of backend calls: 0 = success, anything else = failure
// (the CUDA backend returns CUresult values).
struct SaBackend {
    virtual ~SaBackend() {}
    virtual int create_page(uint64_t* handle, bool compressed) = 0;
    virtual void release_page(uint64_t handle) = 0;
    virtual int reserve_va(uint64_t* va, size_t bytes) = 0; // 2 MiB aligned
    virtual void free_va(uint64_t va, size_t bytes) = 0;
    virtual int map_page(uint64_t va, uint64_t handle) = 0;
    virtual void unmap_page(uint64_t va) = 0;
    virtual int set_access(uint64_t va, size_t bytes) = 0;
    // side (0/1) of byte 0 of `n` consecutive mapped pages starting at `va`
    virtual int probe_pages(uint64_t va, int n, uint8_t* sides, void* stream) = 0;
    virtual void device_sync() = 0;
    virtual void stream_sync(void* stream) = 0;
};

struct SaAllocConfig {
    size_t trim_start = 16ull << 30; // unmap cached blocks on a cache miss once more than this is cached
    size_t trim_end = 2ull << 30;    // ... down to this
    int extra_required = 1;
    int extra_alloc = 10;
    bool compression = false;
    int max_probe_batch = 1024;      // pages probed per temporary mapping
};

struct SaAllocStats {
    uint64_t bytes_live = 0, bytes_cached = 0, pages_created = 0, cross_side_pages = 0;
    uint64_t reuse_hits = 0, large_allocs = 0, trims = 0, pages_pool[2] = {0, 0};
};

class SaAllocator {
public:
    // capacity_bytes: total device memory (0 = unknown); larger requests fail at once
    SaAllocator(SaBackend* backend, bool compression_supported, size_t capacity_bytes = 0)
        : be_(backend), comp_ok_(compression_supported), capacity_(capacity_bytes) {}
    ~SaAllocator();

    // Returns the block address or 0.  `cfg` is read at every call (the setters are global).
    uint64_t malloc(size_t size, void* stream, const SaAllocConfig& cfg);
    // true if `ptr` was a live block of this allocator (it is now cached, still mapped)
    bool free(uint64_t ptr, void* stream);
    bool owns(uint64_t ptr);
    // Unmaps cached blocks (least recently freed first) while more than `end` bytes stay cached,
    // provided more than `start` bytes are cached now.
    void trim(size_t start, size_t end);
    // Unmaps every cached block and releases every pooled page; returns bytes released.
    size_t release_unused();
    SaAllocStats stats();
    // side the first page of blocks of this (page-rounded) size starts on, -1 if never allocated
    int phase_of_size(size_t aligned_size);

private:
    struct Page { uint64_t handle; uint8_t side; };
    struct Block {
        uint64_t base = 0, reserved = 0;
        size_t reserved_bytes = 0, bytes = 0, requested = 0;
        bool compressed = false;
        void* stream = nullptr;
        uint64_t freed_seq = 0;
        std::vector<Page> pages;
    };

    int top_up(size_t num_pages, bool compressed, void* stream, const SaAllocConfig& cfg);
    int create_pages(int count, bool compressed, void* stream, const SaAllocConfig& cfg, int* created);
    bool build_block(Block& b, size_t size, bool compressed, void* stream, const SaAllocConfig& cfg);
    void unmap_block(Block& b);
    void trim_locked(size_t start, size_t end);
    static uint64_t cache_key(size_t bytes, bool compressed) { return (uint64_t)bytes | (compressed ? 1ull : 0ull); }

    SaBackend* be_;
    bool comp_ok_;
    size_t capacity_ = 0;
    std::mutex mu_;
    std::vector<Page> pool_[2][2]; // [compressed][side]
    std::unordered_map<uint64_t, Block> live_;
    std::unordered_map<uint64_t, std::vector<Block>> cache_;
    std::unordered_map<size_t, int> phase_;
    size_t cached_bytes_ = 0;
    uint64_t seq_ = 0;
    uint64_t seen_side_[2] = {0, 0}; // sides of all pages ever created
    bool warned_cross_ = false;
    SaAllocStats st_;
};
