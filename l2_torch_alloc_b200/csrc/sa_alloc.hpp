// Side-aware block allocator for one device.
//
// Physical memory is handled as 2 MiB pages, each its own driver handle, sorted by the L2
// side it is homed on and mapped so that bit 21 of a page's virtual address equals its side.
// Mapped pages live in SEGMENTS (one virtual address range each) that stay mapped; a block is
// a run of consecutive pages of one segment.  Because the bit-21 rule holds for every page
// of a segment, any run can be handed out as long as it STARTS on the side that blocks of
// that size start on (equal sizes => equal side patterns), which costs at most one skipped
// page.  Freed runs stay mapped, coalesce with their neighbours and are reused best-fit.
//
// Why not remap pages into a fresh range per block, as the reference does
// (sideaware.cu:1036-1197)?  On B200 the driver needs about 170 us in cuMemSetAccess and 90 us
// in cuMemUnmap PER 2 MiB MAPPING (a 1 GiB block: ~130 ms), while cuMemMap itself takes 1.5 us;
// sub-ranges of a larger handle cannot be mapped separately.  Reusing mappings is the only
// way to make allocation cheap; the driver is only involved when the mapped set has to grow
// or shrink.
//
// Kept from the reference: 2 MiB granularity, bit 21 == side, same page-rounded size => same
// start side (sideaware.cu:1082-1089), free never unmaps (:1254-1273), cross-stream reuse waits
// for the previous user (:1209-1214), the out-of-memory ladder: unmap free memory above a
// threshold, unmap all of it, release all pooled pages (:1233-1252), cross-side fallback with a
// one-time warning (:1137-1151).  Differences: per-device lock; address ranges are released
// with the size they were reserved with (the reference: :1094 vs :896); a page mapped against
// its side returns to the pool of its TRUE side (:1148-1150); compressed and plain pages are
// kept apart; requests larger than the device fail at once.
//
// All device interaction goes through SaBackend, so the state machine is plain C++ and runs
// against a simulated driver in the CPU tests.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <map>
#include <memory>
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
    // side (0/1) of byte 0 of each of the `n` mapped, accessible pages at the addresses `vas`
    virtual int probe_pages(const uint64_t* vas, int n, uint8_t* sides, void* stream) = 0;
    virtual void device_sync() = 0;
    virtual void stream_sync(void* stream) = 0;
};

struct SaAllocConfig {
    size_t trim_start = 16ull << 30; // when the mapped set must grow and more than this is free-but-mapped, unmap
    size_t trim_end = 2ull << 30;    // ... least recently freed runs down to this
    int extra_required = 1;          // accepted for compatibility with the reference's setter; pages are
    int extra_alloc = 10;            // created on demand, straight into the segment that needs them
    bool compression = false;
};

struct SaAllocStats {
    uint64_t bytes_live = 0, bytes_cached = 0, pages_created = 0, cross_side_pages = 0;
    uint64_t reuse_hits = 0, large_allocs = 0, trims = 0, pages_pool[2] = {0, 0};
    uint64_t segments = 0, free_runs = 0;
};

class SaAllocator {
public:
    // capacity_bytes: total device memory (0 = unknown); larger requests fail at once
    SaAllocator(SaBackend* backend, bool compression_supported, size_t capacity_bytes = 0)
        : be_(backend), comp_ok_(compression_supported), capacity_(capacity_bytes) {}
    ~SaAllocator();

    // Returns the block address or 0.  `cfg` is read at every call (the setters are global).
    uint64_t malloc(size_t size, void* stream, const SaAllocConfig& cfg);
    // true if `ptr` was a live block of this allocator (its pages are now free, still mapped)
    bool free(uint64_t ptr, void* stream);
    bool owns(uint64_t ptr);
    // If more than `start` bytes are free-but-mapped: unmap free runs, least recently freed
    // first, until at most `end` bytes are.
    void trim(size_t start, size_t end);
    // Unmaps every free run and releases every pooled page; returns bytes released.
    size_t release_unused();
    SaAllocStats stats();
    // side the first page of blocks of this (page-rounded) size starts on, -1 if never allocated
    int phase_of_size(size_t aligned_size);

private:
    struct Page { uint64_t handle; uint8_t side; };
    struct Segment {
        uint64_t reserved = 0, base = 0;
        size_t reserved_bytes = 0, num_pages = 0, mapped_pages = 0;
        bool compressed = false;
        std::vector<Page> pages; // handle 0 = unmapped hole
    };
    struct Run { // free, mapped, inside one segment
        size_t pages = 0;
        Segment* seg = nullptr;
        uint64_t freed_seq = 0;
        void* stream = nullptr; // stream of the last user(s); mixed = several
        bool mixed = false;
    };
    struct Block {
        size_t pages = 0, requested = 0;
        Segment* seg = nullptr;
        void* stream = nullptr;
    };

    uint64_t take_from_free(size_t pages, int phase, bool compressed, void* stream);
    uint64_t grow(size_t pages, int phase, bool compressed, void* stream, const SaAllocConfig& cfg);
    void insert_free(uint64_t va, Run run);
    void erase_free(std::map<uint64_t, Run>::iterator it);
    void unmap_run(uint64_t va, const Run& run);
    void trim_locked(size_t start, size_t end);
    void release_pools();
    int choose_phase(size_t bytes, size_t pages, bool compressed);

    SaBackend* be_;
    bool comp_ok_;
    size_t capacity_ = 0;
    std::mutex mu_;
    std::vector<Page> pool_[2][2]; // unmapped pages [compressed][side]
    std::vector<std::unique_ptr<Segment>> segments_;
    std::map<uint64_t, Run> free_;                     // free runs by address
    std::multimap<size_t, uint64_t> free_by_len_[2];   // [compressed]: pages -> address
    std::unordered_map<uint64_t, Block> live_;
    std::unordered_map<size_t, int> phase_;
    size_t cached_bytes_ = 0, live_bytes_ = 0;
    uint64_t seq_ = 0;
    bool warned_cross_ = false;
    SaAllocStats st_;
};
