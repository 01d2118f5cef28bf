// CPU tests of the library's host-side logic, built with g++ (no GPU, no CUDA calls):
//   sched     every 16-byte vector is visited exactly once by the ticket scheduler,
//             for any side placement, hash, base address and array length
//   alloc     allocator state machine on a simulated driver with fault injection
//   topology  SM-side / hash discovery on synthetic latency matrices
//   ring      stage bookkeeping of the bulk-copy kernels, with loads that never arrive
// Usage: test_core <sched|alloc|chunks|topology|ring|all>
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <random>
#include <set>
#include <string>
#include <vector>

#include "../../l2_torch_alloc_b200/csrc/sa_alloc.hpp"
#include "../../l2_torch_alloc_b200/csrc/sa_bulk.cuh"
#include "../../l2_torch_alloc_b200/csrc/sa_probe.hpp"
#include "../../l2_torch_alloc_b200/csrc/sa_sched.cuh"

static int g_failures = 0;
#define CHECK(cond)                                                                  \
    do {                                                                             \
        if (!(cond)) {                                                               \
            std::printf("CHECK failed: %s  (%s:%d)\n", #cond, __FILE__, __LINE__);   \
            ++g_failures;                                                            \
        }                                                                            \
    } while (0)

// ---------------------------------------------------------------------------
// scheduler: replay what the device loop does (sa_for_each_chunk) for both sides
// ---------------------------------------------------------------------------
static void sched_case(uint64_t addr, uint64_t num_vecs, uint32_t hash, uint32_t placement, bool reverse,
                       uint32_t warps_per_side, uint32_t forced_dc_per_ticket) {
    SaSched s;
    std::memset(&s, 0, sizeof(s));
    s.hash = hash;
    s.placement = placement;
    s.reverse = reverse;
    s.dc_per_ticket = forced_dc_per_ticket;
    sa_sched_geometry(s, addr, num_vecs, warps_per_side);
    CHECK(s.lead < SA_DC_VECS);
    CHECK(s.end == s.lead + num_vecs);
    CHECK((uint64_t)s.num_tickets * s.dc_per_ticket >= s.num_dc);
    std::vector<uint8_t> hits(num_vecs, 0);
    std::vector<uint8_t> by_side(num_vecs, 0);
    for (uint32_t side = 0; side < 2; ++side)
        for (uint32_t t = 0; t < s.num_tickets; ++t)
            for (uint32_t d = 0; d < s.dc_per_ticket; ++d) {
                sa_u64 first;
                if (!sa_ticket_chunk(s, t, d, side, &first)) break;
                if (!(first < s.end && first + SA_CHUNK_VECS > s.lead)) continue;
                for (uint32_t v = 0; v < SA_CHUNK_VECS; ++v) {
                    uint64_t a = first + v;
                    if (a >= s.lead && a < s.end) {
                        hits[a - s.lead]++;
                        by_side[a - s.lead] = (uint8_t)side;
                    }
                }
            }
    bool once = true;
    for (uint64_t i = 0; i < num_vecs; ++i) once = once && hits[i] == 1;
    CHECK(once);
    // in aware mode the worker's side equals the hash-predicted side of the byte address
    if (placement == SA_PLACE_AWARE && hash) {
        bool match = true;
        for (uint64_t i = 0; i < num_vecs; i += 37) {
            uint32_t predicted = sa_parity32((uint32_t)(addr + i * 16) & hash);
            match = match && predicted == by_side[i];
        }
        CHECK(match);
    }
    if (placement == SA_PLACE_WRONG && hash) {
        bool inverted = true;
        for (uint64_t i = 0; i < num_vecs; i += 41) {
            uint32_t predicted = sa_parity32((uint32_t)(addr + i * 16) & hash);
            inverted = inverted && predicted != by_side[i];
        }
        CHECK(inverted);
    }
}

// What the blocks of one launch do with the ticket counters, block after block (one of the orders the hardware
// may run them in): opening batch, per-warp claims, block-wide sweep of both sides.  Mirrors sa_for_each_chunk.
static void sched_grid_replay(const SaSched& s, int grid, int blocks_on_side0, int order, std::mt19937_64& rng) {
    const uint32_t M = s.num_tickets;
    std::vector<uint32_t> worked[2] = {std::vector<uint32_t>(M, 0), std::vector<uint32_t>(M, 0)};
    uint32_t counter[2] = {0, 0};
    std::vector<int> blocks(grid);
    for (int b = 0; b < grid; ++b) blocks[b] = b;
    if (order == 1) std::reverse(blocks.begin(), blocks.end());
    if (order == 2) std::shuffle(blocks.begin(), blocks.end(), rng);
    auto work = [&](uint32_t side, uint32_t t) {
        if (t < M) worked[side][t]++;
    };
    for (int b : blocks) {
        const uint32_t my = b < blocks_on_side0 ? 0u : 1u;
        const uint32_t base = counter[my];
        counter[my] += s.opening[my];
        bool drained = false;
        for (uint32_t warp = 0; warp < s.active_warps; ++warp) {
            for (uint32_t dealt = 0; dealt < s.share; ++dealt) {
                const uint32_t mine = dealt * s.active_warps + warp;
                if (mine >= s.opening[my]) break;
                work(my, base + mine);
            }
            if (s.dynamic) {
                for (;;) {
                    if (drained) break;
                    const uint32_t t = counter[my]++;
                    if (t >= M) { drained = true; break; }
                    work(my, t);
                }
            }
        }
        for (;;) { // block-wide leftovers, both sides
            const uint32_t a = counter[my], o = counter[my ^ 1u];
            counter[my] += s.active_warps;
            counter[my ^ 1u] += s.active_warps;
            if (a >= M && o >= M) break;
            for (uint32_t warp = 0; warp < s.active_warps; ++warp) {
                work(my, a + warp);
                work(my ^ 1u, o + warp);
            }
        }
    }
    bool once = true;
    for (uint32_t side = 0; side < 2; ++side)
        for (uint32_t t = 0; t < M; ++t) once = once && worked[side][t] == 1;
    CHECK(once);
}

static void test_sched() {
    const uint32_t hashes[] = {0x1EF000u | (1u << 21), 0xB3000u | (1u << 21), 0x1000u | (1u << 21), 0u};
    std::mt19937_64 rng(1234);
    // dense small sizes: every vector count up to 3 double chunks, aligned and unaligned bases
    for (uint64_t n = 1; n <= 3 * SA_DC_VECS + 5; n += (n < 40 ? 1 : 61)) {
        for (uint64_t off : {0ull, 16ull, 4096ull, 4112ull, 8176ull}) {
            sched_case(0x7f0000200000ull + off, n, hashes[0], SA_PLACE_AWARE, false, 2368, 0);
            sched_case(0x7f0000200000ull + off, n, hashes[1], SA_PLACE_UNAWARE, true, 8, 0);
        }
    }
    // shapes the reference's own test copies (test.py:310-326), in 16-byte vectors
    const uint64_t shapes[] = {4ull * 777 * 4 / 16, 1000ull * 1000 * 2 / 16, 1000ull * 1000 * 8 / 16, 10000ull * 1000 * 4 / 16};
    for (uint64_t n : shapes)
        for (uint32_t p : {SA_PLACE_AWARE, SA_PLACE_UNAWARE, SA_PLACE_WRONG})
            sched_case(0x7f1234600000ull, n, hashes[0], p, false, 2368, 0);
    // random cases: sizes up to 64 MiB, any 16-byte aligned base, every ticket length
    for (int i = 0; i < 60; ++i) {
        uint64_t n = 1 + rng() % (4u << 20);
        uint64_t addr = 0x7e0000000000ull + (rng() % (1ull << 30)) * 16;
        uint32_t per = (uint32_t)(rng() % 9); // 0 = automatic
        sched_case(addr, n, hashes[rng() % 4], (uint32_t)(rng() % 3), rng() & 1, 1 + rng() % 3000, per);
    }
    // hand-out policy: the opening batches never ask for more warps than a block has, always deal
    // at least one ticket, cover small arrays completely on a balanced device, and never launch more
    // blocks than there are tickets
    for (uint64_t n : {1ull, 300ull, 512ull * 100, 4ull << 16, 1ull << 20, 4ull << 20, 1ull << 24, 1ull << 26, 1ull << 30}) {
        for (int warps : {8, 16, 24, 32}) {
            SaSched s;
            std::memset(&s, 0, sizeof(s));
            sa_sched_geometry(s, 0x7f0000000000ull, n, 74 * warps);
            int grid = 0;
            sa_sched_grid(s, 148, warps, &grid);
            CHECK(grid >= 1 && grid <= 148 && (uint64_t)grid <= 2ull * s.num_tickets);
            CHECK(s.active_warps >= 1 && s.active_warps <= (uint32_t)warps && s.share >= 1);
            CHECK(s.total_blocks == (uint32_t)grid);
            uint64_t dealt = (uint64_t)((grid + 1) / 2) * s.active_warps * s.share;
            if (!s.dynamic) CHECK(dealt >= s.num_tickets);
            if (s.dynamic) CHECK(dealt < s.num_tickets && s.active_warps == (uint32_t)warps);
        }
    }
    // the block loop itself (sa_for_each_chunk), replayed on the host: every ticket of both sides is worked on
    // exactly once whatever side the blocks find themselves on - one block per SM with equal or unequal
    // sides, all blocks on one side, fewer blocks than planned for
    for (uint64_t n : {1ull, 700ull, 512ull * 100, 1ull << 18, 1ull << 21, 1ull << 22, 3ull << 22, 1ull << 26, 1ull << 28}) {
        for (int warps : {8, 16, 24, 32}) {
            for (int split : {74, 70, 60, 148, 0}) {
                SaSched s;
                std::memset(&s, 0, sizeof(s));
                sa_sched_geometry(s, 0x7f0000000000ull, n, 74 * warps);
                int grid = 0;
                sa_sched_grid(s, 148, warps, &grid, split, 148 - split);
                CHECK(s.opening[0] <= s.active_warps * s.share && s.opening[1] <= s.active_warps * s.share);
                CHECK(s.opening[0] >= 1 && s.opening[1] >= 1);
                for (int order = 0; order < 3; ++order) sched_grid_replay(s, grid, split, order, rng);
            }
        }
    }
    std::printf("sched: done\n");
}

// ---------------------------------------------------------------------------
// allocator on a simulated driver
// ---------------------------------------------------------------------------
// Simulated driver.  Physical memory is a line of 2 MiB pages handed out in order (memory that
// was released is handed out again first, most recently released first).  Sides of consecutive
// pages follow one of three models:
//   0  what was measured on B200: alternating inside groups of 8 pages; at most group boundaries
//      the side repeats once
//   1  independent random sides (bias_percent = chance of side 1)
//   2  model 0 with the line starting inside a group (a process that created pages before)
struct FakeDriver : SaBackend {
    static int default_model;
    int model = default_model;
    uint64_t next_handle = 1, next_va = 0x7f0000000000ull;
    size_t capacity_pages = 1 << 20;
    size_t next_phys = 0;
    std::vector<std::pair<size_t, size_t>> holes;            // released physical ranges (start, pages), newest last
    std::map<size_t, int> random_side;                        // model 1: side of a physical page once drawn
    struct Handle { size_t phys; int pages; };
    std::map<uint64_t, Handle> handles;                       // live handles
    std::map<uint64_t, size_t> reservations;                  // va -> bytes
    std::map<uint64_t, std::pair<uint64_t, int>> mappings;    // page va -> (handle, page of the handle)
    std::set<uint64_t> accessible;
    std::mt19937 rng{7};
    int fail_create_after = -1, fail_map_after = -1, fail_reserve_after = -1, fail_access_after = -1, fail_probe_after = -1;
    int syncs = 0, stream_syncs = 0, creates = 0, maps = 0, unmaps = 0;
    int bias_percent = 50;

    FakeDriver() { if (model == 2) next_phys = 3; }
    static bool tick(int& counter) {
        if (counter < 0) return false;
        if (counter == 0) { counter = -1; return true; }
        --counter;
        return false;
    }
    size_t live_pages() const {
        size_t n = 0;
        for (auto& h : handles) n += (size_t)h.second.pages;
        return n;
    }
    int side_of_phys(size_t k) {
        if (model == 1) {
            auto it = random_side.find(k);
            if (it == random_side.end()) it = random_side.emplace(k, (int)(rng() % 100) < bias_percent).first;
            return it->second;
        }
        // start side of group g: repeats the last side of group g-1 (a "flip" of the alternation) except at every 8th boundary
        const size_t g = k / 8;
        int start = 0;
        for (size_t b = 1; b <= g; ++b) start ^= (b % 8 == 5) ? 0 : 1;
        return start ^ (int)(k & 1);
    }
    int create_chunk(uint64_t* handle, int pages, bool) override {
        ++creates;
        if (tick(fail_create_after) || live_pages() + (size_t)pages > capacity_pages) return 2;
        size_t phys = 0;
        bool reused = false;
        for (size_t i = holes.size(); i-- > 0 && !reused;)
            if (holes[i].second >= (size_t)pages) {
                phys = holes[i].first;
                holes[i].first += (size_t)pages;
                holes[i].second -= (size_t)pages;
                if (holes[i].second == 0) holes.erase(holes.begin() + (long)i);
                reused = true;
            }
        if (!reused) { phys = next_phys; next_phys += (size_t)pages; }
        *handle = next_handle++;
        handles[*handle] = Handle{phys, pages};
        return 0;
    }
    void release_chunk(uint64_t handle) override {
        CHECK(handles.count(handle) == 1);
        for (auto& m : mappings) CHECK(m.second.first != handle);
        holes.emplace_back(handles[handle].phys, (size_t)handles[handle].pages);
        handles.erase(handle);
    }
    int reserve_va(uint64_t* va, size_t bytes) override {
        if (tick(fail_reserve_after)) return 2;
        CHECK(bytes % kSaPageBytes == 0);
        // alternate the bit-21 phase of what the "driver" returns
        if (rng() & 1) next_va += kSaPageBytes;
        *va = next_va;
        next_va += bytes + 4 * kSaPageBytes;
        reservations[*va] = bytes;
        return 0;
    }
    void free_va(uint64_t va, size_t bytes) override {
        auto it = reservations.find(va);
        CHECK(it != reservations.end());
        if (it != reservations.end()) {
            CHECK(it->second == bytes); // the range must be freed with the size it was reserved with
            for (auto& m : mappings) CHECK(!(m.first >= va && m.first < va + bytes));
            reservations.erase(it);
        }
    }
    bool reserved(uint64_t va, size_t bytes) {
        for (auto& r : reservations)
            if (va >= r.first && va + bytes <= r.first + r.second) return true;
        return false;
    }
    int map_chunk(uint64_t va, uint64_t handle, int pages) override {
        ++maps;
        if (tick(fail_map_after)) return 1;
        CHECK(reserved(va, (size_t)pages * kSaPageBytes));
        CHECK(handles.count(handle) == 1 && handles[handle].pages == pages); // a handle is mapped whole or not at all
        for (auto& m : mappings) CHECK(m.second.first != handle);
        for (int k = 0; k < pages; ++k) {
            CHECK(mappings.count(va + (uint64_t)k * kSaPageBytes) == 0);
            mappings[va + (uint64_t)k * kSaPageBytes] = {handle, k};
        }
        return 0;
    }
    void unmap_chunk(uint64_t va, int pages) override {
        ++unmaps;
        CHECK(mappings.count(va) == 1);
        if (mappings.count(va) != 1) return;
        const uint64_t handle = mappings[va].first;
        CHECK(mappings[va].second == 0 && handles[handle].pages == pages); // exactly one whole mapping
        for (int k = 0; k < pages; ++k) {
            const uint64_t a = va + (uint64_t)k * kSaPageBytes;
            CHECK(mappings.count(a) == 1 && mappings[a].first == handle);
            mappings.erase(a);
            accessible.erase(a);
        }
    }
    int set_access(uint64_t va, size_t bytes) override {
        if (tick(fail_access_after)) return 1;
        for (uint64_t a = va; a < va + bytes; a += kSaPageBytes) {
            CHECK(mappings.count(a) == 1);
            accessible.insert(a);
        }
        return 0;
    }
    int true_side(uint64_t va) {
        auto& m = mappings[va];
        return side_of_phys(handles[m.first].phys + (size_t)m.second);
    }
    int probe_pages(const uint64_t* vas, int n, uint8_t* sides, void*) override {
        if (tick(fail_probe_after)) return 1;
        for (int i = 0; i < n; ++i) {
            CHECK(accessible.count(vas[i]) == 1);
            sides[i] = (uint8_t)true_side(vas[i]);
        }
        return 0;
    }
    void device_sync() override { ++syncs; }
    void order_after(void* earlier, void* later) override { CHECK(earlier != later); ++stream_syncs; }

    // pages of a live block: mapped, accessible, and on the side bit 21 of their address says
    int wrong_side_pages(uint64_t base, size_t bytes) {
        int wrong = 0;
        for (uint64_t a = base; a < base + bytes; a += kSaPageBytes) {
            CHECK(mappings.count(a) == 1);
            CHECK(accessible.count(a) == 1);
            if (mappings.count(a) != 1) { ++wrong; continue; }
            wrong += true_side(a) != (int)((a >> 21) & 1);
        }
        return wrong;
    }
};
int FakeDriver::default_model = 0;

static void test_alloc() {
    SaAllocConfig cfg;
    cfg.extra_alloc = 0; // exact page counts below: no headroom unless a case asks for it
    {   // basic: alignment, side placement, phase rule, reuse
        FakeDriver d;
        SaAllocator a(&d, false);
        uint64_t p1 = a.malloc(100u << 20, (void*)1, cfg);
        CHECK(p1 != 0 && p1 % kSaPageBytes == 0);
        CHECK(d.wrong_side_pages(p1, 100u << 20) == 0);
        uint64_t p2 = a.malloc((100u << 20) - 5, (void*)1, cfg); // same page-rounded size => same phase
        CHECK(p2 != 0 && ((p1 >> 21) & 1) == ((p2 >> 21) & 1));
        CHECK(a.phase_of_size(100u << 20) == (int)((p1 >> 21) & 1));
        CHECK(d.wrong_side_pages(p2, 100u << 20) == 0);
        CHECK(a.owns(p1) && !a.owns(p1 + kSaPageBytes));
        size_t mapped_before = d.mappings.size();
        CHECK(a.free(p1, (void*)1));
        CHECK(!a.free(p1, (void*)1));                 // double free is "not ours"
        CHECK(d.mappings.size() == mapped_before);     // free never unmaps
        uint64_t p3 = a.malloc(100u << 20, (void*)1, cfg);
        CHECK(p3 == p1);                               // exact-size reuse
        CHECK(d.stream_syncs == 0);
        a.free(p3, (void*)1);
        uint64_t p4 = a.malloc(100u << 20, (void*)2, cfg); // other stream => wait for the previous user
        CHECK(p4 == p1 && d.stream_syncs == 1);
        SaAllocStats st = a.stats();
        CHECK(st.reuse_hits == 2 && st.bytes_live == 2 * (100ull << 20) && st.bytes_cached == 0);
        a.free(p4, (void*)2);
        a.free(p2, (void*)1);
        size_t released = a.release_unused();
        CHECK(released == d.next_handle * 0 + released && d.mappings.empty() && d.handles.empty() && d.reservations.empty());
        CHECK(released >= 2 * (100ull << 20));
    }
    {   // one-page and odd-page blocks
        FakeDriver d;
        SaAllocator a(&d, false);
        for (size_t sz : {1ul, (size_t)kSaPageBytes, 3 * kSaPageBytes, 7 * kSaPageBytes + 1}) {
            uint64_t p = a.malloc(sz, nullptr, cfg);
            size_t bytes = (sz + kSaPageBytes - 1) / kSaPageBytes * kSaPageBytes;
            CHECK(p != 0 && d.wrong_side_pages(p, bytes) == 0);
        }
    }
    {   // fault injection: every k-th driver call of each kind fails once; state must stay consistent
        for (int kind = 0; kind < 5; ++kind)
            for (int k = 0; k < 40; k += 3) {
                FakeDriver d;
                SaAllocator a(&d, false);
                uint64_t warm = a.malloc(8u << 20, nullptr, cfg);
                CHECK(warm != 0);
                int* knob = kind == 0 ? &d.fail_create_after : kind == 1 ? &d.fail_map_after : kind == 2 ? &d.fail_reserve_after
                          : kind == 3 ? &d.fail_access_after : &d.fail_probe_after;
                *knob = k;
                uint64_t p = a.malloc(64u << 20, nullptr, cfg); // the ladder retries, so this normally still succeeds
                if (p) CHECK(d.wrong_side_pages(p, 64u << 20) >= 0);
                // conservation: every live handle is either mapped in a live/cached block or pooled
                SaAllocStats st = a.stats();
                size_t accounted = st.pages_pool[0] + st.pages_pool[1] + (st.bytes_live + st.bytes_cached) / kSaPageBytes;
                CHECK(accounted == d.live_pages());
                CHECK(d.mappings.size() == (st.bytes_live + st.bytes_cached) / kSaPageBytes);
                if (p) a.free(p, nullptr);
                a.free(warm, nullptr);
                a.release_unused();
                CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
            }
    }
    {   // growth headroom and free-time top-up (sideaware_prealloc_config)
        FakeDriver d;
        SaAllocator a(&d, false);
        SaAllocConfig c2 = cfg;
        c2.extra_required = 4;
        c2.extra_alloc = 12;
        uint64_t p1 = a.malloc(32u << 20, (void*)1, c2); // 16 pages asked for, 12 more mapped behind them
        CHECK(p1 != 0 && d.wrong_side_pages(p1, 32u << 20) == 0);
        SaAllocStats st = a.stats();
        CHECK(st.headroom_pages == 12 && st.bytes_cached == 12 * kSaPageBytes && st.bytes_live == (32u << 20));
        CHECK(d.wrong_side_pages(p1 + (32u << 20), 12 * kSaPageBytes) == 0); // the headroom is side-placed too
        const int creates = d.creates;
        uint64_t p2 = a.malloc(16u << 20, (void*)1, c2); // served from the headroom: no driver call
        CHECK(p2 == p1 + (32u << 20) && d.creates == creates && d.stream_syncs == 0);
        uint64_t p3 = a.malloc(8u << 20, (void*)2, c2);  // another stream: the headroom was never used, nothing to wait for
        CHECK(p3 != 0 && d.creates == creates && d.stream_syncs == 0);
        // 0 pages left at hand < extra_required: the next free tops up by extra_alloc
        st = a.stats();
        CHECK(st.bytes_cached == 0);
        const bool short_of_pages = st.pages_pool[0] + st.pages_pool[1] < 4; // pooled pages count as "at hand" too
        CHECK(a.top_up((void*)1, c2) == (short_of_pages ? 12u : 0u));
        CHECK(a.top_up((void*)1, c2) == 0); // once per shortage
        st = a.stats();
        if (short_of_pages) CHECK(st.top_ups == 1 && st.headroom_pages == 24 && st.bytes_cached == 12 * kSaPageBytes);
        size_t accounted = st.pages_pool[0] + st.pages_pool[1] + (st.bytes_live + st.bytes_cached) / kSaPageBytes;
        CHECK(accounted == d.live_pages());
        // with plenty at hand nothing is topped up
        uint64_t p4 = a.malloc(2u << 20, (void*)1, c2);
        CHECK(p4 != 0 && a.top_up((void*)1, c2) == 0);
        // switched off: growth maps exactly what is asked for
        SaAllocConfig off = cfg;
        off.extra_alloc = 0;
        const size_t mapped = d.mappings.size();
        uint64_t p5 = a.malloc(64u << 20, (void*)1, off);
        CHECK(p5 != 0 && d.mappings.size() <= mapped + 32 + 1); // at most one page skipped for the side
        for (uint64_t p : {p1, p2, p4, p5}) a.free(p, (void*)1);
        a.free(p3, (void*)2);
        a.release_unused();
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    {   // a top-up or a headroom that the driver refuses half-way leaves everything as it was
        for (int kind = 0; kind < 5; ++kind)
            for (int k = 0; k < 12; ++k) {
                FakeDriver d;
                SaAllocator a(&d, false);
                SaAllocConfig c2 = cfg;
                c2.extra_required = 64;
                c2.extra_alloc = 24;
                uint64_t p1 = a.malloc(8u << 20, nullptr, c2);
                CHECK(p1 != 0);
                SaAllocStats before = a.stats();
                const size_t mapped_before = d.mappings.size();
                int* knob = kind == 0 ? &d.fail_create_after : kind == 1 ? &d.fail_map_after : kind == 2 ? &d.fail_reserve_after
                          : kind == 3 ? &d.fail_access_after : &d.fail_probe_after;
                *knob = k;
                const size_t got = a.top_up(nullptr, c2);
                SaAllocStats after = a.stats();
                CHECK(got == 0 || got == 24);
                if (got == 0) {
                    CHECK(after.bytes_cached == before.bytes_cached && d.mappings.size() == mapped_before);
                } else {
                    CHECK(after.bytes_cached == before.bytes_cached + 24 * kSaPageBytes);
                }
                CHECK(after.bytes_live == before.bytes_live);
                size_t accounted = after.pages_pool[0] + after.pages_pool[1] + (after.bytes_live + after.bytes_cached) / kSaPageBytes;
                CHECK(accounted == d.live_pages());
                CHECK(d.mappings.size() == (after.bytes_live + after.bytes_cached) / kSaPageBytes);
                *knob = -1;
                // a request with headroom whose headroom part fails still gets its block
                *knob = k + 2;
                uint64_t p2 = a.malloc(48u << 20, nullptr, c2);
                *knob = -1;
                if (p2) CHECK(d.wrong_side_pages(p2, 48u << 20) == 0);
                after = a.stats();
                accounted = after.pages_pool[0] + after.pages_pool[1] + (after.bytes_live + after.bytes_cached) / kSaPageBytes;
                CHECK(accounted == d.live_pages());
                if (p2) a.free(p2, nullptr);
                a.free(p1, nullptr);
                a.release_unused();
                CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
            }
    }
    {   // mapping ahead of need: sideaware_prealloc
        FakeDriver d;
        SaAllocator a(&d, false);
        CHECK(a.prealloc(256u << 20, cfg));
        SaAllocStats st = a.stats();
        CHECK(st.bytes_live == 0 && st.bytes_cached >= (256u << 20) && st.large_allocs == 0);
        const int creates = d.creates;
        uint64_t p = a.malloc(200u << 20, (void*)3, cfg);
        CHECK(p != 0 && d.creates == creates && d.wrong_side_pages(p, 200u << 20) == 0); // found mapped
        CHECK(a.prealloc(16u << 20, cfg) && d.creates == creates);                    // already there: nothing to do
        a.free(p, (void*)3);
        a.release_unused();
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    {   // a block handed out on one stream and freed on another is ordered behind both when it is reused
        FakeDriver d;
        SaAllocator a(&d, false);
        SaAllocConfig off = cfg;
        off.extra_alloc = 0;
        uint64_t p = a.malloc(16u << 20, (void*)1, off);
        a.free(p, (void*)2);
        uint64_t q = a.malloc(16u << 20, (void*)1, off); // back on the stream it came from: still has to wait for stream 2
        CHECK(q == p && d.stream_syncs == 1);
        a.free(q, (void*)1);
        q = a.malloc(16u << 20, (void*)3, off);
        CHECK(q == p && d.stream_syncs == 2);             // only stream 1 used it this time
        a.free(q, (void*)4);
        q = a.malloc(16u << 20, (void*)5, off);
        CHECK(q == p && d.stream_syncs == 4);             // streams 3 and 4
        a.free(q, (void*)5);
        a.release_unused();
    }
    {   // out of memory: the ladder unmaps the cache, then gives up cleanly
        FakeDriver d;
        d.capacity_pages = 64;
        SaAllocator a(&d, false);
        uint64_t p = a.malloc(40 * kSaPageBytes, nullptr, cfg);
        CHECK(p != 0);
        a.free(p, nullptr);
        uint64_t q = a.malloc(48 * kSaPageBytes, nullptr, cfg); // needs the cached block's pages back
        CHECK(q != 0);
        CHECK(a.stats().bytes_cached == 0);
        uint64_t r = a.malloc(40 * kSaPageBytes, nullptr, cfg); // cannot fit
        CHECK(r == 0);
        CHECK(a.owns(q));
        CHECK(d.live_pages() <= 64);
        a.free(q, nullptr);
        uint64_t s = a.malloc(60 * kSaPageBytes, nullptr, cfg); // unbalanced pool: cross-side pages allowed, still correct
        CHECK(s != 0);
    }
    {   // thresholds nobody set scale with the device: 16 GiB and 2 GiB become a half and a quarter of its memory
        for (int user_set = 0; user_set < 2; ++user_set) {
            FakeDriver d;
            d.capacity_pages = 80 * 512; // 80 GiB
            SaAllocator a(&d, false, 80ull << 30);
            SaAllocConfig c2 = cfg;
            c2.extra_alloc = 0;
            if (user_set) c2.trim_scaled = false; // what sideaware_free_mapped_thresholds leaves behind
            std::vector<uint64_t> ps;
            for (int i = 0; i < 10; ++i) ps.push_back(a.malloc(2ull << 30, nullptr, c2));
            uint64_t keep = a.malloc(1ull << 30, nullptr, c2);
            for (uint64_t p : ps) a.free(p, nullptr);        // 20 GiB mapped and free: above 16 GiB, below 40 GiB
            uint64_t big = a.malloc(21ull << 30, nullptr, c2); // no run is large enough: the mapped set must grow
            CHECK(big != 0);
            SaAllocStats st = a.stats();
            if (user_set) CHECK(st.trims == 1 && st.bytes_cached <= (2ull << 30) + 16 * kSaPageBytes);
            else CHECK(st.trims == 0 && st.bytes_cached >= (19ull << 30));
            a.free(big, nullptr);
            a.free(keep, nullptr);
            a.release_unused();
            CHECK(d.live_pages() == 0);
        }
    }
    {   // free runs that lie across chunk borders can give back little: a miss then neither waits for the device nor trims
        FakeDriver d;
        SaAllocator a(&d, false);
        SaAllocConfig c2 = cfg;
        c2.extra_alloc = 0;
        c2.trim_start = 64u << 20;
        c2.trim_end = 16u << 20;
        uint64_t whole = a.malloc(100 * kSaPageBytes, nullptr, c2); // one growth: chunks of 7 + 1 pages in a row
        a.free(whole, nullptr);
        uint64_t shift = a.malloc(3 * kSaPageBytes, nullptr, c2);   // carved from it: every later block starts 3 pages into a chunk
        std::vector<uint64_t> ps;
        for (int i = 0; i < 12; ++i) ps.push_back(a.malloc(16u << 20, nullptr, c2));
        for (int i = 0; i < 12; i += 2) a.free(ps[i], nullptr); // six runs of 8 pages between live blocks
        const size_t cached_all = a.stats().bytes_cached;
        CHECK(cached_all >= (96ull << 20));
        const int syncs_before = d.syncs;
        uint64_t big = a.malloc(64u << 20, nullptr, c2); // over the threshold, but only a few whole chunks among the free pages
        CHECK(big != 0);
        if (d.model != 1) { // (model 1's irregular sides break the handles up into shorter chunks, which can be given back)
            CHECK(a.stats().trims == 0 && d.syncs == syncs_before);
            CHECK(a.stats().bytes_cached >= (96ull << 20));
        }
        a.free(big, nullptr);
        a.free(shift, nullptr);
        for (int i = 1; i < 12; i += 2) a.free(ps[i], nullptr);
        a.release_unused();
        CHECK(d.live_pages() == 0);
    }
    {   // threshold trimming: only when the mapped set must grow; least recently freed runs go first
        FakeDriver d;
        SaAllocator a(&d, false);
        SaAllocConfig c2 = cfg;
        c2.trim_start = 64u << 20;
        c2.trim_end = 16u << 20;
        std::vector<uint64_t> ps;
        for (int i = 0; i < 12; ++i) ps.push_back(a.malloc((size_t)(16 + 2 * i) << 20, nullptr, c2));
        for (int i = 0; i < 12; i += 2) a.free(ps[i], nullptr); // every other block: six separate runs of 16..36 MiB
        const size_t cached_all = a.stats().bytes_cached;
        CHECK(cached_all >= (156ull << 20) && cached_all <= (156ull << 20) + 12 * kSaPageBytes);
        int syncs_before = d.syncs;
        uint64_t small = a.malloc(4u << 20, nullptr, c2); // fits into a free run: no driver call, no trim
        CHECK(small != 0 && a.stats().trims == 0 && d.syncs == syncs_before);
        CHECK(a.stats().bytes_cached == cached_all - (4u << 20));
        uint64_t big = a.malloc(64u << 20, nullptr, c2);  // no run is large enough -> trim, then grow
        CHECK(big != 0);
        SaAllocStats st = a.stats();
        // whole chunks inside the free runs are unmapped; pages of chunks shared with live neighbours stay (up to 6 at either end of a run)
        CHECK(st.trims == 1 && d.syncs >= syncs_before + 2);
        CHECK(st.bytes_cached <= (16u << 20) + 6 * 12 * kSaPageBytes && st.bytes_cached < cached_all / 2);
        CHECK(st.pages_pool[0] + st.pages_pool[1] + (st.bytes_live + st.bytes_cached) / kSaPageBytes == d.live_pages());
        CHECK(d.wrong_side_pages(big, 64u << 20) == 0 && d.wrong_side_pages(small, 4u << 20) == 0);
        a.free(small, nullptr);
        a.free(big, nullptr);
        for (int i = 1; i < 12; i += 2) a.free(ps[i], nullptr);
        a.release_unused();
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    {   // runs: split on allocation, merge on free, one skipped page when the run starts on the wrong side
        FakeDriver d;
        SaAllocator a(&d, false);
        uint64_t seg = a.malloc(64 * kSaPageBytes, nullptr, cfg);
        CHECK(seg != 0);
        a.free(seg, nullptr);
        CHECK(a.stats().free_runs == 1 && a.stats().segments == 1);
        size_t maps_before = d.mappings.size();
        uint64_t x = a.malloc(10 * kSaPageBytes, nullptr, cfg);
        uint64_t y = a.malloc(20 * kSaPageBytes, nullptr, cfg);
        uint64_t z = a.malloc(10 * kSaPageBytes, nullptr, cfg);
        CHECK(x && y && z && d.mappings.size() == maps_before); // all carved out of the mapped segment
        CHECK(((x >> 21) & 1) == ((z >> 21) & 1));              // same size, same start side
        for (uint64_t p : {x, y, z}) CHECK(p >= seg && p < seg + 64 * kSaPageBytes);
        CHECK(d.wrong_side_pages(x, 10 * kSaPageBytes) == 0 && d.wrong_side_pages(y, 20 * kSaPageBytes) == 0);
        CHECK(!(x < y + 20 * kSaPageBytes && y < x + 10 * kSaPageBytes));
        a.free(y, nullptr);
        a.free(x, nullptr);
        a.free(z, nullptr);
        SaAllocStats st = a.stats();
        CHECK(st.free_runs == 1 && st.bytes_cached == 64 * kSaPageBytes && st.bytes_live == 0); // merged back
        uint64_t again = a.malloc(64 * kSaPageBytes, nullptr, cfg);
        CHECK(again == seg);
        a.free(again, nullptr);
        // an odd-sized block forces the next equal-sized one onto a run that starts on the other side
        uint64_t o1 = a.malloc(3 * kSaPageBytes, nullptr, cfg);
        uint64_t o2 = a.malloc(3 * kSaPageBytes, nullptr, cfg);
        CHECK(o1 && o2 && ((o1 >> 21) & 1) == ((o2 >> 21) & 1));
        CHECK(d.wrong_side_pages(o1, 3 * kSaPageBytes) == 0 && d.wrong_side_pages(o2, 3 * kSaPageBytes) == 0);
        CHECK(d.mappings.size() == maps_before);
    }
    {   // streams: a run last used on another stream is waited for; merged runs of several streams sync the device
        FakeDriver d;
        SaAllocator a(&d, false);
        uint64_t p1 = a.malloc(8 * kSaPageBytes, (void*)1, cfg);
        uint64_t p2 = a.malloc(8 * kSaPageBytes, (void*)2, cfg);
        a.free(p1, (void*)1);
        uint64_t q = a.malloc(8 * kSaPageBytes, (void*)1, cfg);
        CHECK(q == p1 && d.stream_syncs == 0 && d.syncs == 0);
        a.free(q, (void*)1);
        q = a.malloc(8 * kSaPageBytes, (void*)3, cfg);
        CHECK(q == p1 && d.stream_syncs == 1);
        a.free(q, (void*)3);
        a.free(p2, (void*)2);
        (void)p2;
    }
    {   // free runs last used on different streams stay apart; a request prefers a run of its own stream
        FakeDriver d;
        SaAllocator a(&d, false);
        uint64_t p1 = a.malloc(8 * kSaPageBytes, (void*)1, cfg);
        uint64_t p2 = a.malloc(8 * kSaPageBytes, (void*)2, cfg);
        CHECK(p1 && p2 && d.reservations.size() == 1 && p2 == p1 + 8 * kSaPageBytes); // side by side in one segment
        a.free(p1, (void*)1);
        a.free(p2, (void*)2);
        CHECK(a.stats().free_runs == 2);                     // not merged: two streams
        uint64_t q = a.malloc(8 * kSaPageBytes, (void*)2, cfg);
        CHECK(q == p2 && d.stream_syncs == 0 && d.syncs == 0); // its own stream's run, although p1's comes first
        a.free(q, (void*)2);
        a.trim(1, 0);                                          // a device-wide wait makes every run anybody's
        CHECK(a.stats().bytes_cached == 0 && d.syncs >= 1);
        uint64_t r = a.malloc(16 * kSaPageBytes, (void*)3, cfg);
        CHECK(r != 0 && d.stream_syncs == 0);
        a.free(r, (void*)3);
        uint64_t s1 = a.malloc(8 * kSaPageBytes, (void*)3, cfg), s2 = a.malloc(8 * kSaPageBytes, (void*)3, cfg);
        a.free(s1, (void*)3);
        a.free(s2, (void*)3);
        CHECK(a.stats().free_runs == 1);                     // same stream: merged
        a.release_unused();
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    {   // trimming a run in the middle of a segment leaves the rest usable; the range is released with the last page
        FakeDriver d;
        SaAllocator a(&d, false);
        uint64_t seg = a.malloc(50 * kSaPageBytes, nullptr, cfg);
        a.free(seg, nullptr);
        uint64_t x = a.malloc(10 * kSaPageBytes, nullptr, cfg);
        uint64_t y = a.malloc(30 * kSaPageBytes, nullptr, cfg);
        uint64_t z = a.malloc(10 * kSaPageBytes, nullptr, cfg);
        CHECK(x && y && z && d.reservations.size() == 1);
        a.free(y, nullptr);
        a.trim(0, 0); // unmaps the chunks that lie wholly inside y; pages of chunks shared with x or z stay mapped (and cached)
        SaAllocStats st = a.stats();
        CHECK(st.bytes_cached <= 12 * kSaPageBytes && d.reservations.size() == 1); // at most 6 pages of a 7-page chunk at either end
        CHECK(d.mappings.size() == 20 + st.bytes_cached / kSaPageBytes);
        CHECK(st.pages_pool[0] + st.pages_pool[1] + d.mappings.size() == d.live_pages());
        CHECK(d.wrong_side_pages(x, 10 * kSaPageBytes) == 0 && d.wrong_side_pages(z, 10 * kSaPageBytes) == 0);
        uint64_t w = a.malloc(30 * kSaPageBytes, nullptr, cfg); // into the hole if it is long enough, else behind z; never a new address range
        CHECK(w != 0 && d.wrong_side_pages(w, 30 * kSaPageBytes) == 0 && d.reservations.size() == 1);
        CHECK(d.wrong_side_pages(x, 10 * kSaPageBytes) == 0 && d.wrong_side_pages(z, 10 * kSaPageBytes) == 0);
        a.free(x, nullptr);
        a.free(z, nullptr);
        a.free(w, nullptr);
        size_t released = a.release_unused();
        CHECK(released >= 50 * kSaPageBytes);
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    {   // a request larger than the free run at the end of a segment extends the segment by the missing pages only
        FakeDriver d;
        SaAllocator a(&d, false);
        uint64_t p = a.malloc(20 * kSaPageBytes, nullptr, cfg);
        CHECK(p != 0);
        a.free(p, nullptr);
        const size_t live_before = d.live_pages();
        uint64_t q = a.malloc(30 * kSaPageBytes, nullptr, cfg);
        SaAllocStats st = a.stats();
        CHECK(q != 0 && d.wrong_side_pages(q, 30 * kSaPageBytes) == 0);
        CHECK(st.extensions == 1 && st.segments == 1 && d.reservations.size() == 1);
        CHECK(q == p || q == p + kSaPageBytes);                       // the old run, or the old run less a skipped page
        CHECK(d.live_pages() <= live_before + 11 + 8);                 // about 10 new pages, not 30
        CHECK(st.bytes_live == 30 * kSaPageBytes);
        CHECK(st.pages_pool[0] + st.pages_pool[1] + (st.bytes_live + st.bytes_cached) / kSaPageBytes == d.live_pages());
        a.free(q, nullptr);
        CHECK(a.stats().free_runs == 1);                               // one run again, longer now
        {   // a trimmed tail gives its slots back: the segment can grow into them again, from the pool
            uint64_t keep = a.malloc(8 * kSaPageBytes, nullptr, cfg);  // front of the run stays live
            CHECK(keep != 0);
            a.trim(0, 0);                                              // the rest of the run is unmapped (whole chunks only)
            const int creates_before = d.creates;
            uint64_t big = a.malloc(40 * kSaPageBytes, nullptr, cfg);
            CHECK(big != 0 && d.wrong_side_pages(big, 40 * kSaPageBytes) == 0);
            if (d.model != 1) CHECK(d.creates - creates_before <= 12); // mostly pooled chunks
            a.free(big, nullptr);
            a.free(keep, nullptr);
        }
        const uint64_t ext_before = a.stats().extensions;
        uint64_t r = a.malloc(5000 * kSaPageBytes, nullptr, cfg);     // beyond the reserved room: a new segment
        CHECK(r != 0 && a.stats().segments == 2 && a.stats().extensions == ext_before);
        a.free(r, nullptr);
        a.release_unused();
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    {   // fault injection on the extension path: the old run must survive a failed extension
        for (int kind = 0; kind < 5; ++kind)
            for (int k = 0; k < 12; k += 1) {
                FakeDriver d;
                SaAllocator a(&d, false);
                uint64_t p = a.malloc(16 * kSaPageBytes, nullptr, cfg);
                a.free(p, nullptr);
                int* knob = kind == 0 ? &d.fail_create_after : kind == 1 ? &d.fail_map_after : kind == 2 ? &d.fail_reserve_after
                          : kind == 3 ? &d.fail_access_after : &d.fail_probe_after;
                *knob = k;
                uint64_t q = a.malloc(40 * kSaPageBytes, nullptr, cfg);
                if (q) CHECK(d.wrong_side_pages(q, 40 * kSaPageBytes) >= 0);
                SaAllocStats st = a.stats();
                CHECK(st.pages_pool[0] + st.pages_pool[1] + (st.bytes_live + st.bytes_cached) / kSaPageBytes == d.live_pages());
                CHECK(d.mappings.size() == (st.bytes_live + st.bytes_cached) / kSaPageBytes);
                if (q) a.free(q, nullptr);
                uint64_t again = a.malloc(16 * kSaPageBytes, nullptr, cfg); // still served without the driver's help or with it, but correctly
                CHECK(again != 0 && d.wrong_side_pages(again, 16 * kSaPageBytes) == 0);
                a.free(again, nullptr);
                a.release_unused();
                CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
            }
    }
    {   // a hole that a trim left inside a segment is used again, from the pool, without new address space
        FakeDriver d;
        SaAllocator a(&d, false);
        uint64_t x = a.malloc(10 * kSaPageBytes, nullptr, cfg);
        uint64_t y = a.malloc(60 * kSaPageBytes, nullptr, cfg);
        uint64_t z = a.malloc(10 * kSaPageBytes, nullptr, cfg);
        CHECK(x && y && z && d.reservations.size() == 1);
        a.free(y, nullptr);
        a.trim(0, 0);
        const size_t mapped_after_trim = d.mappings.size();
        CHECK(mapped_after_trim < 80 && mapped_after_trim >= 20);
        const int creates_before = d.creates;
        uint64_t w = a.malloc(30 * kSaPageBytes, nullptr, cfg);
        SaAllocStats st = a.stats();
        CHECK(w != 0 && w > x && w < z && d.wrong_side_pages(w, 30 * kSaPageBytes) == 0); // between its old neighbours
        CHECK(st.hole_refills == 1 && d.reservations.size() == 1);
        if (d.model != 1) CHECK(d.creates - creates_before <= 4);                          // from the pool
        CHECK(st.pages_pool[0] + st.pages_pool[1] + (st.bytes_live + st.bytes_cached) / kSaPageBytes == d.live_pages());
        CHECK(d.mappings.size() == (st.bytes_live + st.bytes_cached) / kSaPageBytes);
        a.free(w, nullptr);
        a.free(x, nullptr);
        a.free(z, nullptr);
        a.release_unused();
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    {   // skewed physical side distribution still yields correctly placed blocks
        FakeDriver d;
        d.bias_percent = 80;
        SaAllocator a(&d, false);
        uint64_t p = a.malloc(256u << 20, nullptr, cfg);
        CHECK(p != 0 && d.wrong_side_pages(p, 256u << 20) == 0);
    }
    {   // compression keeps separate pools and cache keys
        FakeDriver d;
        SaAllocator a(&d, true);
        SaAllocConfig c2 = cfg;
        uint64_t p = a.malloc(8u << 20, nullptr, c2);
        a.free(p, nullptr);
        c2.compression = true;
        uint64_t q = a.malloc(8u << 20, nullptr, c2);
        CHECK(q != 0 && q != p);
    }
    {   // long random churn: blocks never overlap, sit on the right sides, pages are conserved
        FakeDriver d;
        SaAllocator a(&d, false);
        SaAllocConfig c2 = cfg;
        c2.trim_start = 512u << 20;
        c2.trim_end = 64u << 20;
        std::mt19937 rng(3);
        std::vector<std::pair<uint64_t, size_t>> live;
        std::map<size_t, int> phase_seen;
        for (int i = 0; i < 4000; ++i) {
            if (live.empty() || (rng() % 100) < 55) {
                size_t sz = ((size_t)(1 + rng() % 64) << 20) - (rng() % 3);
                uint64_t p = a.malloc(sz, (void*)(uintptr_t)(rng() % 3), c2);
                CHECK(p != 0 && p % kSaPageBytes == 0);
                size_t bytes = (sz + kSaPageBytes - 1) / kSaPageBytes * kSaPageBytes;
                for (auto& l : live) CHECK(!(p < l.first + l.second && l.first < p + bytes));
                if (i % 7 == 0) CHECK(d.wrong_side_pages(p, bytes) == 0);
                int ph = (int)((p >> 21) & 1);
                size_t same = 0;
                for (auto& l : live) same += l.second == bytes;
                if (same && phase_seen.count(bytes)) CHECK(phase_seen[bytes] == ph); // same side as the live blocks of that size
                phase_seen[bytes] = ph;
                live.push_back({p, bytes});
            } else {
                size_t k = rng() % live.size();
                CHECK(a.free(live[k].first, nullptr));
                live.erase(live.begin() + k);
            }
            if (i % 500 == 499) {
                SaAllocStats st = a.stats();
                size_t live_bytes = 0;
                for (auto& l : live) live_bytes += l.second;
                CHECK(st.bytes_live == live_bytes);
                CHECK(st.pages_pool[0] + st.pages_pool[1] + (st.bytes_live + st.bytes_cached) / kSaPageBytes == d.live_pages());
                CHECK(d.mappings.size() == (st.bytes_live + st.bytes_cached) / kSaPageBytes);
            }
        }
        SaAllocStats st = a.stats();
        CHECK(st.cross_side_pages == 0);
        std::printf("alloc churn: %llu allocs, %llu served from mapped runs, %llu pages created, %llu trims, %llu segments, %llu free runs\n",
                    (unsigned long long)st.large_allocs, (unsigned long long)st.reuse_hits, (unsigned long long)st.pages_created,
                    (unsigned long long)st.trims, (unsigned long long)st.segments, (unsigned long long)st.free_runs);
        for (auto& l : live) a.free(l.first, nullptr);
        a.release_unused();
        if (!(d.mappings.empty() && d.handles.empty() && d.reservations.empty())) {
            SaAllocStats e = a.stats();
            std::printf("left: %zu mappings, %zu handles, %zu reservations; cached %llu live %llu pool %llu+%llu runs %llu\n", d.mappings.size(), d.handles.size(),
                        d.reservations.size(), (unsigned long long)e.bytes_cached, (unsigned long long)e.bytes_live, (unsigned long long)e.pages_pool[0], (unsigned long long)e.pages_pool[1], (unsigned long long)e.free_runs);
        }
        CHECK(d.mappings.empty() && d.handles.empty() && d.reservations.empty());
    }
    std::printf("alloc: done\n");
}

// How many driver calls growth needs under each model of the physical layout.
static void test_alloc_chunks() {
    SaAllocConfig cfg;
    cfg.extra_alloc = 0; // exact handle counts below
    const size_t pages = 512; // 1 GiB
    for (int model = 0; model < 3; ++model) {
        FakeDriver d;
        d.model = model;
        if (model == 2) d.next_phys = 3;
        SaAllocator a(&d, false);
        uint64_t p = a.malloc(pages * kSaPageBytes, nullptr, cfg);
        CHECK(p != 0 && d.wrong_side_pages(p, pages * kSaPageBytes) == 0);
        SaAllocStats st = a.stats();
        std::printf("alloc chunks: model %d: %zu pages with %d creates, %d maps, %d unmaps, %llu discarded, %llu pooled pages\n", model, pages,
                    d.creates, d.maps, d.unmaps, (unsigned long long)st.handles_discarded,
                    (unsigned long long)(st.pages_pool[0] + st.pages_pool[1]));
        CHECK(st.pages_pool[0] + st.pages_pool[1] + pages == d.live_pages());
        if (model != 1) {
            CHECK(d.creates <= (int)pages / 3);          // two handles per group of 8 pages, plus what prediction misses cost
            CHECK(d.maps <= (int)pages / 2);
            CHECK(st.pages_pool[0] + st.pages_pool[1] <= 16);
        } else {
            CHECK(d.creates <= (int)pages * 3);           // single pages in the end, as before
        }
        // a second block of the same size reuses nothing and must be as cheap
        const int creates_before = d.creates;
        uint64_t q = a.malloc(pages * kSaPageBytes, nullptr, cfg);
        CHECK(q != 0 && d.wrong_side_pages(q, pages * kSaPageBytes) == 0);
        if (model != 1) CHECK(d.creates - creates_before <= (int)pages / 3);
        // small and odd sizes
        for (size_t n : {1, 2, 3, 5, 7, 8, 9, 15, 16, 17, 33}) {
            uint64_t r = a.malloc(n * kSaPageBytes, nullptr, cfg);
            CHECK(r != 0 && d.wrong_side_pages(r, n * kSaPageBytes) == 0);
        }
        a.free(p, nullptr);
        a.free(q, nullptr);
        // the freed gigabytes come back as chunks from the pool: no create at all
        a.trim(0, 0);
        const int creates_mid = d.creates;
        uint64_t r = a.malloc(pages * kSaPageBytes, nullptr, cfg);
        CHECK(r != 0 && d.wrong_side_pages(r, pages * kSaPageBytes) == 0);
        if (model != 1) CHECK(d.creates - creates_mid <= 8);
        std::printf("alloc chunks: model %d: re-mapping 512 pooled pages took %d creates\n", model, d.creates - creates_mid);
    }
    // many small blocks (4..12 pages each): handles per page must stay well below one
    for (int model = 0; model < 3; model += 2) {
        FakeDriver d;
        d.model = model;
        if (model == 2) d.next_phys = 3;
        SaAllocator a(&d, false);
        std::mt19937 rng(11);
        size_t total = 0;
        for (int i = 0; i < 300; ++i) {
            size_t n = 4 + rng() % 9;
            uint64_t r = a.malloc(n * kSaPageBytes, nullptr, cfg);
            CHECK(r != 0 && d.wrong_side_pages(r, n * kSaPageBytes) == 0);
            total += n;
        }
        SaAllocStats st = a.stats();
        std::printf("alloc chunks: model %d: 300 small blocks, %zu pages: %d creates, %d maps, %d unmaps, %llu discarded, %llu pooled pages\n",
                    model, total, d.creates, d.maps, d.unmaps, (unsigned long long)st.handles_discarded,
                    (unsigned long long)(st.pages_pool[0] + st.pages_pool[1]));
        CHECK(d.creates <= (int)total / 2);
        CHECK(st.pages_pool[0] + st.pages_pool[1] <= total / 16); // odd-sized blocks of one start side leave a surplus of the other side
    }
    std::printf("alloc chunks: done\n");
}

// ---------------------------------------------------------------------------
// topology analysis on synthetic latencies
// ---------------------------------------------------------------------------
static std::vector<uint32_t> offsets64() {
    std::vector<uint32_t> off{0};
    for (int b = 4; b <= 20; ++b) off.push_back(1u << b);
    std::mt19937 rng(99);
    while (off.size() < 64) {
        uint32_t o = rng() & 0x1FFFF0u;
        if (o && (o & (o - 1))) off.push_back(o);
    }
    return off;
}

static void topo_case(uint32_t true_hash, int num_sms, int noise, int far_extra, bool sm0_far_from_addr0, bool expect_usable) {
    std::vector<uint32_t> off = offsets64();
    std::mt19937 rng(num_sms * 31 + noise);
    std::vector<int> sm_side(num_sms);
    for (int i = 0; i < num_sms; ++i) sm_side[i] = (i == 0) ? 0 : (int)(rng() & 1);
    std::vector<uint32_t> lat((size_t)num_sms * off.size());
    std::vector<int> smid(num_sms);
    for (int i = 0; i < num_sms; ++i) {
        smid[i] = i;
        uint32_t base = 5000 + (rng() % 1500); // SMs differ in their distance to L2
        for (size_t j = 0; j < off.size(); ++j) {
            int addr_side = (int)sa_parity32(off[j] & true_hash) ^ (sm0_far_from_addr0 ? 1 : 0);
            bool far = addr_side != sm_side[i];
            lat[i * off.size() + j] = base + (far ? far_extra : 0) + (noise ? rng() % noise : 0);
        }
    }
    SaTopology t;
    t.num_sms = num_sms;
    t.max_smid = num_sms - 1;
    sa_analyse_latency_matrix(lat, num_sms, smid, off, &t);
    if (expect_usable) {
        CHECK(t.hash == true_hash);
        CHECK(t.hash_usable);
        CHECK(t.validation_errors == 0);
        int c[2] = {0, 0};
        bool sides_ok = true;
        for (int i = 0; i < num_sms; ++i) {
            sides_ok = sides_ok && (t.side_index[i] & 1) == sm_side[i];
            CHECK((t.side_index[i] >> 1) == c[sm_side[i]]); // ordinals count up per side
            c[sm_side[i]]++;
        }
        CHECK(sides_ok);
        CHECK(t.count[0] == c[0] && t.count[1] == c[1] && t.min_per_side == std::min(c[0], c[1]));
        CHECK(t.confidence > 0.9);
        CHECK(!t.json.empty());
    } else {
        CHECK(!t.hash_usable);
    }
}

static void test_topology() {
    topo_case(0x1EF000u, 148, 300, 3000, false, true);  // the mask the reference's author saw on a Blackwell part
    topo_case(0x1EF000u, 148, 300, 3000, true, true);
    topo_case(0xB3000u, 132, 800, 2500, false, true);   // Hopper-like
    topo_case(0xAB000u, 132, 100, 1200, true, true);
    topo_case(0x1000u, 8, 50, 2000, false, true);
    topo_case(0x1EF000u, 148, 300, 0, false, false);    // no near/far difference at all: must refuse
    topo_case(0x1EE000u, 148, 300, 3000, false, false); // 8 KiB granularity: chunk pairing would not hold
    topo_case(0x1EF800u, 148, 300, 3000, false, false); // side flips inside a 4 KiB chunk
    {   // topology cache: a file is believed only if it is complete, consistent and written for this very GPU and driver
        SaTopology t;
        t.num_sms = 148;
        t.max_smid = 147;
        t.hash = 0x1EF000u;
        t.hash_usable = true;
        t.validation_offsets = 46;
        t.confidence = 0.987654;
        int ord[2] = {0, 0};
        for (int sm = 0; sm < 148; ++sm) {
            const int side = (sm / 2) % 2 == 0 ? 0 : 1;
            t.side_index[sm] = (uint8_t)(side | (ord[side]++ << 1));
            t.thr[sm] = 500 + sm;
            t.near_lat[sm] = 330 + sm % 7;
            t.far_lat[sm] = 760 + sm % 5;
        }
        t.count[0] = ord[0];
        t.count[1] = ord[1];
        t.min_per_side = std::min(ord[0], ord[1]);
        const std::string uuid = "00112233445566778899aabbccddeeff";
        const std::string text = sa_topology_serialize(t, uuid, 12090);
        SaTopology back;
        std::string why;
        CHECK(sa_topology_parse(text, uuid, 12090, 148, &back, &why));
        CHECK(back.hash == t.hash && back.hash_usable && back.count[0] == t.count[0] && back.count[1] == t.count[1]);
        CHECK(std::memcmp(back.side_index, t.side_index, SA_MAX_SM) == 0 && std::memcmp(back.thr, t.thr, sizeof(t.thr)) == 0);
        CHECK(std::memcmp(back.near_lat, t.near_lat, sizeof(t.near_lat)) == 0 && std::memcmp(back.far_lat, t.far_lat, sizeof(t.far_lat)) == 0);
        CHECK(std::fabs(back.confidence - t.confidence) < 1e-6 && back.max_smid == 147);
        CHECK(!sa_topology_parse(text, "ffffffffffffffffffffffffffffffff", 12090, 148, &back, &why) && why.find("another GPU") != std::string::npos);
        CHECK(!sa_topology_parse(text, uuid, 12080, 148, &back, &why) && why.find("driver") != std::string::npos);
        CHECK(!sa_topology_parse(text, uuid, 12090, 132, &back, &why) && why.find("SM count") != std::string::npos);
        CHECK(!sa_topology_parse(text.substr(0, text.size() / 2), uuid, 12090, 148, &back, &why));       // truncated
        CHECK(!sa_topology_parse("", uuid, 12090, 148, &back, &why));
        CHECK(!sa_topology_parse("something else entirely\n", uuid, 12090, 148, &back, &why));
        std::string edited = text;
        const size_t at = edited.find("sm 17 ");
        CHECK(at != std::string::npos);
        edited[at + 6] = edited[at + 6] == '1' ? '0' : '1';                                             // one SM moved to the other side
        CHECK(!sa_topology_parse(edited, uuid, 12090, 148, &back, &why) && why.find("checksum") != std::string::npos);
        std::string other_hash = text;
        const size_t h = other_hash.find("hash 2027520");
        CHECK(h != std::string::npos);
        other_hash.replace(h, 12, "hash 2023424"); // 0x1EE000: 8 KiB granularity
        CHECK(!sa_topology_parse(other_hash, uuid, 12090, 148, &back, &why));
        SaTopology broken = t;
        broken.count[0] += 1; // counts that do not add up, with a checksum that is right
        CHECK(!sa_topology_parse(sa_topology_serialize(broken, uuid, 12090), uuid, 12090, 148, &back, &why) && why.find("add up") != std::string::npos);
        broken = t;
        broken.hash = 0x1EE000u; // marked usable but side would not flip every 4 KiB
        CHECK(!sa_topology_parse(sa_topology_serialize(broken, uuid, 12090), uuid, 12090, 148, &back, &why) && why.find("required form") != std::string::npos);
    }
    std::printf("topology: done\n");
}

// ---------------------------------------------------------------------------
// stage ring of the bulk-copy kernels (sa_bulk.cuh): replay what lane 0 of a warp does in
// sa_memcpy_bulk_kernel against a model of the mbarriers, with chosen loads never arriving.
// No GPU run can or should force a wait to run out, so the state after one is checked here.
// ---------------------------------------------------------------------------
struct ModelBarrier {
    uint32_t completed = 0;   // phases completed so far
    bool armed = false;       // a load is outstanding on the current phase
    bool will_arrive = false; // ... and the model lets it arrive
};

static void ring_case(uint32_t S, uint32_t in_flight, uint32_t chunks, const std::set<uint32_t>& never_arrive) {
    SaStageRing r;
    sa_ring_reset(r);
    std::vector<ModelBarrier> bar(S);
    std::vector<uint32_t> chunk_of_stage(S, 0xffffffffu);
    std::vector<int> stored(chunks, 0), plain(chunks, 0);
    uint32_t rearmed_incomplete = 0, waits_after_failure_that_arrived = 0, errors = 0;
    auto retire = [&]() {
        const uint32_t st = sa_ring_oldest(r, S);
        ModelBarrier& b = bar[st];
        CHECK(b.armed);
        // mbarrier.try_wait.parity succeeds when the phase with that parity has completed
        const uint32_t parity = sa_ring_oldest_parity(r, S);
        if (b.will_arrive) { b.completed++; b.armed = false; }
        const bool arrived = !b.armed && ((b.completed - 1) & 1u) == parity;
        if (arrived) {
            stored[chunk_of_stage[st]]++;
            if (r.failed) ++waits_after_failure_that_arrived;
        } else {
            ++errors;
        }
        sa_ring_retire(r, S, arrived);
    };
    for (uint32_t c = 0; c < chunks; ++c) {
        if (sa_ring_may_issue(r)) {
            const uint32_t st = sa_ring_issue(r, S);
            if (bar[st].armed) ++rearmed_incomplete; // arming a barrier whose phase never completed
            bar[st].armed = true;
            bar[st].will_arrive = never_arrive.count(c) == 0;
            chunk_of_stage[st] = c;
            while (sa_ring_in_flight(r) > in_flight) retire();
        } else {
            plain[c]++; // the warp has given up on bulk copies
        }
    }
    while (sa_ring_in_flight(r) > 0) retire();
    for (uint32_t st = 0; st < S; ++st)
        if ((r.lost >> st) & 1u) plain[chunk_of_stage[st]]++;
    CHECK(rearmed_incomplete == 0);
    CHECK(r.retired == r.issued);
    CHECK((r.failed != 0) == (errors != 0));
    bool once = true;
    for (uint32_t c = 0; c < chunks; ++c) once = once && stored[c] + plain[c] == 1;
    CHECK(once);
    // nothing that never arrived was stored from shared memory
    for (uint32_t c : never_arrive)
        if (c < chunks) CHECK(stored[c] == 0);
    if (never_arrive.empty()) {
        CHECK(r.failed == 0 && r.lost == 0);
        for (uint32_t c = 0; c < chunks; ++c) CHECK(stored[c] == 1);
    } else if (*never_arrive.begin() < chunks) {
        // the loads that were in flight behind the first lost one each got one more wait
        const uint32_t first = *never_arrive.begin();
        uint32_t expect_late = 0;
        for (uint32_t c = first + 1; c < chunks && c <= first + in_flight; ++c) expect_late += never_arrive.count(c) == 0;
        CHECK(waits_after_failure_that_arrived == expect_late);
        // and nothing was issued after the failure was seen
        CHECK(r.issued <= first + in_flight + 1);
    }
}

static void test_ring() {
    for (uint32_t S : {2u, 3u, 4u, 6u})
        for (uint32_t L = 1; L + 1 < S || L == 1; ++L) {
            if (L >= S) break;
            for (uint32_t chunks : {0u, 1u, 2u, 5u, 64u, 1001u}) {
                ring_case(S, L, chunks, {});
                ring_case(S, L, chunks, {0});
                ring_case(S, L, chunks, {3});
                ring_case(S, L, chunks, {3, 4});
                ring_case(S, L, chunks, {3, 5, 40});
                ring_case(S, L, chunks, {chunks ? chunks - 1 : 0});
            }
        }
    std::printf("ring: done\n");
}

int main(int argc, char** argv) {
    std::string what = argc > 1 ? argv[1] : "all";
    if (what == "sched" || what == "all") test_sched();
    if (what == "alloc" || what == "all") {
        for (int m = 0; m < 3; ++m) {
            FakeDriver::default_model = m;
            std::printf("alloc: simulated driver, physical side model %d\n", m);
            test_alloc();
        }
        FakeDriver::default_model = 0;
    }
    if (what == "chunks" || what == "all") test_alloc_chunks();
    if (what == "topology" || what == "all") test_topology();
    if (what == "ring" || what == "all") test_ring();
    if (g_failures) {
        std::printf("%d CHECK(s) failed\n", g_failures);
        return 1;
    }
    std::printf("OK\n");
    return 0;
}
