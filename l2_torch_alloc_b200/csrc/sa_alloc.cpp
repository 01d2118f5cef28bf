#include "sa_alloc.hpp"

#include <algorithm>
#include <cstdio>

static inline size_t round_to_pages(size_t size) {
    if (size == 0) size = 1;
    return (size + kSaPageBytes - 1) / kSaPageBytes * kSaPageBytes;
}

static inline int side_bit(uint64_t va) { return (int)((va >> kSaSideBit) & 1); }

SaAllocator::~SaAllocator() {
    // Process teardown: the driver reclaims everything; touching it here could run
    // after the CUDA context is gone.
}

// ---------------------------------------------------------------------------
// physical pages
// ---------------------------------------------------------------------------

void SaAllocator::release_pools() {
    for (int c = 0; c < 2; ++c)
        for (int s = 0; s < 2; ++s) {
            for (auto& pg : pool_[c][s]) be_->release_page(pg.handle);
            pool_[c][s].clear();
        }
}

// ---------------------------------------------------------------------------
// free runs
// ---------------------------------------------------------------------------

void SaAllocator::erase_free(std::map<uint64_t, Run>::iterator it) {
    auto range = free_by_len_[it->second.seg->compressed].equal_range(it->second.pages);
    for (auto j = range.first; j != range.second; ++j)
        if (j->second == it->first) { free_by_len_[it->second.seg->compressed].erase(j); break; }
    cached_bytes_ -= it->second.pages * kSaPageBytes;
    free_.erase(it);
}

// Adds a free run and merges it with free neighbours of the same segment.
void SaAllocator::insert_free(uint64_t va, Run run) {
    auto merge = [](Run& into, const Run& other) {
        into.pages += other.pages;
        into.freed_seq = std::max(into.freed_seq, other.freed_seq);
        if (other.mixed || other.stream != into.stream) into.mixed = true;
    };
    auto next = free_.lower_bound(va);
    if (next != free_.end() && next->second.seg == run.seg && va + run.pages * kSaPageBytes == next->first) {
        Run n = next->second;
        erase_free(next);
        merge(run, n);
    }
    auto prev = free_.lower_bound(va);
    if (prev != free_.begin()) {
        --prev;
        if (prev->second.seg == run.seg && prev->first + prev->second.pages * kSaPageBytes == va) {
            Run p = prev->second;
            uint64_t pva = prev->first;
            erase_free(prev);
            merge(p, run);
            run = p;
            va = pva;
        }
    }
    free_.emplace(va, run);
    free_by_len_[run.seg->compressed].emplace(run.pages, va);
    cached_bytes_ += run.pages * kSaPageBytes;
}

// Best fit: the shortest free run that can hold `pages` pages starting on side `phase`
// (a run that starts on the other side needs one page more; that page stays free).
uint64_t SaAllocator::take_from_free(size_t pages, int phase, bool compressed, void* stream) {
    auto& index = free_by_len_[compressed];
    auto it = index.lower_bound(pages);
    std::map<uint64_t, Run>::iterator pick = free_.end();
    for (; it != index.end(); ++it) {
        const bool aligned = side_bit(it->second) == phase;
        if (aligned || it->first >= pages + 1) {
            pick = free_.find(it->second);
            break;
        }
    }
    if (pick == free_.end()) return 0;
    const uint64_t run_va = pick->first;
    const Run run = pick->second;
    erase_free(pick);
    const size_t skip = side_bit(run_va) == phase ? 0 : 1;
    const uint64_t base = run_va + skip * kSaPageBytes;
    if (skip) {
        Run head = run;
        head.pages = 1;
        insert_free(run_va, head);
    }
    const size_t tail = run.pages - skip - pages;
    if (tail) {
        Run rest = run;
        rest.pages = tail;
        insert_free(base + pages * kSaPageBytes, rest);
    }
    // work queued by the previous user(s) of these pages must be done before a different stream touches them
    if (run.mixed) be_->device_sync();
    else if (run.stream != stream) be_->stream_sync(run.stream);
    Block b;
    b.pages = pages;
    b.seg = run.seg;
    b.stream = stream;
    live_.emplace(base, b);
    live_bytes_ += pages * kSaPageBytes;
    return base;
}

// ---------------------------------------------------------------------------
// growing and shrinking the mapped set
// ---------------------------------------------------------------------------

// Maps a new segment of exactly `pages` pages whose first page is on side `phase` and hands all
// of it out as one block.
//
// Pages come from the per-side pools where they can.  The rest is created fresh and mapped
// STRAIGHT INTO PLACE: only then can a page's side be measured, and about half of the fresh pages
// turn out to sit in a slot of the right side already.  Misplaced ones are exchanged pairwise (a
// side-1 page in a side-0 slot with a side-0 page in a side-1 slot); what cannot be paired goes
// to the pool of its true side and its slot is filled in the next round.  The reference probes
// every new page through a temporary mapping first (sideaware.cu:947-1019), which on B200 costs
// one more cuMemSetAccess (~170 us) and cuMemUnmap (~90 us) per page than this does for the half
// that lands well.
uint64_t SaAllocator::grow(size_t pages, int phase, bool compressed, void* stream, const SaAllocConfig& cfg) {
    (void)cfg;
    auto& pools = pool_[compressed];
    std::unique_ptr<Segment> seg(new Segment());
    seg->compressed = compressed;
    seg->num_pages = pages;
    // one spare page of address space lets us pick the phase of bit 21
    seg->reserved_bytes = (pages + 1) * kSaPageBytes;
    if (be_->reserve_va(&seg->reserved, seg->reserved_bytes)) return 0;
    seg->base = seg->reserved;
    if (side_bit(seg->base) != phase) seg->base += kSaPageBytes;
    seg->pages.assign(pages, Page{0, 0});
    auto slot_va = [&](size_t i) { return seg->base + i * kSaPageBytes; };

    bool ok = true;
    std::vector<size_t> missing; // slots without a page yet
    // 1) pooled pages of the matching side
    for (size_t i = 0; i < pages && ok; ++i) {
        const int want = side_bit(slot_va(i));
        if (pools[want].empty()) { missing.push_back(i); continue; }
        Page pg = pools[want].back();
        pools[want].pop_back();
        if (be_->map_page(slot_va(i), pg.handle)) {
            pools[pg.side].push_back(pg);
            ok = false;
            break;
        }
        seg->pages[i] = pg;
    }
    // access for what is mapped so far, in contiguous pieces (a range with holes cannot be opened at once)
    auto open_ranges = [&](const std::vector<size_t>& slots) -> bool { // slots ascending
        size_t k = 0;
        while (k < slots.size()) {
            size_t e = k;
            while (e + 1 < slots.size() && slots[e + 1] == slots[e] + 1) ++e;
            if (be_->set_access(slot_va(slots[k]), (e - k + 1) * kSaPageBytes)) return false;
            k = e + 1;
        }
        return true;
    };
    if (ok) {
        std::vector<size_t> pooled;
        for (size_t i = 0; i < pages; ++i)
            if (seg->pages[i].handle) pooled.push_back(i);
        ok = open_ranges(pooled);
    }
    // 2) fresh pages, probed where they are
    std::vector<uint64_t> vas;
    std::vector<uint8_t> sides;
    for (int round = 0; ok && !missing.empty() && round < 48; ++round) { // leftovers halve every round
        std::vector<size_t> fresh;
        for (size_t i : missing) {
            uint64_t h = 0;
            if (be_->create_page(&h, compressed)) break; // device memory exhausted: step 3 decides
            if (be_->map_page(slot_va(i), h)) { be_->release_page(h); ok = false; break; }
            seg->pages[i] = Page{h, 2}; // side unknown
            fresh.push_back(i);
            st_.pages_created++;
        }
        if (!ok || fresh.empty()) break;
        if (!open_ranges(fresh)) { ok = false; break; }
        vas.clear();
        for (size_t i : fresh) vas.push_back(slot_va(i));
        sides.assign(fresh.size(), 0);
        if (be_->probe_pages(vas.data(), (int)fresh.size(), sides.data(), stream)) { ok = false; break; }
        std::vector<size_t> wrong[2]; // wrong[w]: slots that want side w and hold a page of side 1 - w
        for (size_t k = 0; k < fresh.size(); ++k) {
            const size_t i = fresh[k];
            seg->pages[i].side = sides[k] & 1;
            const int want = side_bit(slot_va(i));
            if ((int)seg->pages[i].side != want) wrong[want].push_back(i);
        }
        // exchange misplaced pages pairwise
        while (ok && !wrong[0].empty() && !wrong[1].empty()) {
            const size_t i = wrong[0].back(), j = wrong[1].back();
            wrong[0].pop_back();
            wrong[1].pop_back();
            be_->unmap_page(slot_va(i));
            be_->unmap_page(slot_va(j));
            std::swap(seg->pages[i], seg->pages[j]);
            if (be_->map_page(slot_va(i), seg->pages[i].handle)) { pools[seg->pages[i].side].push_back(seg->pages[i]); seg->pages[i] = Page{0, 0}; ok = false; }
            if (be_->map_page(slot_va(j), seg->pages[j].handle)) { pools[seg->pages[j].side].push_back(seg->pages[j]); seg->pages[j] = Page{0, 0}; ok = false; }
            if (ok && (be_->set_access(slot_va(i), kSaPageBytes) || be_->set_access(slot_va(j), kSaPageBytes))) ok = false;
        }
        // what is left over is all of one kind: those pages wait in the pool of their true side
        std::vector<size_t> still;
        for (int w = 0; w < 2; ++w)
            for (size_t i : wrong[w]) {
                be_->unmap_page(slot_va(i));
                pools[seg->pages[i].side].push_back(seg->pages[i]);
                seg->pages[i] = Page{0, 0};
                still.push_back(i);
            }
        // slots for which no page could be created stay missing too
        for (size_t i : missing)
            if (!seg->pages[i].handle && std::find(still.begin(), still.end(), i) == still.end()) still.push_back(i);
        std::sort(still.begin(), still.end());
        missing.swap(still);
    }
    // 3) no page of the right side to be had: one of the other side still works, only slower
    if (ok && !missing.empty()) {
        std::vector<size_t> crossed;
        for (size_t i : missing) {
            const int other = side_bit(slot_va(i)) ^ 1;
            if (pools[other].empty()) { ok = false; break; }
            if (!warned_cross_) {
                std::fprintf(stderr, "sideaware: no free page on side %d, mapping a page of the other side (slower, still correct)\n", other ^ 1);
                warned_cross_ = true;
            }
            Page pg = pools[other].back();
            pools[other].pop_back();
            if (be_->map_page(slot_va(i), pg.handle)) { pools[pg.side].push_back(pg); ok = false; break; }
            seg->pages[i] = pg;
            st_.cross_side_pages++;
            crossed.push_back(i);
        }
        if (ok) ok = open_ranges(crossed);
    }
    if (!ok) {
        for (size_t i = 0; i < pages; ++i) {
            Page& pg = seg->pages[i];
            if (!pg.handle) continue;
            be_->unmap_page(slot_va(i));
            if (pg.side <= 1) pools[pg.side].push_back(pg);
            else be_->release_page(pg.handle); // never measured: give it back
        }
        be_->free_va(seg->reserved, seg->reserved_bytes);
        return 0;
    }
    seg->mapped_pages = pages;
    Block b;
    b.pages = pages;
    b.seg = seg.get();
    b.stream = stream;
    const uint64_t base = seg->base;
    live_.emplace(base, b);
    live_bytes_ += pages * kSaPageBytes;
    segments_.push_back(std::move(seg));
    return base;
}

// Unmaps the pages of a free run (already removed from the free indices) and returns them to
// the pools.  The hole stays reserved until the whole segment is unmapped.
void SaAllocator::unmap_run(uint64_t va, const Run& run) {
    Segment* seg = run.seg;
    const size_t first = (size_t)((va - seg->base) / kSaPageBytes);
    for (size_t i = 0; i < run.pages; ++i) {
        Page& pg = seg->pages[first + i];
        be_->unmap_page(va + i * kSaPageBytes);
        pool_[seg->compressed][pg.side].push_back(pg);
        pg.handle = 0;
    }
    seg->mapped_pages -= run.pages;
    if (seg->mapped_pages == 0) {
        be_->free_va(seg->reserved, seg->reserved_bytes);
        for (size_t i = 0; i < segments_.size(); ++i)
            if (segments_[i].get() == seg) {
                segments_[i] = std::move(segments_.back());
                segments_.pop_back();
                break;
            }
    }
}

void SaAllocator::trim_locked(size_t start, size_t end) {
    if (cached_bytes_ <= start || cached_bytes_ == 0) return;
    be_->device_sync(); // freed pages may still be in use by queued work
    st_.trims++;
    // least recently freed first
    std::vector<std::pair<uint64_t, uint64_t>> order; // (freed_seq, va)
    order.reserve(free_.size());
    for (auto& kv : free_) order.emplace_back(kv.second.freed_seq, kv.first);
    std::sort(order.begin(), order.end());
    for (auto& o : order) {
        if (cached_bytes_ <= end) break;
        auto it = free_.find(o.second);
        if (it == free_.end()) continue;
        const uint64_t va = it->first;
        const Run run = it->second;
        erase_free(it);
        unmap_run(va, run);
    }
    be_->device_sync();
}

// ---------------------------------------------------------------------------
// public operations
// ---------------------------------------------------------------------------

// Blocks of one page-rounded size always start on the same side.  A size seen for the first
// time takes the side that needs no skipped page in the best-fitting free run, else the side
// with more pooled pages (the reference's rule, sideaware.cu:1084-1088).
int SaAllocator::choose_phase(size_t bytes, size_t pages, bool compressed) {
    auto it = phase_.find(bytes);
    if (it != phase_.end()) return it->second;
    int phase;
    auto fit = free_by_len_[compressed].lower_bound(pages);
    if (fit != free_by_len_[compressed].end()) phase = side_bit(fit->second);
    else phase = pool_[compressed][0].size() >= pool_[compressed][1].size() ? 0 : 1;
    phase_.emplace(bytes, phase);
    return phase;
}

uint64_t SaAllocator::malloc(size_t size, void* stream, const SaAllocConfig& cfg) {
    std::lock_guard<std::mutex> lock(mu_);
    const size_t bytes = round_to_pages(size);
    const size_t pages = bytes / kSaPageBytes;
    const bool compressed = cfg.compression && comp_ok_;
    if (capacity_ && bytes > capacity_) return 0; // can never fit: do not drain the device trying
    const int phase = choose_phase(bytes, pages, compressed);

    // 1) a free run of still-mapped pages (no driver call at all)
    uint64_t p = take_from_free(pages, phase, compressed, stream);
    if (p) {
        live_[p].requested = size;
        st_.reuse_hits++;
        st_.large_allocs++;
        return p;
    }
    // 2..4) the ladder of sideaware.cu:1233-1252: unmap free memory above the threshold, unmap
    // all of it, give all pooled pages back to the driver; try to map a new segment after each
    for (int step = 0; step < 3; ++step) {
        if (step == 0) trim_locked(cfg.trim_start, cfg.trim_end);
        else if (step == 1) trim_locked(0, 0);
        else {
            trim_locked(0, 0);
            release_pools();
            be_->device_sync();
        }
        p = grow(pages, phase, compressed, stream, cfg);
        if (p) {
            live_[p].requested = size;
            st_.large_allocs++;
            return p;
        }
    }
    // nothing worked: do not sit on the pages gathered while trying
    release_pools();
    return 0;
}

bool SaAllocator::free(uint64_t ptr, void* stream) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = live_.find(ptr);
    if (it == live_.end()) return false;
    Block b = it->second;
    live_.erase(it);
    live_bytes_ -= b.pages * kSaPageBytes;
    (void)stream; // the run remembers the stream the block was handed out on (sideaware.cu:1209-1214)
    Run run;
    run.pages = b.pages;
    run.seg = b.seg;
    run.freed_seq = ++seq_;
    run.stream = b.stream;
    insert_free(ptr, run);
    return true;
}

bool SaAllocator::owns(uint64_t ptr) {
    std::lock_guard<std::mutex> lock(mu_);
    return live_.count(ptr) != 0;
}

void SaAllocator::trim(size_t start, size_t end) {
    std::lock_guard<std::mutex> lock(mu_);
    trim_locked(start, end);
}

size_t SaAllocator::release_unused() {
    std::lock_guard<std::mutex> lock(mu_);
    trim_locked(0, 0);
    size_t released = 0;
    for (int c = 0; c < 2; ++c)
        for (int s = 0; s < 2; ++s) released += pool_[c][s].size() * kSaPageBytes;
    release_pools();
    be_->device_sync();
    return released;
}

SaAllocStats SaAllocator::stats() {
    std::lock_guard<std::mutex> lock(mu_);
    SaAllocStats s = st_;
    s.bytes_live = live_bytes_;
    s.bytes_cached = cached_bytes_;
    s.pages_pool[0] = pool_[0][0].size() + pool_[1][0].size();
    s.pages_pool[1] = pool_[0][1].size() + pool_[1][1].size();
    s.segments = segments_.size();
    s.free_runs = free_.size();
    return s;
}

int SaAllocator::phase_of_size(size_t aligned_size) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = phase_.find(aligned_size);
    return it == phase_.end() ? -1 : it->second;
}
