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

// Creates `count` physical pages, learns their side through a temporary mapping and
// files them in the pools.  Partial success is success (as sideaware.cu:1029-1033).
int SaAllocator::create_pages(int count, bool compressed, void* stream, const SaAllocConfig& cfg, int* created) {
    int last_error = 0;
    *created = 0;
    const int batch_cap = std::max(1, cfg.max_probe_batch);
    std::vector<uint8_t> sides;
    while (count > 0) {
        int batch = std::min(count, batch_cap);
        uint64_t va = 0;
        last_error = be_->reserve_va(&va, (size_t)batch * kSaPageBytes);
        if (last_error) break;
        std::vector<uint64_t> handles;
        handles.reserve(batch);
        for (int i = 0; i < batch; ++i) {
            uint64_t h = 0;
            last_error = be_->create_page(&h, compressed);
            if (last_error) break;
            last_error = be_->map_page(va + (uint64_t)i * kSaPageBytes, h);
            if (last_error) { be_->release_page(h); break; }
            handles.push_back(h);
        }
        int got = (int)handles.size();
        bool ok = got > 0;
        if (ok) {
            last_error = be_->set_access(va, (size_t)got * kSaPageBytes);
            ok = last_error == 0;
        }
        if (ok) {
            sides.assign(got, 0);
            last_error = be_->probe_pages(va, got, sides.data(), stream);
            ok = last_error == 0;
        }
        for (int i = 0; i < got; ++i) be_->unmap_page(va + (uint64_t)i * kSaPageBytes);
        be_->free_va(va, (size_t)batch * kSaPageBytes);
        if (!ok) {
            for (uint64_t h : handles) be_->release_page(h);
            break;
        }
        for (int i = 0; i < got; ++i) {
            pool_[compressed][sides[i] & 1].push_back(Page{handles[i], (uint8_t)(sides[i] & 1)});
            seen_side_[sides[i] & 1]++;
        }
        st_.pages_created += got;
        *created += got;
        count -= got;
        if (got < batch) break; // device memory exhausted
    }
    return *created > 0 ? 0 : (last_error ? last_error : 1);
}

// Makes sure both pools can serve about half of `num_pages` each.  New pages land on
// either side at random, hence the over-allocation (sideaware.cu:1064-1080) and several
// rounds before the caller falls back to cross-side mapping.
int SaAllocator::top_up(size_t num_pages, bool compressed, void* stream, const SaAllocConfig& cfg) {
    int rc = 0;
    for (int round = 0; round < 4; ++round) {
        // a block alternates sides page by page; the side it starts on takes the odd page
        size_t need = (num_pages + 1) / 2 + (size_t)std::max(0, cfg.extra_required) / 2;
        size_t have0 = pool_[compressed][0].size(), have1 = pool_[compressed][1].size();
        size_t short0 = need > have0 ? need - have0 : 0, short1 = need > have1 ? need - have1 : 0;
        size_t worst = std::max(short0, short1);
        if (worst == 0) return 0;
        // how often has a new page landed on the side we are short of? (1/2 on a balanced device)
        int short_side = short1 > short0 ? 1 : 0;
        double frac = (double)(seen_side_[short_side] + 1) / (double)(seen_side_[0] + seen_side_[1] + 2);
        frac = std::min(0.5, std::max(0.05, frac));
        size_t want = (size_t)((double)worst / frac * (round == 0 ? 1.0 : 1.15)) + (round == 0 ? (size_t)std::max(0, cfg.extra_alloc) : 2);
        int created = 0;
        rc = create_pages((int)std::min<size_t>(want, 1u << 30), compressed, stream, cfg, &created);
        if (rc) return rc;
    }
    return 0;
}

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

// Maps a new segment of exactly `pages` pages whose first page is on side `phase`
// and hands all of it out as one block.
uint64_t SaAllocator::grow(size_t pages, int phase, bool compressed, void* stream, const SaAllocConfig& cfg) {
    top_up(pages, compressed, stream, cfg); // failure is handled below: we may still have enough pages
    auto& pools = pool_[compressed];
    if (pools[0].size() + pools[1].size() < pages) return 0;

    std::unique_ptr<Segment> seg(new Segment());
    seg->compressed = compressed;
    seg->num_pages = pages;
    // one spare page of address space lets us pick the phase of bit 21
    seg->reserved_bytes = (pages + 1) * kSaPageBytes;
    if (be_->reserve_va(&seg->reserved, seg->reserved_bytes)) return 0;
    seg->base = seg->reserved;
    if (side_bit(seg->base) != phase) seg->base += kSaPageBytes;

    seg->pages.reserve(pages);
    bool ok = true;
    for (size_t i = 0; i < pages && ok; ++i) {
        uint64_t va = seg->base + i * kSaPageBytes;
        int want = side_bit(va);
        int from = want;
        if (pools[from].empty()) {
            from ^= 1;
            if (pools[from].empty()) { ok = false; break; }
            if (!warned_cross_) {
                std::fprintf(stderr, "sideaware: no free page on side %d, mapping a page of the other side (slower, still correct)\n", want);
                warned_cross_ = true;
            }
            st_.cross_side_pages++;
        }
        Page pg = pools[from].back();
        pools[from].pop_back();
        if (be_->map_page(va, pg.handle)) {
            pools[pg.side].push_back(pg);
            ok = false;
            break;
        }
        seg->pages.push_back(pg);
    }
    if (ok && be_->set_access(seg->base, pages * kSaPageBytes)) ok = false;
    if (!ok) {
        for (size_t i = 0; i < seg->pages.size(); ++i) {
            be_->unmap_page(seg->base + i * kSaPageBytes);
            pools[seg->pages[i].side].push_back(seg->pages[i]);
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
