#include "sa_alloc.hpp"

#include <algorithm>
#include <cstdio>

static inline size_t round_to_pages(size_t size) {
    if (size == 0) size = 1;
    return (size + kSaPageBytes - 1) / kSaPageBytes * kSaPageBytes;
}

SaAllocator::~SaAllocator() {
    // Process teardown: the driver reclaims everything; touching it here could run
    // after the CUDA context is gone.
}

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
// either side at random, hence the over-allocation (sideaware.cu:1064-1080) and up to
// three rounds before the caller falls back to cross-side mapping.
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

bool SaAllocator::build_block(Block& b, size_t size, bool compressed, void* stream, const SaAllocConfig& cfg) {
    b.bytes = round_to_pages(size);
    b.requested = size;
    b.compressed = compressed;
    b.stream = stream;
    const size_t num_pages = b.bytes / kSaPageBytes;

    top_up(num_pages, compressed, stream, cfg); // failure is handled below: we may still have enough pages
    auto& pools = pool_[compressed];
    if (pools[0].size() + pools[1].size() < num_pages) return false;

    // every block of this size starts on the same side, so equal-size buffers have equal side patterns
    auto it = phase_.find(b.bytes);
    if (it == phase_.end()) it = phase_.emplace(b.bytes, pools[0].size() >= pools[1].size() ? 0 : 1).first;
    const int start_side = it->second;

    // one spare page of address space lets us pick the phase of bit 21
    b.reserved_bytes = b.bytes + kSaPageBytes;
    if (be_->reserve_va(&b.reserved, b.reserved_bytes)) return false;
    b.base = b.reserved;
    if ((int)((b.base >> kSaSideBit) & 1) != start_side) b.base += kSaPageBytes;

    b.pages.clear();
    b.pages.reserve(num_pages);
    bool ok = true;
    for (size_t i = 0; i < num_pages && ok; ++i) {
        uint64_t va = b.base + i * kSaPageBytes;
        int want = (int)((va >> kSaSideBit) & 1);
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
        b.pages.push_back(pg);
    }
    if (ok && be_->set_access(b.base, b.bytes)) ok = false;
    if (!ok) {
        for (size_t i = 0; i < b.pages.size(); ++i) {
            be_->unmap_page(b.base + i * kSaPageBytes);
            pools[b.pages[i].side].push_back(b.pages[i]);
        }
        b.pages.clear();
        be_->free_va(b.reserved, b.reserved_bytes);
        return false;
    }
    return true;
}

void SaAllocator::unmap_block(Block& b) {
    for (size_t i = 0; i < b.pages.size(); ++i) {
        be_->unmap_page(b.base + i * kSaPageBytes);
        pool_[b.compressed][b.pages[i].side].push_back(b.pages[i]);
    }
    b.pages.clear();
    be_->free_va(b.reserved, b.reserved_bytes);
}

void SaAllocator::trim_locked(size_t start, size_t end) {
    if (cached_bytes_ <= start || cached_bytes_ == 0) return;
    be_->device_sync(); // cached blocks may still be in use by queued work
    st_.trims++;
    while (cached_bytes_ > end) {
        std::vector<Block>* oldest_vec = nullptr;
        size_t oldest_idx = 0;
        uint64_t oldest = ~0ull;
        for (auto& kv : cache_)
            for (size_t i = 0; i < kv.second.size(); ++i)
                if (kv.second[i].freed_seq < oldest) { oldest = kv.second[i].freed_seq; oldest_vec = &kv.second; oldest_idx = i; }
        if (!oldest_vec) break;
        Block b = std::move((*oldest_vec)[oldest_idx]);
        oldest_vec->erase(oldest_vec->begin() + oldest_idx);
        cached_bytes_ -= b.bytes;
        unmap_block(b);
    }
    be_->device_sync();
}

uint64_t SaAllocator::malloc(size_t size, void* stream, const SaAllocConfig& cfg) {
    std::lock_guard<std::mutex> lock(mu_);
    const size_t bytes = round_to_pages(size);
    const bool compressed = cfg.compression && comp_ok_;
    if (capacity_ && bytes > capacity_) return 0; // can never fit: do not drain the device trying

    // 1) exact-size reuse of a block that is still mapped (sideaware.cu:1199-1219)
    auto hit = cache_.find(cache_key(bytes, compressed));
    if (hit != cache_.end() && !hit->second.empty()) {
        Block b = std::move(hit->second.back());
        hit->second.pop_back();
        cached_bytes_ -= b.bytes;
        if (b.stream != stream) {
            be_->stream_sync(b.stream); // work queued by the previous user must be done
            b.stream = stream;
        }
        b.requested = size;
        uint64_t base = b.base;
        live_.emplace(base, std::move(b));
        st_.reuse_hits++;
        st_.large_allocs++;
        return base;
    }

    // 2..4) the ladder of sideaware.cu:1233-1252: trim over the threshold, trim everything,
    // give all pooled pages back to the driver; try to build the block after each step
    for (int step = 0; step < 3; ++step) {
        if (step == 0) trim_locked(cfg.trim_start, cfg.trim_end);
        else if (step == 1) trim_locked(0, 0);
        else {
            trim_locked(0, 0);
            for (int c = 0; c < 2; ++c)
                for (int s = 0; s < 2; ++s) {
                    for (auto& pg : pool_[c][s]) be_->release_page(pg.handle);
                    pool_[c][s].clear();
                }
            be_->device_sync();
        }
        Block b;
        if (build_block(b, size, compressed, stream, cfg)) {
            uint64_t base = b.base;
            live_.emplace(base, std::move(b));
            st_.large_allocs++;
            return base;
        }
    }
    // nothing worked: do not sit on the pages gathered while trying
    for (int c = 0; c < 2; ++c)
        for (int s = 0; s < 2; ++s) {
            for (auto& pg : pool_[c][s]) be_->release_page(pg.handle);
            pool_[c][s].clear();
        }
    return 0;
}

bool SaAllocator::free(uint64_t ptr, void* stream) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = live_.find(ptr);
    if (it == live_.end()) return false;
    Block b = std::move(it->second);
    live_.erase(it);
    (void)stream; // the block remembers the stream it was handed out on (sideaware.cu:1209-1214)
    b.freed_seq = ++seq_;
    cached_bytes_ += b.bytes;
    cache_[cache_key(b.bytes, b.compressed)].push_back(std::move(b));
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
        for (int s = 0; s < 2; ++s) {
            for (auto& pg : pool_[c][s]) { be_->release_page(pg.handle); released += kSaPageBytes; }
            pool_[c][s].clear();
        }
    be_->device_sync();
    return released;
}

SaAllocStats SaAllocator::stats() {
    std::lock_guard<std::mutex> lock(mu_);
    SaAllocStats s = st_;
    s.bytes_live = 0;
    for (auto& kv : live_) s.bytes_live += kv.second.bytes;
    s.bytes_cached = cached_bytes_;
    s.pages_pool[0] = pool_[0][0].size() + pool_[1][0].size();
    s.pages_pool[1] = pool_[0][1].size() + pool_[1][1].size();
    return s;
}

int SaAllocator::phase_of_size(size_t aligned_size) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = phase_.find(aligned_size);
    return it == phase_.end() ? -1 : it->second;
}
