#include "sa_alloc.hpp"

#include <algorithm>
#include <cstdio>

static inline size_t round_to_pages(size_t size) {
    if (size == 0) size = 1;
    return (size + kSaPageBytes - 1) / kSaPageBytes * kSaPageBytes;
}

static inline int side_bit(uint64_t va) { return (int)((va >> kSaSideBit) & 1); }

// Pages created between two measurements.  Guesses about a chunk build on guesses about the
// chunks before it, so with chunks a round is two groups long: one boundary that does not behave
// as expected then costs one group, not many.  Single pages are judged one by one, and a long
// round saves probe launches.
constexpr int kChunkRound = 2 * kSaGroupPages;
constexpr int kSinglesRound = 64;

SaAllocator::~SaAllocator() {
    // Process teardown: the driver reclaims everything; touching it here could run
    // after the CUDA context is gone.
}

// ---------------------------------------------------------------------------
// physical memory not mapped anywhere
// ---------------------------------------------------------------------------

void SaAllocator::release_pools() {
    for (int c = 0; c < 2; ++c)
        for (int s = 0; s < 2; ++s)
            for (int l = 1; l <= kSaMaxChunkPages; ++l) {
                for (auto& ch : pool_[c][s][l]) be_->release_chunk(ch.handle);
                pool_[c][s][l].clear();
            }
}

void SaAllocator::pool_push(bool compressed, const Chunk& c) {
    if (c.side > 1 || c.len < 1 || c.len > kSaMaxChunkPages) { // never measured: nothing is known about it
        be_->release_chunk(c.handle);
        return;
    }
    pool_[compressed][c.side][c.len].push_back(c);
}

bool SaAllocator::pool_pop(bool compressed, int side, int len, Chunk* out) {
    auto& v = pool_[compressed][side][len];
    if (v.empty()) return false;
    *out = v.back();
    v.pop_back();
    return true;
}

// pooled pages homed on `side` (a chunk's pages alternate from the side of its page 0)
size_t SaAllocator::pooled_pages(bool compressed, int side) const {
    size_t n = 0;
    for (int s = 0; s < 2; ++s)
        for (int l = 1; l <= kSaMaxChunkPages; ++l)
            n += pool_[compressed][s][l].size() * (size_t)(s == side ? (l + 1) / 2 : l / 2);
    return n;
}

// Keeps the guess about the physical layout up to date: `sides` are those of newly created
// pages in the order they were created.  Inside a group sides alternate; a side seen twice in a
// row marks a group boundary just before the second one.  Most boundaries repeat a side; the ones
// that do not come at regular distances (every 8th group on the GPUs measured, with a few extra),
// so the distances between them are remembered and the commonest one is expected again.
void SaAllocator::note_fresh_sides(const uint8_t* sides, int n) {
    for (int i = 0; i < n; ++i) {
        const int x = sides[i] & 1;
        if (phys_last_side_ >= 0) {
            const bool repeated = x == phys_last_side_;
            if (repeated) phys_pos_ = 0; // wherever we thought we were
            if (phys_pos_ == 0) {        // this page opens a group
                if (repeated) {
                    ++groups_since_plain_;
                } else {
                    plain_gaps_[plain_gap_count_++ % kGapHistory] = groups_since_plain_ + 1;
                    groups_since_plain_ = 0;
                }
            }
        }
        phys_pos_ = (phys_pos_ + 1) % kSaGroupPages;
        phys_last_side_ = x;
    }
}

// The distance (in groups) at which the next boundary WITHOUT a repeated side is expected, 0 = no idea.
int SaAllocator::expected_plain_gap() const {
    const int have = std::min(plain_gap_count_, kGapHistory);
    if (have < 2) return 0;
    int best = 0, best_votes = 0;
    for (int i = 0; i < have; ++i) {
        int votes = 0;
        for (int j = 0; j < have; ++j) votes += plain_gaps_[j] == plain_gaps_[i];
        if (votes > best_votes || (votes == best_votes && plain_gaps_[i] > best)) { best = plain_gaps_[i]; best_votes = votes; }
    }
    return best_votes >= 2 ? best : 0;
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

// Adds a free run and merges it with free neighbours of the same segment that were last used on
// the same stream.  (Runs of different streams stay apart: a merged run would have to wait for
// every stream that ever touched a part of it, and with few long segments such runs would soon
// be the rule.  Each stream so keeps runs of its own, as in torch's caching allocator.)
void SaAllocator::insert_free(uint64_t va, Run run) {
    auto merge = [](Run& into, const Run& other) {
        into.pages += other.pages;
        into.freed_seq = std::max(into.freed_seq, other.freed_seq);
        if (into.clean) { // the other one's users are the only ones to wait for
            into.stream = other.stream;
            into.free_stream = other.free_stream;
            into.clean = other.clean;
        }
    };
    auto same_user = [](const Run& a, const Run& b) {
        return a.clean || b.clean || (a.stream == b.stream && a.free_stream == b.free_stream);
    };
    auto next = free_.lower_bound(va);
    if (next != free_.end() && next->second.seg == run.seg && va + run.pages * kSaPageBytes == next->first &&
        same_user(next->second, run)) {
        Run n = next->second;
        erase_free(next);
        merge(run, n);
    }
    auto prev = free_.lower_bound(va);
    if (prev != free_.begin()) {
        --prev;
        if (prev->second.seg == run.seg && prev->first + prev->second.pages * kSaPageBytes == va && same_user(prev->second, run)) {
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

// Work queued by the previous users of a run (the stream it was handed out on and, if the caller moved the block,
// the stream it was freed on) must be done before a different stream touches the pages: ordered on the device
// through an event, the host does not wait (the reference blocks the host, sideaware.cu:1209-1214).
void SaAllocator::wait_for_users(const Run& run, void* stream) {
    if (run.clean) return;
    if (run.stream != stream) be_->order_after(run.stream, stream);
    if (run.free_stream != run.stream && run.free_stream != stream) be_->order_after(run.free_stream, stream);
}

// Best fit: the shortest free run that can hold `pages` pages starting on side `phase`
// (a run that starts on the other side needs one page more; that page stays free).  Among the
// shortest few, one last used on the asking stream is preferred: it needs no waiting.
uint64_t SaAllocator::take_from_free(size_t pages, int phase, bool compressed, void* stream) {
    auto& index = free_by_len_[compressed];
    auto it = index.lower_bound(pages);
    std::map<uint64_t, Run>::iterator pick = free_.end();
    int looked = 0;
    for (; it != index.end() && looked < 16; ++it) {
        const bool aligned = side_bit(it->second) == phase;
        if (!(aligned || it->first >= pages + 1)) continue;
        auto cand = free_.find(it->second);
        ++looked;
        if (pick == free_.end()) pick = cand;
        if (cand->second.clean || (cand->second.stream == stream && cand->second.free_stream == stream)) { pick = cand; break; }
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
    wait_for_users(run, stream);
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

// Fills the empty slots [lo, hi) of a segment with physical memory.  True if all of them are
// mapped and accessible afterwards; otherwise everything this call mapped is taken out again.
//
// 1) Pooled chunks (their sides are known) are put where they fit, largest first.
// 2) The rest is created fresh, a few chunks per round, each mapped where the pages seen so far
//    suggest it will fit, then measured IN PLACE (only a mapped page can be measured): a chunk that
//    fits stays, one that alternates but starts on the other side is moved to a place that wants it
//    or pooled, one whose pages do not alternate is given back and re-made in two pieces split
//    where the side repeated.  The reference probes every new page through a temporary mapping
//    first (sideaware.cu:947-1019), at one more cuMemSetAccess and cuMemUnmap per page.
// 3) If device memory ran out on the way, pooled chunks of the other side fill what is left
//    (slower, still correct).
bool SaAllocator::map_slots(Segment* seg, size_t lo, size_t hi, void* stream) {
    const bool compressed = seg->compressed;
    std::vector<Slot>& slots = seg->pages;
    auto slot_va = [&](size_t i) { return seg->base + i * kSaPageBytes; };
    auto want = [&](size_t i) { return side_bit(slot_va(i)); };
    const size_t pages = hi; // scans below stop here

    bool ok = true;
    size_t empty = hi - lo;
    size_t first_empty = lo;

    // maps chunk `c` at slot `at`; a chunk that cannot be mapped goes back to the pool (or the driver)
    auto put = [&](size_t at, const Chunk& c) -> bool {
        if (be_->map_chunk(slot_va(at), c.handle, c.len)) {
            pool_push(compressed, c);
            return false;
        }
        for (int k = 0; k < c.len; ++k) {
            Slot& sl = slots[at + k];
            sl.handle = c.handle;
            sl.len = c.len;
            sl.idx = (uint8_t)k;
            sl.side = c.side <= 1 ? (uint8_t)(c.side ^ (k & 1)) : (uint8_t)2;
        }
        empty -= c.len;
        return true;
    };
    // unmaps the chunk that starts at slot `at`
    auto lift = [&](size_t at) -> Chunk {
        Chunk c;
        c.handle = slots[at].handle;
        c.len = slots[at].len;
        c.side = slots[at].side;
        be_->unmap_chunk(slot_va(at), c.len);
        for (int k = 0; k < c.len; ++k) slots[at + k] = Slot{};
        empty += c.len;
        if (at < first_empty) first_empty = at;
        return c;
    };
    // access for newly mapped chunks, one call per contiguous stretch
    auto open = [&](std::vector<std::pair<size_t, int>>& placed) -> bool { // (slot, len)
        std::sort(placed.begin(), placed.end());
        size_t k = 0;
        while (k < placed.size()) {
            size_t from = placed[k].first, to = from + placed[k].second;
            while (k + 1 < placed.size() && placed[k + 1].first == to) to += placed[++k].second;
            if (be_->set_access(slot_va(from), (to - from) * kSaPageBytes)) return false;
            ++k;
        }
        placed.clear();
        return true;
    };
    // leftmost place where `len` empty slots start with one that wants side `s`: the start of an
    // empty stretch, or its second slot (the first is then left for a single page)
    auto find_place = [&](int len, int s, size_t* at) -> bool {
        while (first_empty < pages && slots[first_empty].handle) ++first_empty;
        size_t i = first_empty;
        while (i < pages) {
            if (slots[i].handle) { ++i; continue; }
            const size_t cand = want(i) == s ? i : i + 1;
            size_t e = i;
            while (e < pages && e < cand + len && !slots[e].handle) ++e;
            if (e >= cand + len) { *at = cand; return true; }
            while (e < pages && !slots[e].handle) ++e; // too short: skip the rest of this stretch
            i = e;
        }
        return false;
    };
    auto largest_room = [&](int cap) -> int { // longest empty stretch, counted up to `cap`
        int best = 0;
        size_t i = first_empty;
        while (i < pages && best < cap) {
            if (slots[i].handle) { ++i; continue; }
            int run = 0;
            while (i < pages && !slots[i].handle) { ++i; if (++run >= cap) break; }
            best = std::max(best, run);
        }
        return best;
    };

    std::vector<std::pair<size_t, int>> placed;
    // Pooled chunks, exactly where they fit: every empty stretch is filled from its left end, largest
    // chunk first, until nothing pooled starts on the side the next slot wants.  (Going on behind a
    // slot that cannot be served would cut the stretch into single-slot holes, which only single
    // pages can fill; one slot is skipped only if a chunk of two pages or more fits right after it.)
    // `leftovers_only`: stretches of a group or more are left alone, they are cheaper to fill with fresh groups.
    auto fill_from_pool = [&](bool leftovers_only) -> bool {
        size_t i = leftovers_only ? first_empty : lo; // nothing is empty before first_empty
        while (i < pages) {
            if (slots[i].handle) { ++i; continue; }
            size_t e = i;
            while (e < pages && !slots[e].handle) ++e; // empty stretch [i, e)
            if (!(leftovers_only && e - i >= (size_t)kSaGroupPages)) {
                while (i < e) {
                    const int room = (int)std::min<size_t>(e - i, kSaMaxChunkPages);
                    const int w = want(i);
                    Chunk c;
                    bool found = false;
                    for (int l = room; l >= 1 && !found; --l) found = pool_pop(compressed, w, l, &c);
                    if (!found && room >= 3) { // a longer chunk one slot further on?
                        for (int l = room - 1; l >= 2 && !found; --l) found = pool_pop(compressed, w ^ 1, l, &c);
                        if (found) ++i;
                    }
                    if (!found) break;
                    if (!put(i, c)) return false;
                    placed.emplace_back(i, c.len);
                    i += c.len;
                }
            }
            i = e;
        }
        return open(placed);
    };
    // 1) what the pool can give
    ok = fill_from_pool(false);

    // 2) fresh chunks, measured where they are mapped
    struct Fresh { size_t at; int len; bool remade; };
    std::vector<Fresh> fresh;
    std::vector<uint64_t> vas;
    std::vector<uint8_t> sides;
    std::vector<Chunk> displaced;
    bool memory_left = true;
    const int max_rounds = 64 + (int)((hi - lo) / 4);
    auto leftmost = [&](int len, size_t* at) -> bool {
        size_t a0 = 0, a1 = 0;
        const bool h0 = find_place(len, 0, &a0), h1 = find_place(len, 1, &a1);
        if (!h0 && !h1) return false;
        *at = (h0 && (!h1 || a0 <= a1)) ? a0 : a1;
        return true;
    };
    for (int round = 0; ok && empty > 0 && memory_left && round < max_rounds; ++round) {
        if (round > 0 && !fill_from_pool(true)) { ok = false; break; } // holes that chunks pooled meanwhile can fill
        if (empty == 0) break;
        fresh.clear();
        // what the pages about to be created are expected to look like
        int pred_pos = phys_pos_, pred_last = phys_last_side_, pred_since = groups_since_plain_;
        const int plain_gap = expected_plain_gap();
        const size_t budget = std::min<size_t>(empty, (size_t)(singles_left_ > 0 ? kSinglesRound : round_pages_));
        size_t planned = 0;
        while (ok && planned < budget) {
            // size: never across the expected group boundary; 7 at the start of a group, so that the
            // group's last page comes as a single and the eight can be laid down either way round
            int len, s_hat;
            const bool remade = !forced_.empty();
            if (remade) {
                len = forced_.back().first;
                s_hat = forced_.back().second;
            } else {
                len = singles_left_ > 0 ? 1 : (pred_pos == 0 ? kSaMaxChunkPages : kSaGroupPages - pred_pos);
                // inside a group sides alternate; a new group mostly starts on the side the last one ended on
                const bool repeats = pred_pos == 0 && !(plain_gap && pred_since + 1 == plain_gap);
                s_hat = pred_last < 0 ? -1 : (repeats ? pred_last : pred_last ^ 1);
            }
            len = std::min<int>(len, (int)std::min<size_t>(budget - planned, kSaMaxChunkPages));
            len = std::min(len, largest_room(len));
            if (len < 1) break;
            size_t at = 0;
            if (s_hat < 0 || !find_place(len, s_hat, &at)) {
                // no expectation, or no room where that side is wanted: one page shorter fits one slot further on
                if (s_hat >= 0 && len > 1 && find_place(len - 1, s_hat, &at)) len -= 1;
                else if (!leftmost(len, &at)) break;
            }
            uint64_t h = 0;
            if (be_->create_chunk(&h, len, compressed)) {
                forced_.clear();
                if (len > 1) { singles_left_ = 64; continue; } // no piece of that size left: single pages may still be had
                memory_left = false;
                break;
            }
            st_.handles_created++;
            st_.pages_created += (uint64_t)len;
            if (remade) forced_.pop_back();
            else if (singles_left_ > 0) --singles_left_;
            Chunk c;
            c.handle = h;
            c.len = (uint8_t)len;
            c.side = 2;
            if (!put(at, c)) { ok = false; break; }
            placed.emplace_back(at, len);
            fresh.push_back(Fresh{at, len, remade});
            planned += (size_t)len;
            if (!remade) {
                const int first = s_hat >= 0 ? s_hat : want(at);
                if (pred_pos == 0) pred_since = (plain_gap && pred_since + 1 == plain_gap) ? 0 : pred_since + 1;
                pred_last = first ^ ((len - 1) & 1);
                pred_pos = (pred_pos + len) % kSaGroupPages;
            }
        }
        if (!ok || fresh.empty()) break;
        if (!open(placed)) { ok = false; break; }
        vas.clear();
        for (auto& f : fresh)
            for (int k = 0; k < f.len; ++k) vas.push_back(slot_va(f.at + (size_t)k));
        sides.assign(vas.size(), 0);
        if (be_->probe_pages(vas.data(), (int)vas.size(), sides.data(), stream)) { ok = false; break; }
        // judge them in the order they were created
        displaced.clear();
        size_t off = 0;
        int bad = 0;
        for (auto& f : fresh) {
            const uint8_t* sd = &sides[off];
            off += (size_t)f.len;
            if (!f.remade) note_fresh_sides(sd, f.len); // a re-made piece lies behind what came after it: it says nothing new
            int rep = 0; // first page on the same side as the page before it
            for (int k = 1; k < f.len && !rep; ++k)
                if ((sd[k] & 1) == (sd[k - 1] & 1)) rep = k;
            if (rep) {
                // Unusable as a whole.  The driver hands freed memory out again first, so the same pages
                // can be had as two chunks that end and begin at the boundary just found.
                Chunk c = lift(f.at);
                be_->release_chunk(c.handle);
                st_.handles_discarded++;
                ++bad;
                if (!f.remade) {
                    forced_.emplace_back(f.len - rep, sd[rep] & 1);
                    forced_.emplace_back(rep, sd[0] & 1); // taken from the back: this one first
                }
                continue;
            }
            const int s0 = sd[0] & 1;
            if (s0 == want(f.at)) {
                for (int k = 0; k < f.len; ++k) slots[f.at + (size_t)k].side = (uint8_t)(s0 ^ (k & 1));
                continue;
            }
            Chunk c = lift(f.at);
            c.side = (uint8_t)s0;
            displaced.push_back(c);
        }
        // what did not fit where it was put: its sides are known now, so place it exactly, largest first
        const size_t moved = displaced.size();
        std::sort(displaced.begin(), displaced.end(), [](const Chunk& a, const Chunk& b) { return a.len > b.len; });
        for (auto& c : displaced) {
            size_t at = 0;
            if (ok && find_place(c.len, c.side, &at)) {
                if (!put(at, c)) { ok = false; continue; }
                placed.emplace_back(at, (int)c.len);
            } else {
                pool_push(compressed, c);
            }
        }
        if (ok && !placed.empty()) ok = open(placed);
        // longer rounds while the guesses hold, short ones and finally single pages while they do not
        if (bad) {
            round_pages_ = kSaGroupPages;
            recent_bad_ += bad;
            if (recent_bad_ >= 3) {
                // physical memory is not laid out as hoped (fragmented by earlier use): single pages for a
                // while, for twice as long every time chunks fail again
                singles_left_ = singles_span_;
                singles_span_ = std::min(singles_span_ * 2, 8192);
                forced_.clear();
                recent_bad_ = 0;
            }
        } else {
            if (recent_bad_ > 0) --recent_bad_;
            if (moved * 4 <= fresh.size()) round_pages_ = std::min(kChunkRound, round_pages_ * 2);
            if (singles_left_ == 0 && fresh.size() >= 2 && fresh[0].len > 1) singles_span_ = 64; // chunks work again
        }
    }
    // 3) device memory ran out: whatever is pooled fills the rest, whichever side it is on
    if (ok && empty > 0) {
        size_t i = lo;
        while (ok && i < pages) {
            if (slots[i].handle) { ++i; continue; }
            int room = 0;
            while (i + (size_t)room < pages && room < kSaMaxChunkPages && !slots[i + (size_t)room].handle) ++room;
            Chunk c;
            bool found = false;
            for (int l = room; l >= 1 && !found; --l)
                for (int s = 0; s < 2 && !found; ++s) found = pool_pop(compressed, want(i) ^ s, l, &c);
            if (!found) { ok = false; break; }
            if (!put(i, c)) { ok = false; break; }
            placed.emplace_back(i, (int)c.len);
            for (int k = 0; k < c.len; ++k)
                if ((int)slots[i + (size_t)k].side != want(i + (size_t)k)) st_.cross_side_pages++;
            if (c.side != want(i) && !warned_cross_) {
                std::fprintf(stderr, "sideaware: device memory is short, mapping pages against their side (slower, still correct)\n");
                warned_cross_ = true;
            }
            i += c.len;
        }
        if (ok) ok = open(placed);
    }
    if (!ok) {
        for (size_t i = lo; i < hi; ++i) {
            if (!slots[i].handle || slots[i].idx != 0) continue;
            Chunk c = lift(i);
            pool_push(compressed, c); // a chunk that was never measured goes back to the driver
        }
        return false;
    }
    return true;
}

// Address space reserved behind a new segment: later blocks are put there, next to the earlier
// ones, so that freed neighbours merge into runs that larger requests can use (separate segments
// never merge).  Address space is plentiful (47 bits); nothing is mapped until it is needed.
static size_t segment_slack(size_t pages) { return std::max<size_t>(3 * pages, 4096); }

// Maps a new segment of `pages` pages whose first page is on side `phase` and hands all of it out
// as one block; `headroom` more pages are mapped behind it as a free run (dropped if memory is short).
uint64_t SaAllocator::grow(size_t pages, int phase, bool compressed, void* stream, size_t headroom) {
    std::unique_ptr<Segment> seg(new Segment());
    seg->compressed = compressed;
    // one spare page of address space lets us pick the phase of bit 21
    seg->capacity = pages + headroom + segment_slack(pages);
    seg->reserved_bytes = (seg->capacity + 1) * kSaPageBytes;
    if (be_->reserve_va(&seg->reserved, seg->reserved_bytes)) {
        // address space is short: no room to extend, then
        headroom = 0;
        seg->capacity = pages;
        seg->reserved_bytes = (pages + 1) * kSaPageBytes;
        if (be_->reserve_va(&seg->reserved, seg->reserved_bytes)) return 0;
    }
    seg->base = seg->reserved;
    if (side_bit(seg->base) != phase) seg->base += kSaPageBytes;
    seg->pages.assign(pages + headroom, Slot{});
    seg->num_pages = pages + headroom;
    if (!map_slots(seg.get(), 0, pages + headroom, stream)) {
        // memory may be too short for the headroom: the request alone, then
        bool ok = false;
        if (headroom) {
            headroom = 0;
            seg->pages.assign(pages, Slot{});
            seg->num_pages = pages;
            ok = map_slots(seg.get(), 0, pages, stream);
        }
        if (!ok) {
            be_->free_va(seg->reserved, seg->reserved_bytes);
            return 0;
        }
    }
    seg->mapped_pages = pages + headroom;
    Block b;
    b.pages = pages;
    b.seg = seg.get();
    b.stream = stream;
    const uint64_t base = seg->base;
    live_.emplace(base, b);
    live_bytes_ += pages * kSaPageBytes;
    if (headroom) { // mapped and measured, never used: a free run right behind the block
        Run spare;
        spare.pages = headroom;
        spare.seg = seg.get();
        spare.freed_seq = ++seq_;
        spare.stream = spare.free_stream = stream;
        spare.clean = true;
        insert_free(base + pages * kSaPageBytes, spare);
        st_.headroom_pages += headroom;
    }
    segments_.push_back(std::move(seg));
    return base;
}

// Puts a block behind the last page of an existing segment (in the address space reserved with
// it) instead of opening a new segment.  If the segment ends in a free run, the run is part of the
// block and only the missing pages are mapped: the segment that leaves the fewest pages to map is
// taken.  Otherwise the block starts right behind the segment's last block (one page further if
// that slot is on the wrong side; the skipped page is mapped too and becomes a free run, so that
// the neighbours can still merge across it).
uint64_t SaAllocator::extend(size_t pages, int phase, bool compressed, void* stream, size_t headroom) {
    Segment* best = nullptr;
    uint64_t best_va = 0;
    size_t best_have = 0, best_room = 0, best_lead = 0;
    for (auto& sp : segments_) {
        Segment* seg = sp.get();
        if (seg->compressed != compressed || seg->num_pages >= seg->capacity) continue;
        const uint64_t end = seg->base + seg->num_pages * kSaPageBytes;
        size_t have = 0;
        uint64_t run_va = 0;
        auto it = free_.lower_bound(end);
        if (it != free_.begin()) {
            --it;
            if (it->second.seg == seg && it->first + it->second.pages * kSaPageBytes == end) {
                const size_t skip = side_bit(it->first) == phase ? 0 : 1;
                if (it->second.pages > skip) {
                    have = it->second.pages - skip;
                    run_va = it->first;
                }
            }
        }
        if (have >= pages) continue; // take_from_free would have served it
        const size_t lead = have ? 0 : (side_bit(end) == phase ? 0 : 1);
        if (seg->num_pages + lead + (pages - have) > seg->capacity) continue;
        const size_t room = seg->capacity - seg->num_pages;
        // most pages already there; then no page wasted on getting the side right; then most room left
        if (!best || have > best_have || (have == best_have && (lead < best_lead || (lead == best_lead && room > best_room)))) {
            best = seg;
            best_va = run_va;
            best_have = have;
            best_room = room;
            best_lead = lead;
        }
    }
    if (!best) return 0;
    Run run;
    size_t skip = 0;
    if (best_have) {
        auto it = free_.find(best_va);
        run = it->second;
        erase_free(it);
        skip = run.pages - best_have;
    }
    const size_t old_pages = best->num_pages;
    const uint64_t end = best->base + old_pages * kSaPageBytes;
    const size_t lead = best_have ? 0 : (side_bit(end) == phase ? 0 : 1);
    const size_t extra = lead + (pages - best_have);
    // pages beyond the request, as far as the segment has room: they stay behind the block as a free run
    headroom = std::min(headroom, best->capacity - (old_pages + extra));
    best->pages.resize(old_pages + extra + headroom, Slot{});
    if (!map_slots(best, old_pages, old_pages + extra + headroom, stream)) {
        bool ok = false;
        if (headroom) { // memory may be too short for the headroom: the request alone, then
            headroom = 0;
            best->pages.resize(old_pages + extra);
            ok = map_slots(best, old_pages, old_pages + extra, stream);
        }
        if (!ok) {
            best->pages.resize(old_pages);
            if (best_have) insert_free(best_va, run);
            return 0;
        }
    }
    best->num_pages = old_pages + extra + headroom;
    best->mapped_pages += extra + headroom;
    if (headroom) {
        Run spare;
        spare.pages = headroom;
        spare.seg = best;
        spare.freed_seq = ++seq_;
        spare.stream = spare.free_stream = stream;
        spare.clean = true; // never used
        insert_free(best->base + (old_pages + extra) * kSaPageBytes, spare);
        st_.headroom_pages += headroom;
    }
    uint64_t base;
    if (best_have) {
        if (skip) {
            Run head = run;
            head.pages = 1;
            insert_free(best_va, head);
        }
        wait_for_users(run, stream);
        base = best_va + skip * kSaPageBytes;
    } else {
        if (lead) {
            Run gap;
            gap.pages = 1;
            gap.seg = best;
            gap.freed_seq = ++seq_;
            gap.stream = gap.free_stream = stream;
            gap.clean = true; // never used
            insert_free(end, gap);
        }
        base = end + lead * kSaPageBytes;
    }
    Block b;
    b.pages = pages;
    b.seg = best;
    b.stream = stream;
    live_.emplace(base, b);
    live_bytes_ += pages * kSaPageBytes;
    st_.extensions++;
    return base;
}

// A stretch of slots that a trim left unmapped in the middle of a segment, long enough for the
// block (best fit over all segments): the block goes there, next to its old neighbours, instead
// of taking new address space.  A segment has such holes exactly when it maps fewer pages than it has slots.
uint64_t SaAllocator::refill(size_t pages, int phase, bool compressed, void* stream) {
    Segment* best = nullptr;
    size_t best_start = 0, best_len = (size_t)-1;
    for (auto& sp : segments_) {
        Segment* seg = sp.get();
        if (seg->compressed != compressed || seg->num_pages - seg->mapped_pages < pages) continue;
        size_t i = 0;
        while (i < seg->num_pages) {
            if (seg->pages[i].handle) { ++i; continue; }
            size_t e = i;
            while (e < seg->num_pages && !seg->pages[e].handle) ++e; // hole [i, e)
            const size_t start = i + (side_bit(seg->base + i * kSaPageBytes) == phase ? 0 : 1);
            if (start + pages <= e && e - i < best_len) {
                best = seg;
                best_start = start;
                best_len = e - i;
            }
            i = e;
        }
    }
    if (!best) return 0;
    if (!map_slots(best, best_start, best_start + pages, stream)) return 0;
    best->mapped_pages += pages;
    const uint64_t base = best->base + best_start * kSaPageBytes;
    Block b;
    b.pages = pages;
    b.seg = best;
    b.stream = stream;
    live_.emplace(base, b);
    live_bytes_ += pages * kSaPageBytes;
    st_.hole_refills++;
    return base;
}

// Unmaps what can be unmapped of a free run (already removed from the free indices) and returns
// it to the pools.  A mapping can only be undone as a whole, so pages of chunks that reach beyond
// the run stay mapped and go back into the free indices.  Holes stay reserved (refill() uses them
// again) until the whole segment is unmapped.
void SaAllocator::unmap_run(uint64_t va, const Run& run) {
    Segment* seg = run.seg;
    const size_t first = (size_t)((va - seg->base) / kSaPageBytes), last = first + run.pages;
    const size_t none = (size_t)-1;
    size_t kept_from = none;
    auto keep_until = [&](size_t end) {
        if (kept_from == none) return;
        Run rest = run;
        rest.pages = end - kept_from;
        insert_free(seg->base + kept_from * kSaPageBytes, rest);
        kept_from = none;
    };
    size_t i = first;
    while (i < last) {
        const Slot sl = seg->pages[i];
        const size_t c0 = i - sl.idx, c1 = c0 + sl.len; // slots of the chunk this page belongs to
        if (c0 >= first && c1 <= last) {
            keep_until(i);
            be_->unmap_chunk(seg->base + c0 * kSaPageBytes, sl.len);
            Chunk c;
            c.handle = sl.handle;
            c.len = sl.len;
            c.side = seg->pages[c0].side;
            pool_push(seg->compressed, c);
            for (size_t k = c0; k < c1; ++k) seg->pages[k] = Slot{};
            seg->mapped_pages -= sl.len;
            i = c1;
        } else {
            if (kept_from == none) kept_from = i;
            i = std::min(c1, last);
        }
    }
    keep_until(last);
    // slots that fell empty at the end of the segment are room to grow into again
    while (seg->num_pages > 0 && !seg->pages[seg->num_pages - 1].handle) --seg->num_pages;
    seg->pages.resize(seg->num_pages);
    if (seg->mapped_pages == 0) {
        be_->free_va(seg->reserved, seg->reserved_bytes);
        for (size_t k = 0; k < segments_.size(); ++k)
            if (segments_[k].get() == seg) {
                segments_[k] = std::move(segments_.back());
                segments_.pop_back();
                break;
            }
    }
}

// pages of the run that belong to chunks lying wholly inside it (only such chunks can be unmapped)
size_t SaAllocator::reclaimable_pages(uint64_t va, const Run& run) const {
    const Segment* seg = run.seg;
    const size_t first = (size_t)((va - seg->base) / kSaPageBytes), last = first + run.pages;
    size_t n = 0, i = first;
    while (i < last) {
        const Slot& sl = seg->pages[i];
        const size_t c0 = i - sl.idx, c1 = c0 + sl.len;
        if (c0 >= first && c1 <= last) n += sl.len;
        i = std::min(c1, last);
    }
    return n;
}

// If more than `start` bytes could be given back (free runs, less the pieces of chunks that reach
// into live neighbours: those stay mapped whatever happens): unmaps free runs, least recently
// freed first, until at most `end` bytes could still be given back.
// After a device-wide synchronisation nobody's work is pending on any free run: neighbours
// merge whatever stream they were last used on.
void SaAllocator::merge_all_free_runs() {
    std::vector<uint64_t> all;
    all.reserve(free_.size());
    for (auto& kv : free_) {
        kv.second.clean = true;
        all.push_back(kv.first);
    }
    for (uint64_t va : all) {
        auto it = free_.find(va);
        if (it == free_.end()) continue; // already swallowed by its predecessor
        const Run r = it->second;
        erase_free(it);
        insert_free(va, r);
    }
}

void SaAllocator::trim_locked(size_t start, size_t end) {
    if (cached_bytes_ <= start || cached_bytes_ == 0) return;
    // What could be given back once neighbouring free runs are merged (they are, after the wait below), by
    // arithmetic alone: with many short runs between live blocks most free pages belong to chunks that reach into
    // a neighbour, and a device-wide wait for a trim that then finds nothing to do is the expensive part.
    size_t could = 0;
    for (auto it = free_.begin(); it != free_.end();) {
        const uint64_t va = it->first;
        Run merged = it->second;
        auto next = std::next(it);
        while (next != free_.end() && next->second.seg == merged.seg && next->first == va + merged.pages * kSaPageBytes) {
            merged.pages += next->second.pages;
            ++next;
        }
        could += reclaimable_pages(va, merged) * kSaPageBytes;
        it = next;
    }
    if (could == 0 || could <= start) return;
    be_->device_sync(); // freed pages may still be in use by queued work
    merge_all_free_runs();
    struct Cand { uint64_t seq, va; size_t pages; };
    std::vector<Cand> order;
    order.reserve(free_.size());
    size_t reclaimable = 0;
    for (auto& kv : free_) {
        const size_t n = reclaimable_pages(kv.first, kv.second);
        if (!n) continue;
        order.push_back(Cand{kv.second.freed_seq, kv.first, n});
        reclaimable += n * kSaPageBytes;
    }
    if (reclaimable == 0 || reclaimable <= start) return;
    std::sort(order.begin(), order.end(), [](const Cand& a, const Cand& b) { return a.seq < b.seq; });
    st_.trims++;
    for (auto& o : order) {
        if (reclaimable <= end) break;
        auto it = free_.find(o.va);
        if (it == free_.end()) continue; // merged into a neighbour that was handled before
        const uint64_t va = it->first;
        const Run run = it->second;
        erase_free(it);
        unmap_run(va, run);
        reclaimable -= std::min(reclaimable, o.pages * kSaPageBytes);
    }
    be_->device_sync();
}

// ---------------------------------------------------------------------------
// public operations
// ---------------------------------------------------------------------------

// Blocks of one page-rounded size that exist at the same time always start on the same side
// (kernels rely on equal-sized buffers having equal side patterns).  A size that has no live block
// takes the side that needs no skipped page in the best-fitting free run, else the side with more
// pooled pages (the reference's rule for a size it sees for the first time, sideaware.cu:1084-1088;
// choosing again whenever the size has died out lets odd-sized blocks use up whichever side the
// pools have too much of).
int SaAllocator::choose_phase(size_t bytes, size_t pages, bool compressed) {
    auto it = phase_.find(bytes);
    if (it != phase_.end()) {
        auto lc = live_of_size_.find(bytes);
        if (lc != live_of_size_.end() && lc->second > 0) return it->second;
        phase_.erase(it);
    }
    int phase;
    auto fit = free_by_len_[compressed].lower_bound(pages);
    const size_t pooled0 = pooled_pages(compressed, 0), pooled1 = pooled_pages(compressed, 1);
    if (fit != free_by_len_[compressed].end()) phase = side_bit(fit->second);
    else if (pooled0 != pooled1) phase = pooled0 > pooled1 ? 0 : 1;
    else phase = 0;
    phase_.emplace(bytes, phase);
    return phase;
}

// free pages a request could be served from without creating physical memory: mapped-and-free plus pooled
size_t SaAllocator::pages_at_hand(bool compressed) const {
    return cached_bytes_ / kSaPageBytes + pooled_pages(compressed, 0) + pooled_pages(compressed, 1);
}

uint64_t SaAllocator::malloc(size_t size, void* stream, const SaAllocConfig& cfg) {
    std::lock_guard<std::mutex> lock(mu_);
    return malloc_locked(size, stream, cfg);
}

uint64_t SaAllocator::malloc_locked(size_t size, void* stream, const SaAllocConfig& cfg) {
    const size_t bytes = round_to_pages(size);
    const size_t pages = bytes / kSaPageBytes;
    const bool compressed = cfg.compression && comp_ok_;
    if (capacity_ && bytes > capacity_) return 0; // can never fit: do not drain the device trying
    const int phase = choose_phase(bytes, pages, compressed);
    auto served = [&](uint64_t p) {
        live_[p].requested = size;
        live_of_size_[bytes]++;
        st_.large_allocs++;
        // too little left at hand for the next request: the next free() maps some more (top_up)
        want_top_up_ = cfg.extra_required > 0 && cfg.extra_alloc > 0 && pages_at_hand(compressed) < (size_t)cfg.extra_required;
        return p;
    };

    // 1) a free run of still-mapped pages (no driver call at all)
    uint64_t p = take_from_free(pages, phase, compressed, stream);
    if (p) {
        st_.reuse_hits++;
        return served(p);
    }
    // 2..4) the ladder of sideaware.cu:1233-1252: unmap free memory above the threshold, unmap
    // all of it, give all pooled pages back to the driver; try to grow the mapped set after each.
    // Growing: into a hole an earlier trim left, else behind the last page of a segment (using the free run
    // there, if any), else a new segment.  While memory is not short the mapped set grows by extra_alloc pages
    // more than asked for (the reference creates that many spare pages whenever it has to create any,
    // sideaware.cu:1074-1076): the fixed cost of a round of driver calls and measurements is paid less often.
    for (int step = 0; step < 3; ++step) {
        if (step == 0) {
            size_t start = cfg.trim_start, end = cfg.trim_end;
            if (cfg.trim_scaled && capacity_) {
                start = std::max(start, capacity_ / 2);
                end = std::max(end, capacity_ / 4);
            }
            trim_locked(start, end);
        }
        else if (step == 1) trim_locked(0, 0);
        else {
            trim_locked(0, 0);
            release_pools();
            be_->device_sync();
        }
        const size_t headroom = (step == 0 && cfg.extra_alloc > 0) ? (size_t)cfg.extra_alloc : 0;
        p = refill(pages, phase, compressed, stream);
        if (!p && step == 0) p = extend(pages, phase, compressed, stream, headroom);
        if (!p) p = grow(pages, phase, compressed, stream, headroom);
        if (p) return served(p);
    }
    // nothing worked: do not sit on the pages gathered while trying
    release_pools();
    return 0;
}

// Maps `pages` more pages as a free run: behind the last page of the segment with the most pages that has room
// (blocks cluster there), else as a segment of its own.  Returns the pages mapped; 0 leaves everything as it was.
size_t SaAllocator::add_headroom(size_t pages, bool compressed, void* stream) {
    if (pages == 0) return 0;
    Segment* best = nullptr;
    for (auto& sp : segments_) {
        Segment* seg = sp.get();
        if (seg->compressed != compressed || seg->num_pages + pages > seg->capacity) continue;
        if (!best || seg->num_pages > best->num_pages) best = seg;
    }
    Run spare;
    spare.pages = pages;
    spare.freed_seq = ++seq_;
    spare.stream = spare.free_stream = stream;
    spare.clean = true; // never used
    if (best) {
        const size_t old_pages = best->num_pages;
        best->pages.resize(old_pages + pages, Slot{});
        if (!map_slots(best, old_pages, old_pages + pages, stream)) {
            best->pages.resize(old_pages);
            return 0;
        }
        best->num_pages = old_pages + pages;
        best->mapped_pages += pages;
        spare.seg = best;
        insert_free(best->base + old_pages * kSaPageBytes, spare);
    } else {
        std::unique_ptr<Segment> seg(new Segment());
        seg->compressed = compressed;
        seg->capacity = pages + segment_slack(pages);
        seg->reserved_bytes = (seg->capacity + 1) * kSaPageBytes;
        if (be_->reserve_va(&seg->reserved, seg->reserved_bytes)) return 0;
        seg->base = seg->reserved;
        seg->pages.assign(pages, Slot{});
        seg->num_pages = pages;
        if (!map_slots(seg.get(), 0, pages, stream)) {
            be_->free_va(seg->reserved, seg->reserved_bytes);
            return 0;
        }
        seg->mapped_pages = pages;
        spare.seg = seg.get();
        insert_free(seg->base, spare);
        segments_.push_back(std::move(seg));
    }
    st_.headroom_pages += pages;
    return pages;
}

size_t SaAllocator::top_up(void* stream, const SaAllocConfig& cfg) {
    std::lock_guard<std::mutex> lock(mu_);
    if (!want_top_up_) return 0;
    want_top_up_ = false;
    const bool compressed = cfg.compression && comp_ok_;
    if (cfg.extra_alloc <= 0 || pages_at_hand(compressed) >= (size_t)std::max(cfg.extra_required, 0)) return 0;
    const size_t got = add_headroom((size_t)cfg.extra_alloc, compressed, stream);
    if (got) st_.top_ups++;
    return got;
}

bool SaAllocator::prealloc(size_t size, const SaAllocConfig& cfg) {
    std::lock_guard<std::mutex> lock(mu_);
    const size_t want_pages = round_to_pages(size) / kSaPageBytes;
    // a free run that holds the size whichever side it has to start on: nothing to do (and its last user's
    // ordering stays as it is)
    if (free_by_len_[cfg.compression && comp_ok_].lower_bound(want_pages + 1) != free_by_len_[cfg.compression && comp_ok_].end()) return true;
    // a block of that size, given straight back: what stays is a free run nobody has used
    SaAllocConfig plain = cfg;
    plain.extra_alloc = 0;
    const uint64_t p = malloc_locked(size, nullptr, plain);
    if (!p) return false;
    auto it = live_.find(p);
    Block b = it->second;
    live_.erase(it);
    live_bytes_ -= b.pages * kSaPageBytes;
    auto lc = live_of_size_.find(b.pages * kSaPageBytes);
    if (lc != live_of_size_.end() && lc->second > 0) lc->second--;
    st_.large_allocs--;
    Run run;
    run.pages = b.pages;
    run.seg = b.seg;
    run.freed_seq = ++seq_;
    run.stream = run.free_stream = nullptr;
    run.clean = false; // the pages may have come from a run whose last user is still at work: keep its ordering
    insert_free(p, run);
    want_top_up_ = false;
    return true;
}

bool SaAllocator::free(uint64_t ptr, void* stream) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = live_.find(ptr);
    if (it == live_.end()) return false;
    Block b = it->second;
    live_.erase(it);
    live_bytes_ -= b.pages * kSaPageBytes;
    auto lc = live_of_size_.find(b.pages * kSaPageBytes);
    if (lc != live_of_size_.end() && lc->second > 0) lc->second--;
    // the run remembers the stream the block was handed out on (sideaware.cu:1209-1214) and the one it is freed on:
    // whoever gets these pages next is ordered behind both
    Run run;
    run.pages = b.pages;
    run.seg = b.seg;
    run.freed_seq = ++seq_;
    run.stream = b.stream;
    run.free_stream = stream;
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
        for (int s = 0; s < 2; ++s) released += pooled_pages(c != 0, s) * kSaPageBytes;
    release_pools();
    be_->device_sync();
    return released;
}

SaAllocStats SaAllocator::stats() {
    std::lock_guard<std::mutex> lock(mu_);
    SaAllocStats s = st_;
    s.bytes_live = live_bytes_;
    s.bytes_cached = cached_bytes_;
    s.pages_pool[0] = pooled_pages(false, 0) + pooled_pages(true, 0);
    s.pages_pool[1] = pooled_pages(false, 1) + pooled_pages(true, 1);
    s.segments = segments_.size();
    s.free_runs = free_.size();
    return s;
}

int SaAllocator::phase_of_size(size_t aligned_size) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = phase_.find(aligned_size);
    return it == phase_.end() ? -1 : it->second;
}
