// Latency probing kernels and their orchestration (sm_100a).
//
// The measurement primitive is a short chain of dependent L2 atomics on one
// word, timed with the SM clock: atomics are resolved at the L2 slice that
// owns the address, so the round trip tells near side from far side.  The
// atomic adds a zero that comes from a kernel parameter: memory contents never
// change, which makes it safe to probe live allocations.
// Behaviour re-created from the reference: test_latency_l2 (sideaware.cu:632-642),
// init_side_info (sideaware.cu:644-718), test_page_latency (sideaware.cu:720-738).
// Differences: every SM probes many addresses (signature matrix analysed on the
// host, see sa_topology.cpp), pages are probed by all SMs in parallel with two
// votes per page, and no kernel waits on another block.
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <unordered_map>

#include "sa_probe.hpp"

namespace {

constexpr int kNumAddr = 64;        // probe addresses inside the probe page
constexpr int kChain = 16;          // timed dependent atomics per measurement
constexpr int kDiscoverReps = 4;
constexpr int kProbeReps = 3;
constexpr int kVotes = 2;
constexpr int kMaxBatch = 8192;     // addresses per probe launch
constexpr int kTicketStride = 128;  // uint32 per slot (three counters on separate 128-byte lines)
// Every stream has its own ring of ticket slots.  Launches of one stream run in order, so a slot
// is free again once the launch that used it has ended.  A launch may begin while its predecessor
// on the stream drains (programmatic dependent launch), and so may the one after it: what bounds
// how many launches of a stream are under way at once is that every kChainLength-th launch waits
// for its predecessor to END.  The ring is twice that long.  Launches of different streams never
// share a slot, however long one of them runs.
constexpr int kRingSlots = 64;
constexpr int kChainLength = 32;
constexpr int kRingsPerBlock = 64;  // rings carved from one 2 MiB device block
constexpr int kMaxRings = 1024;     // distinct streams served before the rings are handed out afresh
constexpr size_t kRingBlockBytes = sizeof(uint32_t) * kTicketStride * kRingSlots * kRingsPerBlock;
constexpr uint32_t kSentinel = 0x9E3779B9u;

__device__ __forceinline__ uint32_t atom_add_u32(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

__device__ __forceinline__ long long read_clock() {
    long long t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
    return t;
}

// kChain round trips to the L2 slice owning *p.  Each address depends on the
// previous result, so the atomics cannot overlap.
__device__ uint32_t measure(uint32_t* p, uint32_t zero, int chain) {
    uint32_t old = atom_add_u32(p, zero); // brings the line to its home slice
    uint32_t off = (old == kSentinel) ? 1u : 0u;
    old = atom_add_u32(p + off, zero);
    off = (old == kSentinel) ? 1u : 0u;
    long long t0 = read_clock();
#pragma unroll 1
    for (int i = 0; i < chain; ++i) {
        old = atom_add_u32(p + off, zero);
        off = (old == kSentinel) ? 1u : 0u;
    }
    // one more dependent access closes the last timed round trip
    old = atom_add_u32(p + off, zero);
    long long t1 = read_clock();
    if (old == kSentinel - 1u) t1 += 1; // keeps the final result live
    return (uint32_t)(t1 - t0);
}

__global__ void sa_discover_kernel(uint8_t* page, const uint32_t* offsets, int naddr, uint32_t* lat,
                                   uint32_t* seen, uint32_t zero, int reps, int chain) {
    extern __shared__ unsigned char keep_one_block_per_sm[];
    if (threadIdx.x != 0) return;
    uint32_t smid = sa_smid();
    if (smid >= SA_MAX_SM) return;
    atomicAdd(&seen[smid], 1u);
    for (int rep = 0; rep < reps; ++rep) {
        for (int jj = 0; jj < naddr; ++jj) {
            // different SMs walk the addresses in different phases so few collide on one word
            int j = (jj + (int)smid * 5 + rep * 11) % naddr;
            uint32_t m = measure((uint32_t*)(page + offsets[j]), zero, chain);
            atomicMin(&lat[smid * naddr + j], m);
        }
    }
}

__global__ void sa_probe_addr_kernel(const uint64_t* addrs, int n, int votes, uint32_t* out_lat,
                                     uint16_t* out_smid, uint32_t zero, int reps, int chain) {
    if (threadIdx.x != 0) return;
    uint32_t smid = sa_smid();
    for (int v = 0; v < votes; ++v) {
        // the v-th vote on an address comes from another block (so, most likely, another SM)
        int shift = (v * (gridDim.x / 2 + 1)) % gridDim.x;
        for (int i = ((int)blockIdx.x + shift) % (int)gridDim.x; i < n; i += gridDim.x) {
            uint32_t best = 0xffffffffu;
            for (int r = 0; r < reps; ++r) best = min(best, measure((uint32_t*)addrs[i], zero, chain));
            out_lat[v * n + i] = best;
            out_smid[v * n + i] = (uint16_t)smid;
        }
    }
}

} // namespace

struct SaProbeDevice {
    int device = -1;
    uint8_t* page = nullptr;      // 2 MiB probe page (owned by the caller)
    uint8_t* meta = nullptr;      // one cudaMalloc block, carved below
    uint32_t* lat = nullptr;      // [SA_MAX_SM][kNumAddr]
    uint32_t* seen = nullptr;     // [SA_MAX_SM]
    uint32_t* offsets = nullptr;  // [kNumAddr]
    unsigned char* gpu_side_index = nullptr; // [SA_MAX_SM]
    uint32_t* tickets = nullptr;  // first block of rings: [kRingsPerBlock][kRingSlots][kTicketStride]
    uint64_t* addrs = nullptr;    // [kMaxBatch]
    uint32_t* out_lat = nullptr;  // [kVotes][kMaxBatch]
    uint16_t* out_smid = nullptr; // [kVotes][kMaxBatch]
    // one word of pinned host memory that kernels with bounded waits count into when a wait runs out
    // (system-scope atomic): the host reads it without synchronising with the device
    uint32_t* wait_errors_host = nullptr;
    uint32_t* wait_errors_dev = nullptr;
    std::mutex mu;
    // ticket rings
    struct Ring { uint32_t* base = nullptr; unsigned next = 0; };
    std::mutex ring_mu;
    std::unordered_map<void*, Ring*> ring_of_stream;
    std::vector<std::unique_ptr<Ring>> rings;  // all rings ever carved
    std::vector<Ring*> idle_rings;             // carved, not owned by a stream
    std::vector<uint32_t*> ring_blocks;        // device blocks (the first one lives in `meta`)
};

static std::vector<uint32_t> make_offsets() {
    std::vector<uint32_t> off;
    off.push_back(0);
    for (int b = 4; b <= 20; ++b) off.push_back(1u << b);
    // validation offsets: fixed pseudo-random multiples of 16 inside the 2 MiB page
    uint32_t x = 0x2545F491u;
    while ((int)off.size() < kNumAddr) {
        x ^= x << 13; x ^= x >> 17; x ^= x << 5;
        uint32_t o = (x & 0x1FFFF0u);
        if (o == 0 || (o & (o - 1)) == 0) continue;
        if (std::find(off.begin(), off.end(), o) != off.end()) continue;
        off.push_back(o);
    }
    return off;
}

cudaError_t sa_probe_create(int device, uint64_t probe_page_va, SaProbeDevice** out, SaTopology* topo, std::string* why) {
    auto fail = [&](cudaError_t e, const char* what) {
        if (why) *why = std::string(what) + ": " + cudaGetErrorString(e);
        return e;
    };
    cudaError_t e;
    SaProbeDevice* p = new SaProbeDevice();
    p->device = device;
    p->page = (uint8_t*)probe_page_va;

    size_t sz_lat = sizeof(uint32_t) * SA_MAX_SM * kNumAddr;
    size_t sz_seen = sizeof(uint32_t) * SA_MAX_SM;
    size_t sz_off = sizeof(uint32_t) * kNumAddr;
    size_t sz_side = SA_MAX_SM;
    size_t sz_tick = kRingBlockBytes;
    size_t sz_addr = sizeof(uint64_t) * kMaxBatch;
    size_t sz_olat = sizeof(uint32_t) * kVotes * kMaxBatch;
    size_t sz_osm = sizeof(uint16_t) * kVotes * kMaxBatch;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    size_t total = up(sz_lat) + up(sz_seen) + up(sz_off) + up(sz_side) + up(sz_tick) + up(sz_addr) + up(sz_olat) + up(sz_osm);
    if ((e = cudaMalloc(&p->meta, total)) != cudaSuccess) { delete p; return fail(e, "cudaMalloc(probe meta)"); }
    if ((e = cudaMemset(p->meta, 0, total)) != cudaSuccess) { cudaFree(p->meta); delete p; return fail(e, "cudaMemset(probe meta)"); }
    uint8_t* c = p->meta;
    p->lat = (uint32_t*)c; c += up(sz_lat);
    p->seen = (uint32_t*)c; c += up(sz_seen);
    p->offsets = (uint32_t*)c; c += up(sz_off);
    p->gpu_side_index = c; c += up(sz_side);
    p->tickets = (uint32_t*)c; c += up(sz_tick);
    p->ring_blocks.push_back(p->tickets);
    p->addrs = (uint64_t*)c; c += up(sz_addr);
    p->out_lat = (uint32_t*)c; c += up(sz_olat);
    p->out_smid = (uint16_t*)c; c += up(sz_osm);

    if ((e = cudaHostAlloc((void**)&p->wait_errors_host, 64, cudaHostAllocMapped)) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "cudaHostAlloc(wait-error word)"); }
    *p->wait_errors_host = 0u;
    if ((e = cudaHostGetDevicePointer((void**)&p->wait_errors_dev, p->wait_errors_host, 0)) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "cudaHostGetDevicePointer"); }

    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "cudaGetDeviceProperties"); }
    topo->device = device;
    topo->num_sms = prop.multiProcessorCount;

    std::vector<uint32_t> offsets = make_offsets();
    if ((e = cudaMemcpy(p->offsets, offsets.data(), sz_off, cudaMemcpyHostToDevice)) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "upload offsets"); }
    if ((e = cudaMemset(p->lat, 0xff, sz_lat)) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "cudaMemset(lat)"); }

    // Topology cache (off unless SIDEAWARE_TOPOLOGY_CACHE names a directory): what an earlier process found on this
    // very GPU under this driver, confirmed before use by re-measuring the 64 probe addresses (one launch of about
    // 40 us) against what the file claims: sides of the SMs, their thresholds and the hash at once.
    std::string cache_path, gpu_uuid;
    int driver_version = 0;
    if (const char* dir = std::getenv("SIDEAWARE_TOPOLOGY_CACHE")) {
        char hex[33];
        for (int i = 0; i < 16; ++i) std::snprintf(hex + 2 * i, 3, "%02x", (unsigned)(unsigned char)prop.uuid.bytes[i]);
        gpu_uuid = hex;
        cudaDriverGetVersion(&driver_version);
        cache_path = std::string(dir) + "/sideaware-" + gpu_uuid + ".topo";
        std::string text, reason;
        if (FILE* f = std::fopen(cache_path.c_str(), "rb")) {
            char buf[4096];
            size_t got;
            while ((got = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
            std::fclose(f);
            SaTopology cached;
            if (!sa_topology_parse(text, gpu_uuid, driver_version, topo->num_sms, &cached, &reason)) {
                std::fprintf(stderr, "sideaware: topology cache %s not used: %s\n", cache_path.c_str(), reason.c_str());
            } else if (!cached.hash_usable) {
                // nothing worth keeping: discover again
            } else {
                cached.device = device;
                std::vector<uint64_t> addrs(kNumAddr);
                for (int j = 0; j < kNumAddr; ++j) addrs[j] = probe_page_va + offsets[j];
                std::vector<uint8_t> measured(kNumAddr);
                int ambiguous = 0, wrong = 0;
                e = sa_probe_sides(p, cached, addrs.data(), kNumAddr, measured.data(), nullptr, &ambiguous);
                if (e != cudaSuccess) { sa_probe_destroy(p); return fail(e, "spot check of the cached topology"); }
                for (int j = 0; j < kNumAddr; ++j) wrong += measured[j] != (measured[0] ^ sa_parity32(offsets[j] & cached.hash));
                if (wrong <= 1 && ambiguous <= 2) {
                    *topo = cached;
                    topo->from_cache = true;
                    topo->discovery_passes = 0;
                    if ((e = cudaMemcpy(p->gpu_side_index, topo->side_index, SA_MAX_SM, cudaMemcpyHostToDevice)) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "upload side index"); }
                    *out = p;
                    return cudaSuccess;
                }
                std::fprintf(stderr, "sideaware: topology cache %s not used: %d of %d re-measured addresses disagree with it (%d ambiguous)\n",
                             cache_path.c_str(), wrong, kNumAddr, ambiguous);
            }
        }
    }

    // more than half of an SM's shared memory per block: at most one block resident per SM
    int smem = (int)std::min<size_t>(prop.sharedMemPerBlockOptin, 120 * 1024);
    if (smem > 48 * 1024) cudaFuncSetAttribute(sa_discover_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);

    // Latencies are kept as minima over all passes (noise - another process on the GPU, a clock ramp -
    // only ever adds latency), so a pass that leaves doubts is simply followed by another one.
    std::vector<uint32_t> h_lat((size_t)SA_MAX_SM * kNumAddr), h_seen(SA_MAX_SM);
    for (int pass = 0; pass < 4; ++pass) {
        sa_discover_kernel<<<2 * topo->num_sms, 32, smem>>>(p->page, p->offsets, kNumAddr, p->lat, p->seen, 0u, kDiscoverReps, kChain);
        if ((e = cudaGetLastError()) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "launch sa_discover_kernel"); }
        if ((e = cudaDeviceSynchronize()) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "sa_discover_kernel"); }
        if ((e = cudaMemcpy(h_seen.data(), p->seen, sz_seen, cudaMemcpyDeviceToHost)) != cudaSuccess ||
            (e = cudaMemcpy(h_lat.data(), p->lat, sz_lat, cudaMemcpyDeviceToHost)) != cudaSuccess) {
            sa_probe_destroy(p);
            return fail(e, "download latencies");
        }
        std::vector<uint32_t> rows;
        std::vector<int> row_smid;
        topo->max_smid = -1;
        for (int sm = 0; sm < SA_MAX_SM; ++sm) {
            if (!h_seen[sm]) continue;
            topo->max_smid = sm;
            row_smid.push_back(sm);
            rows.insert(rows.end(), h_lat.begin() + (size_t)sm * kNumAddr, h_lat.begin() + (size_t)(sm + 1) * kNumAddr);
        }
        sa_analyse_latency_matrix(rows, (int)row_smid.size(), row_smid, offsets, topo);
        topo->discovery_passes = pass + 1;
        if ((int)row_smid.size() >= topo->num_sms && topo->hash_usable && topo->confidence >= 0.95) break;
    }
    if ((e = cudaMemcpy(p->gpu_side_index, topo->side_index, SA_MAX_SM, cudaMemcpyHostToDevice)) != cudaSuccess) { sa_probe_destroy(p); return fail(e, "upload side index"); }
    if (!cache_path.empty() && topo->hash_usable) { // written whole or not at all: temporary name, then rename
        const std::string tmp = cache_path + ".tmp" + std::to_string((long long)getpid());
        if (FILE* f = std::fopen(tmp.c_str(), "wb")) {
            const std::string text = sa_topology_serialize(*topo, gpu_uuid, driver_version);
            const bool ok = std::fwrite(text.data(), 1, text.size(), f) == text.size();
            if (std::fclose(f) == 0 && ok) std::rename(tmp.c_str(), cache_path.c_str());
            else std::remove(tmp.c_str());
        }
    }
    *out = p;
    return cudaSuccess;
}

void sa_probe_destroy(SaProbeDevice* p) {
    if (!p) return;
    for (size_t i = 1; i < p->ring_blocks.size(); ++i) cudaFree(p->ring_blocks[i]);
    if (p->meta) cudaFree(p->meta);
    if (p->wait_errors_host) cudaFreeHost(p->wait_errors_host);
    delete p;
}

unsigned char* sa_probe_gpu_side_index(SaProbeDevice* p) { return p->gpu_side_index; }

// The ring of `stream`, made on first sight of the stream.  Called with ring_mu held.
static SaProbeDevice::Ring* ring_for_stream(SaProbeDevice* p, void* stream) {
    auto it = p->ring_of_stream.find(stream);
    if (it != p->ring_of_stream.end()) return it->second;
    if (p->idle_rings.empty()) {
        if ((int)p->rings.size() >= kMaxRings) {
            // More stream handles than rings (a program that keeps creating streams): once nothing
            // is running on the device every ring is idle and can be handed out again.
            if (cudaDeviceSynchronize() != cudaSuccess) return nullptr;
            p->ring_of_stream.clear();
            for (auto& r : p->rings) p->idle_rings.push_back(r.get());
        } else {
            // carve the next block (the first one came zeroed with the probe buffers)
            size_t block = p->rings.size() / kRingsPerBlock;
            if (block >= p->ring_blocks.size()) {
                void* mem = nullptr;
                if (cudaMalloc(&mem, kRingBlockBytes) != cudaSuccess) return nullptr;
                if (cudaMemset(mem, 0, kRingBlockBytes) != cudaSuccess) { cudaFree(mem); return nullptr; }
                p->ring_blocks.push_back((uint32_t*)mem);
            }
            for (int i = kRingsPerBlock - 1; i >= 0; --i) {
                std::unique_ptr<SaProbeDevice::Ring> r(new SaProbeDevice::Ring());
                r->base = p->ring_blocks[block] + (size_t)i * kRingSlots * kTicketStride;
                p->idle_rings.push_back(r.get());
                p->rings.push_back(std::move(r));
            }
        }
    }
    SaProbeDevice::Ring* r = p->idle_rings.back();
    p->idle_rings.pop_back();
    p->ring_of_stream.emplace(stream, r);
    return r;
}

uint32_t* sa_probe_ticket_slot(SaProbeDevice* p, void* stream, bool* may_overlap_predecessor) {
    std::lock_guard<std::mutex> lock(p->ring_mu);
    SaProbeDevice::Ring* r = ring_for_stream(p, stream);
    if (!r) return nullptr;
    unsigned n = r->next++;
    *may_overlap_predecessor = (n % kChainLength) != 0;
    return r->base + (size_t)(n % kRingSlots) * kTicketStride;
}

unsigned long long sa_probe_wait_timeouts(SaProbeDevice* p) {
    return p->wait_errors_host ? (unsigned long long)*(volatile uint32_t*)p->wait_errors_host : 0ull;
}

uint32_t* sa_probe_wait_error_word(SaProbeDevice* p) { return p->wait_errors_dev; }

cudaError_t sa_probe_sides(SaProbeDevice* p, const SaTopology& topo, const uint64_t* addrs, int n,
                           uint8_t* sides_out, cudaStream_t stream, int* ambiguous_out) {
    std::lock_guard<std::mutex> lock(p->mu);
    cudaError_t e;
    int ambiguous = 0;
    std::vector<uint32_t> lat((size_t)kVotes * kMaxBatch);
    std::vector<uint16_t> smid((size_t)kVotes * kMaxBatch);
    for (int done = 0; done < n; done += kMaxBatch) {
        int m = std::min(kMaxBatch, n - done);
        if ((e = cudaMemcpyAsync(p->addrs, addrs + done, sizeof(uint64_t) * m, cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e;
        int grid = std::min(m, 4 * std::max(1, topo.num_sms));
        if (grid < 2) grid = 2;
        sa_probe_addr_kernel<<<grid, 32, 0, stream>>>(p->addrs, m, kVotes, p->out_lat, p->out_smid, 0u, kProbeReps, kChain);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        if ((e = cudaMemcpyAsync(lat.data(), p->out_lat, sizeof(uint32_t) * kVotes * m, cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
        if ((e = cudaMemcpyAsync(smid.data(), p->out_smid, sizeof(uint16_t) * kVotes * m, cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return e;
        for (int i = 0; i < m; ++i) {
            int best_side = 0;
            double best_margin = -1.0;
            bool agree = true;
            int first = -1;
            for (int v = 0; v < kVotes; ++v) {
                int sm = smid[(size_t)v * m + i];
                if (sm >= SA_MAX_SM) sm = 0;
                uint32_t l = lat[(size_t)v * m + i];
                int far = l > topo.thr[sm];
                int side = (topo.side_index[sm] & 1) ^ far;
                double span = std::max(1.0, (double)topo.far_lat[sm] - (double)topo.near_lat[sm]);
                double margin = std::fabs((double)l - (double)topo.thr[sm]) / span;
                if (first < 0) first = side; else if (side != first) agree = false;
                if (margin > best_margin) { best_margin = margin; best_side = side; }
            }
            if (!agree) ++ambiguous;
            sides_out[done + i] = (uint8_t)best_side;
        }
    }
    if (ambiguous_out) *ambiguous_out = ambiguous;
    return cudaSuccess;
}
