// Topology discovery for one GPU: which L2 side every SM is nearest to, the
// XOR hash that flips the side inside a 2 MiB page, and the side of arbitrary
// addresses (physical pages, 4 KiB chunks) by latency probing.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "sa_sched.cuh"

struct SaTopology {
    int device = -1;
    int num_sms = 0;
    int sms_seen = 0;
    int discovery_passes = 0;     // probe kernel launches it took (more than 1 = the first pass left doubts)
    int max_smid = -1;
    uint8_t side_index[SA_MAX_SM] = {0}; // byte = side | ordinal << 1 (the reference's format, sideaware.cu:669-675)
    int count[2] = {0, 0};
    int min_per_side = 0;
    uint32_t hash = 0;            // toggling bits among address bits 4..20
    bool hash_usable = false;     // bit 12 set, nothing below, validated on random offsets
    int validation_offsets = 0;
    int validation_errors = 0;
    double confidence = 0.0;      // min over SMs of |hamming - n/2| / (n/2)
    uint32_t thr[SA_MAX_SM] = {0}, near_lat[SA_MAX_SM] = {0}, far_lat[SA_MAX_SM] = {0};
    std::string json;             // raw data for diagnostics
    bool from_cache = false;      // taken from a topology cache file (and confirmed by a spot check), not discovered
};

struct SaProbeDevice; // device-side buffers, opaque

// Allocates the probe buffers on `device` (which must be current) and runs discovery
// on `probe_page_va`, one zero-filled, 2 MiB aligned physical page owned by the caller.
// Returns cudaSuccess or the failing CUDA error; `why` receives a description.
cudaError_t sa_probe_create(int device, uint64_t probe_page_va, SaProbeDevice** out, SaTopology* topo, std::string* why);
void sa_probe_destroy(SaProbeDevice* p);

// Side (0/1) of each address in `addrs` (device-accessible memory that may hold
// live data; probing adds zero atomically and changes nothing).  Synchronous.
cudaError_t sa_probe_sides(SaProbeDevice* p, const SaTopology& topo, const uint64_t* addrs, int n,
                           uint8_t* sides_out, cudaStream_t stream, int* ambiguous_out);

// Device pointers owned by the probe object.
unsigned char* sa_probe_gpu_side_index(SaProbeDevice* p);
// Ticket slot for the next launch on `stream` (every stream has its own ring of slots), or nullptr if
// a ring could not be made.  *may_overlap_predecessor is false for the launches that have to wait for
// the end of their predecessor on the stream, so that the ring is never overrun.
uint32_t* sa_probe_ticket_slot(SaProbeDevice* p, void* stream, bool* may_overlap_predecessor);
// How many bounded waits inside kernels have run out so far on this device.  The kernels count into a
// word of pinned host memory, so this neither synchronises nor copies.
unsigned long long sa_probe_wait_timeouts(SaProbeDevice* p);
// Device address of that word, a parameter of every kernel that waits on an mbarrier.
uint32_t* sa_probe_wait_error_word(SaProbeDevice* p);

// Pure host analysis of a latency matrix lat[sm][addr] (exposed for CPU tests).
// offsets[j] is the byte offset of address j inside the probe page; offsets[0] == 0,
// offsets[1..17] == 1<<4 .. 1<<20, the rest are validation offsets.
void sa_analyse_latency_matrix(const std::vector<uint32_t>& lat, int num_rows, const std::vector<int>& row_smid,
                               const std::vector<uint32_t>& offsets, SaTopology* topo);

// Topology cache (text; pure functions, exposed for CPU tests).  A file is accepted only if it was written for the
// same GPU (UUID), driver version and SM count, is complete (checksum) and consistent in itself; the caller then
// confirms it by measurement before use.
std::string sa_topology_serialize(const SaTopology& t, const std::string& gpu_uuid, int driver_version);
bool sa_topology_parse(const std::string& text, const std::string& gpu_uuid, int driver_version, int num_sms,
                       SaTopology* out, std::string* why);
