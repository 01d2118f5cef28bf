// Host-side analysis of the discovery measurements (no CUDA calls in this file).
//
// Input: lat[sm][addr], the minimum latency of a short chain of dependent L2
// atomics from every SM to a set of addresses inside one 2 MiB physical page.
// An address is homed on one of two L2 sides; an SM sees it "near" or "far".
// Each SM therefore has a bimodal row, split at its own largest gap - no
// threshold is shared between SMs, so SMs with a longer path to their L2 do
// not get mislabelled.  The near/far pattern over the addresses is the SM's
// signature: SMs of one side share it, the other side sees the complement.
//
// The reference classifies SMs with one probe address and the mean latency of
// all SMs as the threshold (sideaware.cu:653-675) and derives the hash from one
// SM's single-bit probes (sideaware.cu:692-705); here every address gets a vote
// from every SM and the hash is validated on multi-bit offsets.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <sstream>

#include "sa_probe.hpp"

namespace {

struct RowSplit {
    uint32_t thr = 0, near_lat = 0, far_lat = 0;
    double quality = 0.0; // gap / (far - near), 0 when the row is not bimodal
};

RowSplit split_row(const uint32_t* v, int n) {
    RowSplit r;
    std::vector<uint32_t> s(v, v + n);
    std::sort(s.begin(), s.end());
    int lo = std::max(1, n / 8), hi = n - std::max(1, n / 8);
    uint32_t best_gap = 0;
    int best = -1;
    for (int i = lo; i <= hi && i < n; ++i) {
        uint32_t gap = s[i] - s[i - 1];
        if (gap > best_gap) { best_gap = gap; best = i; }
    }
    if (best < 0) return r;
    r.thr = s[best - 1] + best_gap / 2;
    r.near_lat = s[(best - 1) / 2];
    r.far_lat = s[best + (n - best) / 2];
    double span = (double)r.far_lat - (double)r.near_lat;
    // a real two-sided row has a gap that is a sizeable part of the near/far distance
    // and a far latency clearly above the near one
    if (span > 0 && (double)r.far_lat > 1.04 * (double)r.near_lat) r.quality = best_gap / span;
    return r;
}

} // namespace

void sa_analyse_latency_matrix(const std::vector<uint32_t>& lat, int num_rows, const std::vector<int>& row_smid,
                               const std::vector<uint32_t>& offsets, SaTopology* topo) {
    const int n = (int)offsets.size();
    SaTopology& T = *topo;
    T.sms_seen = num_rows;
    T.hash = 0;
    T.hash_usable = false;
    T.validation_errors = 0;
    T.validation_offsets = 0;
    T.confidence = 0.0;
    T.count[0] = T.count[1] = 0;
    for (int i = 0; i < SA_MAX_SM; ++i) { T.side_index[i] = 0; T.thr[i] = T.near_lat[i] = T.far_lat[i] = 0; }
    if (num_rows <= 0 || n < 18) return;

    std::vector<RowSplit> split(num_rows);
    std::vector<std::vector<uint8_t>> sig(num_rows, std::vector<uint8_t>(n, 0));
    for (int i = 0; i < num_rows; ++i) {
        split[i] = split_row(&lat[(size_t)i * n], n);
        for (int j = 0; j < n; ++j) sig[i][j] = lat[(size_t)i * n + j] > split[i].thr;
    }

    // first guess: compare every signature with the first well-split row
    int ref = 0;
    for (int i = 0; i < num_rows; ++i) if (split[i].quality > 0.25) { ref = i; break; }
    std::vector<uint8_t> side(num_rows, 0);
    for (int i = 0; i < num_rows; ++i) {
        int hd = 0;
        for (int j = 0; j < n; ++j) hd += sig[i][j] != sig[ref][j];
        side[i] = hd * 2 > n;
    }
    // address sides by vote of all SMs, then SM sides by vote of all addresses (two rounds)
    std::vector<uint8_t> addr_side(n, 0);
    std::vector<int> agree(num_rows, 0);
    for (int round = 0; round < 2; ++round) {
        for (int j = 0; j < n; ++j) {
            int votes = 0, total = 0;
            for (int i = 0; i < num_rows; ++i) {
                if (split[i].quality <= 0.0) continue;
                votes += side[i] ^ sig[i][j]; // near (sig 0) => the address is on the SM's own side
                ++total;
            }
            addr_side[j] = votes * 2 > total;
        }
        for (int i = 0; i < num_rows; ++i) {
            int as_side1 = 0;
            for (int j = 0; j < n; ++j) as_side1 += sig[i][j] ^ addr_side[j];
            side[i] = as_side1 * 2 > n;
            agree[i] = side[i] ? as_side1 : n - as_side1;
        }
    }
    // the lowest SM id defines side 0, as in the reference (sideaware.cu:662-664)
    if (side[0]) {
        for (auto& s : side) s ^= 1;
        for (auto& a : addr_side) a ^= 1;
    }

    double conf = 1.0;
    for (int i = 0; i < num_rows; ++i) {
        double c = split[i].quality > 0.0 ? (2.0 * agree[i] - n) / n : 0.0;
        conf = std::min(conf, c);
    }
    T.confidence = conf;

    // hash: single-bit offsets that land on the other side than offset 0
    uint32_t hash = 0;
    for (int j = 1; j <= 17 && j < n; ++j)
        if (addr_side[j] != addr_side[0]) hash |= offsets[j];
    T.hash = hash;
    for (int j = 18; j < n; ++j) {
        uint32_t predicted = addr_side[0] ^ sa_parity32(offsets[j] & hash);
        T.validation_offsets++;
        T.validation_errors += predicted != addr_side[j];
    }
    T.hash_usable = (hash & 4096u) && !(hash & 4095u) && T.validation_errors == 0 && conf > 0.5;

    // per-SM table in SM-id order
    int ord[2] = {0, 0};
    std::vector<int> row_of(SA_MAX_SM, -1);
    for (int i = 0; i < num_rows; ++i)
        if (row_smid[i] >= 0 && row_smid[i] < SA_MAX_SM) row_of[row_smid[i]] = i;
    int limit = std::max(T.num_sms, T.max_smid + 1);
    if (limit > SA_MAX_SM) limit = SA_MAX_SM;
    for (int sm = 0; sm < limit; ++sm) {
        int r = row_of[sm];
        // an SM that never ran a probe block is put on the less populated side
        int s = r >= 0 ? side[r] : (ord[0] <= ord[1] ? 0 : 1);
        int o = ord[s]++;
        T.side_index[sm] = (uint8_t)((s & 1) | ((o & 127) << 1));
        if (r >= 0) { T.thr[sm] = split[r].thr; T.near_lat[sm] = split[r].near_lat; T.far_lat[sm] = split[r].far_lat; }
    }
    T.count[0] = ord[0];
    T.count[1] = ord[1];
    T.min_per_side = std::min(ord[0], ord[1]);
    // SMs without a measurement inherit the median threshold so page probes from them still work
    std::vector<uint32_t> thrs, nears, fars;
    for (int sm = 0; sm < limit; ++sm) if (T.thr[sm]) { thrs.push_back(T.thr[sm]); nears.push_back(T.near_lat[sm]); fars.push_back(T.far_lat[sm]); }
    if (!thrs.empty()) {
        std::sort(thrs.begin(), thrs.end()); std::sort(nears.begin(), nears.end()); std::sort(fars.begin(), fars.end());
        for (int sm = 0; sm < SA_MAX_SM; ++sm)
            if (!T.thr[sm]) { T.thr[sm] = thrs[thrs.size() / 2]; T.near_lat[sm] = nears[nears.size() / 2]; T.far_lat[sm] = fars[fars.size() / 2]; }
    }

    std::ostringstream js;
    js << "{\"device\":" << T.device << ",\"num_sms\":" << T.num_sms << ",\"sms_seen\":" << num_rows
       << ",\"hash\":" << T.hash << ",\"hash_usable\":" << (T.hash_usable ? "true" : "false")
       << ",\"validation_offsets\":" << T.validation_offsets << ",\"validation_errors\":" << T.validation_errors
       << ",\"confidence\":" << T.confidence << ",\"side0\":" << T.count[0] << ",\"side1\":" << T.count[1]
       << ",\"offsets\":[";
    for (int j = 0; j < n; ++j) js << (j ? "," : "") << offsets[j];
    js << "],\"addr_side\":[";
    for (int j = 0; j < n; ++j) js << (j ? "," : "") << (int)addr_side[j];
    js << "],\"sm\":[";
    for (int i = 0; i < num_rows; ++i) {
        js << (i ? "," : "") << "{\"smid\":" << row_smid[i] << ",\"side\":" << (int)side[i] << ",\"thr\":" << split[i].thr
           << ",\"near\":" << split[i].near_lat << ",\"far\":" << split[i].far_lat << ",\"q\":" << split[i].quality
           << ",\"agree\":" << agree[i] << ",\"lat\":[";
        for (int j = 0; j < n; ++j) js << (j ? "," : "") << lat[(size_t)i * n + j];
        js << "]}";
    }
    js << "]}";
    T.json = js.str();
}

// ---------------------------------------------------------------------------
// Topology cache: what discovery found, as text, keyed by the GPU it was found on
// ---------------------------------------------------------------------------
// The reference probes every device on every start (sideaware.cu:837-868).  Discovery here takes a few
// milliseconds; a program that starts often can keep its result in a file.  A cached topology is only a
// CLAIM: the caller re-measures a handful of addresses against it before using it (sa_probe.cu), and the key
// (GPU UUID, driver version, SM count, format version) must match to the letter.
static const char kCacheMagic[] = "sideaware-topology-v1";

std::string sa_topology_serialize(const SaTopology& t, const std::string& gpu_uuid, int driver_version) {
    std::ostringstream o;
    o << kCacheMagic << "\n";
    o << "uuid " << gpu_uuid << "\n";
    o << "driver " << driver_version << "\n";
    o << "num_sms " << t.num_sms << "\n";
    o << "max_smid " << t.max_smid << "\n";
    o << "hash " << t.hash << "\n";
    o << "hash_usable " << (t.hash_usable ? 1 : 0) << "\n";
    o << "validation " << t.validation_offsets << " " << t.validation_errors << "\n";
    o << "confidence " << (long long)std::llround(t.confidence * 1e6) << "\n";
    o << "count " << t.count[0] << " " << t.count[1] << " " << t.min_per_side << "\n";
    unsigned long long sum = 0;
    for (int sm = 0; sm < SA_MAX_SM; ++sm) {
        o << "sm " << sm << " " << (int)t.side_index[sm] << " " << t.thr[sm] << " " << t.near_lat[sm] << " " << t.far_lat[sm] << "\n";
        sum = sum * 1000003ull + t.side_index[sm] + 7ull * t.thr[sm] + 13ull * t.near_lat[sm] + 17ull * t.far_lat[sm];
    }
    o << "check " << (sum ^ t.hash) << "\n";
    return o.str();
}

bool sa_topology_parse(const std::string& text, const std::string& gpu_uuid, int driver_version, int num_sms,
                       SaTopology* out, std::string* why) {
    auto fail = [&](const char* w) {
        if (why) *why = w;
        return false;
    };
    std::istringstream in(text);
    std::string word;
    if (!(in >> word) || word != kCacheMagic) return fail("not a topology cache file of this format");
    SaTopology t;
    std::string uuid;
    long long driver = -1, usable = -1, conf = -1;
    if (!(in >> word >> uuid) || word != "uuid") return fail("malformed (uuid)");
    if (uuid != gpu_uuid) return fail("written for another GPU");
    if (!(in >> word >> driver) || word != "driver") return fail("malformed (driver)");
    if (driver != driver_version) return fail("written under another driver version");
    if (!(in >> word >> t.num_sms) || word != "num_sms") return fail("malformed (num_sms)");
    if (t.num_sms != num_sms || num_sms <= 0 || num_sms > SA_MAX_SM) return fail("SM count differs");
    if (!(in >> word >> t.max_smid) || word != "max_smid" || t.max_smid < 0 || t.max_smid >= SA_MAX_SM) return fail("malformed (max_smid)");
    if (!(in >> word >> t.hash) || word != "hash") return fail("malformed (hash)");
    if (!(in >> word >> usable) || word != "hash_usable" || (usable != 0 && usable != 1)) return fail("malformed (hash_usable)");
    t.hash_usable = usable == 1;
    if (!(in >> word >> t.validation_offsets >> t.validation_errors) || word != "validation") return fail("malformed (validation)");
    if (!(in >> word >> conf) || word != "confidence" || conf < 0 || conf > 1000000) return fail("malformed (confidence)");
    t.confidence = conf / 1e6;
    if (!(in >> word >> t.count[0] >> t.count[1] >> t.min_per_side) || word != "count") return fail("malformed (count)");
    unsigned long long sum = 0;
    int ones = 0, zeros = 0;
    for (int sm = 0; sm < SA_MAX_SM; ++sm) {
        int idx = -1, side = -1;
        if (!(in >> word >> idx >> side >> t.thr[sm] >> t.near_lat[sm] >> t.far_lat[sm]) || word != "sm" || idx != sm || side < 0 || side > 255)
            return fail("malformed (per-SM line)");
        t.side_index[sm] = (uint8_t)side;
        if (sm <= t.max_smid) (side & 1 ? ones : zeros)++;
        sum = sum * 1000003ull + t.side_index[sm] + 7ull * t.thr[sm] + 13ull * t.near_lat[sm] + 17ull * t.far_lat[sm];
    }
    unsigned long long check = 0;
    if (!(in >> word >> check) || word != "check" || check != (sum ^ t.hash)) return fail("checksum mismatch (truncated or edited file)");
    // what the numbers claim must hang together before anything is measured against them
    if (t.count[0] + t.count[1] != t.num_sms || t.min_per_side != std::min(t.count[0], t.count[1])) return fail("SM counts do not add up");
    if (t.hash_usable && (!(t.hash & 4096u) || (t.hash & 4095u) || (t.hash & ~0x1FFFF0u))) return fail("hash marked usable but not of the required form");
    (void)ones;
    (void)zeros;
    t.json = "{\"from_cache\":true,\"num_sms\":" + std::to_string(t.num_sms) + ",\"sms_seen\":" + std::to_string(t.num_sms) +
             ",\"hash\":" + std::to_string(t.hash) + ",\"hash_usable\":" + (t.hash_usable ? "true" : "false") +
             ",\"side0\":" + std::to_string(t.count[0]) + ",\"side1\":" + std::to_string(t.count[1]) + "}";
    *out = t;
    return true;
}
