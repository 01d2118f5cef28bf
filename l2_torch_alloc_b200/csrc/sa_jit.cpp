#include "sa_jit.hpp"

#include <dlfcn.h>
#include <unistd.h>

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "sa_context.hpp"
#include "sa_kernels.hpp"

#include "_gen/sa_embedded_sources.inc" // kSaSchedSource, kSaJitTemplateSource

namespace {

// ---- NVRTC, resolved at run time ------------------------------------------
typedef struct _nvrtcProgram* nvrtcProgram;
struct Nvrtc {
    int (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
    int (*CompileProgram)(nvrtcProgram, int, const char* const*);
    int (*GetProgramLogSize)(nvrtcProgram, size_t*);
    int (*GetProgramLog)(nvrtcProgram, char*);
    int (*GetCUBINSize)(nvrtcProgram, size_t*);
    int (*GetCUBIN)(nvrtcProgram, char*);
    int (*DestroyProgram)(nvrtcProgram*);
    const char* (*GetErrorString)(int);
};
Nvrtc g_nvrtc;
bool g_nvrtc_ok = false;
std::string g_nvrtc_why;
std::once_flag g_nvrtc_once;

void load_nvrtc() {
    const char* names[] = {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so.13", "libnvrtc.so"};
    void* h = nullptr;
    if (const char* p = std::getenv("SIDEAWARE_NVRTC")) h = dlopen(p, RTLD_NOW);
    for (const char* n : names) {
        if (h) break;
        h = dlopen(n, RTLD_NOW);
    }
    if (!h) { g_nvrtc_why = "cannot load libnvrtc (set SIDEAWARE_NVRTC to its path)"; return; }
    bool ok = true;
    auto sym = [&](const char* name) {
        void* p = dlsym(h, name);
        if (!p) { ok = false; g_nvrtc_why = std::string("libnvrtc lacks ") + name; }
        return p;
    };
#define SA_SYM(field, name) g_nvrtc.field = reinterpret_cast<decltype(g_nvrtc.field)>(sym(name))
    SA_SYM(CreateProgram, "nvrtcCreateProgram");
    SA_SYM(CompileProgram, "nvrtcCompileProgram");
    SA_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize");
    SA_SYM(GetProgramLog, "nvrtcGetProgramLog");
    SA_SYM(GetCUBINSize, "nvrtcGetCUBINSize");
    SA_SYM(GetCUBIN, "nvrtcGetCUBIN");
    SA_SYM(DestroyProgram, "nvrtcDestroyProgram");
    SA_SYM(GetErrorString, "nvrtcGetErrorString");
#undef SA_SYM
    g_nvrtc_ok = ok;
}

std::string cuda_include_dir() {
    std::vector<std::string> cands;
    if (const char* p = std::getenv("SIDEAWARE_CUDA_INCLUDE")) cands.push_back(p);
    for (const char* env : {"CUDA_HOME", "CUDA_PATH"})
        if (const char* p = std::getenv(env)) cands.push_back(std::string(p) + "/include");
    cands.push_back("/usr/local/cuda/include");
    for (auto& c : cands)
        if (access((c + "/cuda_fp16.h").c_str(), R_OK) == 0) return c;
    return "/usr/local/cuda/include";
}

// ---- registry ---------------------------------------------------------------
struct Header { std::string text; int groups; };
std::mutex g_reg_mu;
std::vector<Header> g_headers{Header{"", 4}}; // id 0 = memcpy
std::unordered_map<std::string, int> g_ids;

} // namespace

struct SaJitDeviceCache {
    struct Entry {
        CUmodule mod[2] = {nullptr, nullptr};
        CUfunction fn[2] = {nullptr, nullptr};
        int max_threads[2] = {0, 0};
        std::string error[2];
    };
    std::vector<Entry> entries;
};

SaJitDeviceCache* sa_jit_new_device_cache() { return new SaJitDeviceCache(); }
void sa_jit_delete_device_cache(SaJitDeviceCache* c) { delete c; }

// Constructs that the reference's launch shape allowed and this one does not: blocks here are one-dimensional
// (the reference launches (256, groups), sideaware.cu:1407), one WARP owns a 4 KiB chunk and different warps take
// different numbers of chunks, so a barrier across a 256-thread group or the block can neither be reached by all
// its threads nor does it delimit a chunk.
std::string sa_jit_contract_warnings(const char* header) {
    std::string text(header ? header : ""), out;
    for (const char* word : {"threadIdx.y", "blockDim.y", "__syncthreads", "bar.sync", "barrier.sync"})
        if (text.find(word) != std::string::npos) {
            if (!out.empty()) out += ", ";
            out += word;
        }
    if (out.empty()) return out;
    return "warning: the functor header uses " + out + "; blocks are one-dimensional here, a warp (not a 256-thread group) owns a "
           "4 KiB chunk and warps take different numbers of chunks, so group-wide indexing or barriers inside "
           "vector_op / elementwise_op / indexing do not work as under the reference's (256, groups) launch";
}

int sa_jit_register(const char* header, int default_groups) {
    std::lock_guard<std::mutex> lock(g_reg_mu);
    std::string text(header);
    auto it = g_ids.find(text);
    if (it != g_ids.end()) return it->second;
    const std::string warn = sa_jit_contract_warnings(header);
    if (!warn.empty()) std::fprintf(stderr, "sideaware: %s\n", warn.c_str());
    int id = (int)g_headers.size();
    g_headers.push_back(Header{text, default_groups > 0 ? (default_groups > 4 ? 4 : default_groups) : 4});
    g_ids.emplace(std::move(text), id);
    return id;
}

int sa_jit_num_kernels() {
    std::lock_guard<std::mutex> lock(g_reg_mu);
    return (int)g_headers.size();
}

int sa_jit_default_groups(int id) {
    std::lock_guard<std::mutex> lock(g_reg_mu);
    return (id >= 0 && id < (int)g_headers.size()) ? g_headers[id].groups : 4;
}

// The translation unit for one functor: the four definitions the reference prepends
// (sideaware.cu:786-795), the user's header, the scheduler and the kernel template.
static std::string build_source(const std::string& header, int num_sms, uint32_t hash, bool wide, bool batch_as_written) {
    std::string src;
    if (batch_as_written) src += "#define SA_BATCH_AS_WRITTEN 1\n";
    src += "#define MAX_SM " + std::to_string(num_sms) + "\n";
    src += "#define HASH " + std::to_string((hash | (1u << 21)) / 16u) + "\n";
    src += wide ? "using size_type = long long;\nconstexpr bool aligned_2MiB = false;\n"
                : "using size_type = int;\nconstexpr bool aligned_2MiB = true;\n";
    src += "#line 1 \"functor_header\"\n";
    src += header;
    src += "\n#line 1 \"sa_sched.cuh\"\n";
    src += kSaSchedSource;
    src += "\n#line 1 \"sa_jit_template.cuh\"\n";
    src += kSaJitTemplateSource;
    return src;
}

// NVRTC for sm_100a only.  Returns false and fills *why (with the compiler log) on failure.
static bool nvrtc_compile(const std::string& src, int id, bool wide, std::vector<char>* cubin, std::string* why,
                          long* spill_bytes = nullptr) {
    std::call_once(g_nvrtc_once, load_nvrtc);
    if (!g_nvrtc_ok) { *why = g_nvrtc_why; return false; }
    std::string inc = "-I" + cuda_include_dir();
    const char* opts[] = {"--gpu-architecture=sm_100a", "--generate-line-info", "-use_fast_math", "-std=c++17",
                          "--ptxas-options=-v", inc.c_str()};
    nvrtcProgram prog = nullptr;
    int rc = g_nvrtc.CreateProgram(&prog, src.c_str(), "side_aware.cu", 0, nullptr, nullptr);
    if (rc != 0) { *why = std::string("nvrtcCreateProgram: ") + g_nvrtc.GetErrorString(rc); return false; }
    rc = g_nvrtc.CompileProgram(prog, (int)(sizeof(opts) / sizeof(opts[0])), opts);
    std::string log;
    size_t log_size = 0;
    if (g_nvrtc.GetProgramLogSize(prog, &log_size) == 0 && log_size > 1) {
        log.resize(log_size);
        g_nvrtc.GetProgramLog(prog, &log[0]);
    }
    std::string log_file;
    {
        std::lock_guard<std::mutex> lock(sa_config().mu);
        log_file = sa_config().log_file;
    }
    if (!log_file.empty()) {
        if (FILE* f = std::fopen(log_file.c_str(), "a")) {
            std::time_t now = std::time(nullptr);
            char stamp[64];
            std::strftime(stamp, sizeof(stamp), "%F %T", std::localtime(&now));
            std::fprintf(f, "==== side-aware functor %d (%s indexing) compiled %s: %s ====\n%s\n---- source ----\n%s\n==== end ====\n",
                         id, wide ? "64-bit" : "32-bit", stamp, rc == 0 ? "ok" : g_nvrtc.GetErrorString(rc), log.c_str(), src.c_str());
            std::fclose(f);
        }
    }
    if (spill_bytes) { // "... N bytes spill stores, M bytes spill loads" in the ptxas part of the log
        *spill_bytes = 0;
        size_t pos = 0;
        while ((pos = log.find(" bytes spill stores", pos)) != std::string::npos) {
            size_t b = pos;
            while (b > 0 && std::isdigit((unsigned char)log[b - 1])) --b;
            *spill_bytes += std::atol(log.substr(b, pos - b).c_str());
            pos += 10;
        }
    }
    if (rc != 0) {
        *why = std::string("NVRTC compilation failed (") + g_nvrtc.GetErrorString(rc) + "):\n" + log;
        g_nvrtc.DestroyProgram(&prog);
        return false;
    }
    if (!log.empty() && std::getenv("SIDEAWARE_VERBOSE")) std::fprintf(stderr, "sideaware: NVRTC log for functor %d:\n%s\n", id, log.c_str());
    size_t cubin_size = 0;
    g_nvrtc.GetCUBINSize(prog, &cubin_size);
    cubin->resize(cubin_size);
    rc = g_nvrtc.GetCUBIN(prog, cubin->data());
    g_nvrtc.DestroyProgram(&prog);
    if (rc != 0 || cubin_size == 0) { *why = "nvrtcGetCUBIN failed"; return false; }
    return true;
}

bool sa_jit_compile_only(const char* header, bool wide, std::string* why) {
    std::vector<char> cubin;
    return nvrtc_compile(build_source(header ? header : "", 148, 0x1EF000u, wide, false), -1, wide, &cubin, why);
}

static bool compile_variant(SaDevice* dev, int id, bool wide, CUfunction* fn_out, CUmodule* mod_out, std::string* why) {
    std::string header;
    {
        std::lock_guard<std::mutex> lock(g_reg_mu);
        header = g_headers[id].text;
    }
    std::vector<char> cubin;
    long spills = 0;
    if (!nvrtc_compile(build_source(header, dev->topo.num_sms, dev->topo.hash, wide, false), id, wide, &cubin, why, &spills)) return false;
    if (spills > 0) {
        // the widened batch does not fit the register budget of this functor: use the batch the header asks for
        std::vector<char> narrow;
        std::string why2;
        long spills2 = 0;
        if (nvrtc_compile(build_source(header, dev->topo.num_sms, dev->topo.hash, wide, true), id, wide, &narrow, &why2, &spills2) &&
            spills2 < spills)
            cubin.swap(narrow);
    }
    CUresult r = dev->drv->ModuleLoadData(mod_out, cubin.data());
    if (r != CUDA_SUCCESS) { *why = "cuModuleLoadData: " + sa_cu_error(dev->drv, r); return false; }
    r = dev->drv->ModuleGetFunction(fn_out, *mod_out, "sideaware_elementwise");
    if (r != CUDA_SUCCESS) {
        dev->drv->ModuleUnload(*mod_out);
        *mod_out = nullptr;
        *why = "cuModuleGetFunction(sideaware_elementwise): " + sa_cu_error(dev->drv, r);
        return false;
    }
    dev->jit_compiles.fetch_add(1);
    return true;
}

static CUfunction get_function(SaDevice* dev, int id, bool wide, std::string* why) {
    if (id <= 0 || id >= sa_jit_num_kernels()) { *why = "kernel id " + std::to_string(id) + " is not a registered functor"; return nullptr; }
    std::lock_guard<std::mutex> lock(dev->jit_mu);
    auto& entries = dev->jit->entries;
    if ((int)entries.size() <= id) entries.resize(id + 1);
    auto& e = entries[id];
    int v = wide ? 1 : 0;
    if (e.fn[v]) return e.fn[v];
    if (!e.error[v].empty()) { *why = e.error[v]; return nullptr; }
    SaScopedDevice guard(dev->id);
    if (!compile_variant(dev, id, wide, &e.fn[v], &e.mod[v], why)) {
        e.error[v] = *why;
        e.fn[v] = nullptr;
        return nullptr;
    }
    return e.fn[v];
}

int sa_jit_max_threads(SaDevice* dev, int id, bool wide, std::string* why) {
    CUfunction fn = get_function(dev, id, wide, why);
    if (!fn) return 0;
    std::lock_guard<std::mutex> lock(dev->jit_mu);
    int& cached = dev->jit->entries[id].max_threads[wide ? 1 : 0];
    if (cached == 0) {
        int v = 0;
        CUresult r = dev->drv->FuncGetAttribute(&v, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, fn);
        if (r != CUDA_SUCCESS || v <= 0) { *why = "cuFuncGetAttribute: " + sa_cu_error(dev->drv, r); return 0; }
        cached = v;
    }
    return cached;
}

bool sa_jit_precompile(SaDevice* dev, int id, std::string* why) {
    return get_function(dev, id, false, why) != nullptr && get_function(dev, id, true, why) != nullptr;
}

namespace {
struct ArgsNarrow { int num_vecs; void* out[4]; const void* in[4]; int* mem; int val; };
struct ArgsWide { long long num_vecs; void* out[4]; const void* in[4]; int* mem; int val; };
} // namespace

cudaError_t sa_jit_launch(SaDevice* dev, int id, bool wide, const SaSched& sched, int grid, int threads,
                          unsigned long long num_vecs, void* const out[4], const void* const in[4],
                          void* mem, int val, cudaStream_t stream, std::string* why) {
    CUfunction fn = get_function(dev, id, wide, why);
    if (!fn) return cudaErrorInvalidKernelImage;
    SaSched s = sched;
    ArgsNarrow an;
    ArgsWide aw;
    SaSideTable sides = dev->side_table;
    void* params[3] = {&s, &sides, nullptr};
    if (wide) {
        aw.num_vecs = (long long)num_vecs;
        for (int i = 0; i < 4; ++i) { aw.out[i] = out[i]; aw.in[i] = in[i]; }
        aw.mem = (int*)mem;
        aw.val = val;
        params[2] = &aw;
    } else {
        an.num_vecs = (int)num_vecs;
        for (int i = 0; i < 4; ++i) { an.out[i] = out[i]; an.in[i] = in[i]; }
        an.mem = (int*)mem;
        an.val = val;
        params[2] = &an;
    }
    // same launch attribute as the ahead-of-time kernels (SaLaunch)
    CUlaunchConfig cfg{};
    cfg.gridDimX = (unsigned)grid; cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = (unsigned)threads; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = 0;
    cfg.hStream = (CUstream)stream;
    CUlaunchAttribute attr[1];
    attr[0].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr[0].value.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (sa_pdl_enabled() && s.overlap) ? 1 : 0;
    CUresult r = dev->drv->LaunchKernelEx(&cfg, fn, params, nullptr);
    if (r != CUDA_SUCCESS) {
        *why = "cuLaunchKernelEx: " + sa_cu_error(dev->drv, r);
        return cudaErrorLaunchFailure;
    }
    return cudaSuccess;
}
