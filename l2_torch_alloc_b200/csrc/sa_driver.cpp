#include "sa_driver.hpp"

#include <dlfcn.h>

#include <mutex>

namespace {
SaDriver g_driver;
bool g_ok = false;
std::string g_why;
std::once_flag g_once;

void load() {
    void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        g_why = "sideaware: cannot load libcuda.so.1 (no NVIDIA driver on this machine); this library has no CPU path";
        return;
    }
    bool ok = true;
    auto sym = [&](const char* name) -> void* {
        void* p = dlsym(h, name);
        if (!p) { ok = false; g_why = std::string("sideaware: libcuda.so.1 lacks ") + name; }
        return p;
    };
#define SA_SYM(field, name) g_driver.field = reinterpret_cast<decltype(g_driver.field)>(sym(name))
    SA_SYM(GetErrorString, "cuGetErrorString");
    SA_SYM(DeviceGetAttribute, "cuDeviceGetAttribute");
    SA_SYM(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    SA_SYM(MemCreate, "cuMemCreate");
    SA_SYM(MemRelease, "cuMemRelease");
    SA_SYM(MemAddressReserve, "cuMemAddressReserve");
    SA_SYM(MemAddressFree, "cuMemAddressFree");
    SA_SYM(MemMap, "cuMemMap");
    SA_SYM(MemUnmap, "cuMemUnmap");
    SA_SYM(MemSetAccess, "cuMemSetAccess");
    SA_SYM(ModuleLoadData, "cuModuleLoadData");
    SA_SYM(ModuleUnload, "cuModuleUnload");
    SA_SYM(ModuleGetFunction, "cuModuleGetFunction");
    SA_SYM(FuncGetAttribute, "cuFuncGetAttribute");
    SA_SYM(LaunchKernel, "cuLaunchKernel");
    SA_SYM(LaunchKernelEx, "cuLaunchKernelEx");
#undef SA_SYM
    g_ok = ok;
}
} // namespace

const SaDriver* sa_driver(std::string* why) {
    std::call_once(g_once, load);
    if (!g_ok) {
        if (why) *why = g_why;
        return nullptr;
    }
    return &g_driver;
}

std::string sa_cu_error(const SaDriver* d, CUresult r) {
    const char* s = nullptr;
    if (d && d->GetErrorString) d->GetErrorString(r, &s);
    return std::string(s ? s : "unknown driver error") + " (CUresult " + std::to_string((int)r) + ")";
}
