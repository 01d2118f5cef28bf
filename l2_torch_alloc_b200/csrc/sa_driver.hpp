// CUDA driver entry points resolved at run time from libcuda.so.1, so the
// library can be loaded (and its symbols checked) on a machine without a GPU
// driver; the first call that needs the GPU fails with a clear message there.
#pragma once
#include <cuda.h>

#include <string>

struct SaDriver {
    CUresult (*GetErrorString)(CUresult, const char**);
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
    CUresult (*ModuleLoadData)(CUmodule*, const void*);
    CUresult (*ModuleUnload)(CUmodule);
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*);
    CUresult (*FuncGetAttribute)(int*, CUfunction_attribute, CUfunction);
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             CUstream, void**, void**);
    CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**);
};

// nullptr (and *why filled) when libcuda.so.1 or one of the symbols is missing.
const SaDriver* sa_driver(std::string* why);
std::string sa_cu_error(const SaDriver* d, CUresult r);
