// Run-time compilation of user functor headers (NVRTC, sm_100a only) and the
// registry that maps a header text to a kernel id.
// Replaces compileStringToCUBIN / loadCUBIN / sideaware_get_kernel /
// sideaware_create_kernel_advanced of the reference (sideaware.cu:524-607,
// :772-813, :1421-1458).  Kernel id 0 is the built-in memcpy and never compiled here.
#pragma once
#include <cuda_runtime.h>

#include <string>

#include "sa_sched.cuh"

struct SaDevice;
struct SaJitDeviceCache;

SaJitDeviceCache* sa_jit_new_device_cache();
void sa_jit_delete_device_cache(SaJitDeviceCache*);

// Registers `header` (or finds it) and returns its id >= 1.  The registry is process
// wide, so ids are identical on every device.
int sa_jit_register(const char* header, int default_groups);
int sa_jit_num_kernels();         // ids 0 .. n-1 are valid
int sa_jit_default_groups(int id);

// Compiles (first use) and launches functor `id` on `dev`; `wide` selects 64-bit indexing.
// On failure returns a CUDA error number and fills *why.
cudaError_t sa_jit_launch(SaDevice* dev, int id, bool wide, const SaSched& sched, int grid, int threads,
                          unsigned long long num_vecs, void* const out[4], const void* const in[4],
                          void* mem, int val, cudaStream_t stream, std::string* why);
// Most threads per block the compiled functor can be launched with (its LAUNCH_BOUNDS and register use decide);
// compiles on first use.  0 (and *why) on failure.
int sa_jit_max_threads(SaDevice* dev, int id, bool wide, std::string* why);
// Compiles both variants now; false (and *why) on failure.
bool sa_jit_precompile(SaDevice* dev, int id, std::string* why);
// "" or one line naming the constructs in `header` that do not carry over from the reference's launch shape.
std::string sa_jit_contract_warnings(const char* header);
// Compiles `header` for sm_100a without loading it (no GPU needed); for build-time checks.
bool sa_jit_compile_only(const char* header, bool wide, std::string* why);
