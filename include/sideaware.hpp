// Type-safe C++ conveniences over sideaware.h, for code that used to #include the
// reference's sideaware.cu and its templated wrappers (sideaware.cu:1529-1571).
// Header only; link or dlopen sideaware.so as usual.  Unlike the reference's kernel
// wrappers (which `return` a void call and so cannot be instantiated), these compile.
#pragma once
#include <cstddef>

#include "sideaware.h"

namespace sideaware {

template <typename T>
inline sideaware_status_t malloc(T** dev_ptr, size_t bytes) {
    return ::sideaware_malloc(reinterpret_cast<void**>(dev_ptr), bytes);
}
template <typename T>
inline sideaware_status_t malloc_async(T** dev_ptr, size_t bytes, sideaware_stream_t stream = nullptr) {
    return ::sideaware_malloc_async(reinterpret_cast<void**>(dev_ptr), bytes, stream);
}
template <typename T>
inline sideaware_status_t free(T* ptr) {
    return ::sideaware_free(const_cast<void*>(static_cast<const void*>(ptr)));
}
template <typename T>
inline sideaware_status_t free_async(T* ptr, sideaware_stream_t stream = nullptr) {
    return ::sideaware_free_async(const_cast<void*>(static_cast<const void*>(ptr)), stream);
}

// Number of elements, not bytes: the byte count is derived from the element type.
template <typename T>
inline void memcpy(T* out, const T* in, size_t count, int device = 0, sideaware_stream_t stream = nullptr) {
    ::sideaware_memcpy(out, in, count * sizeof(T), device, stream);
}

template <typename Out, typename In>
inline void one_to_one(int kernel_id, Out* out0, const In* in0, size_t num_bytes_of_widest, int device = 0,
                       sideaware_stream_t stream = nullptr) {
    ::sideaware_one_to_one(kernel_id, num_bytes_of_widest, out0, in0, device, stream);
}

inline void elementwise(int kernel_id, size_t num_bytes, void* out0, void* out1 = nullptr, void* out2 = nullptr,
                        void* out3 = nullptr, const void* in0 = nullptr, const void* in1 = nullptr,
                        const void* in2 = nullptr, const void* in3 = nullptr, void* sideband_memory = nullptr,
                        int sideband_value = 0, int parallel_groups = 0, int forced_per_side = 0, int device = 0,
                        sideaware_stream_t stream = nullptr) {
    ::sideaware_elementwise(kernel_id, num_bytes, out0, out1, out2, out3, in0, in1, in2, in3, sideband_memory,
                            sideband_value, parallel_groups, forced_per_side, device, stream);
}

} // namespace sideaware

// The reference's own wrapper names, at global scope (sideaware.cu:1532-1547): a translation unit that used to
// `#include "sideaware.cu"` and call sideaware_malloc(&typed_pointer, bytes) inside cudaCheck(...) compiles unchanged
// against this header (example_llmc_rope.cu:265, :314 does exactly that).  Only where the CUDA runtime's types are
// known; the kernel launchers need no wrapper, their C declarations take any pointer.
#if defined(__CUDACC__) || defined(__CUDA_RUNTIME_H__) || defined(__CUDA_RUNTIME_API_H__)
template <typename T>
static inline cudaError_t sideaware_malloc(T** dev_ptr, size_t bytes) {
    return static_cast<cudaError_t>(::sideaware_malloc(reinterpret_cast<void**>(dev_ptr), bytes));
}
template <typename T>
static inline cudaError_t sideaware_malloc_async(T** dev_ptr, size_t bytes, cudaStream_t stream = 0) {
    return static_cast<cudaError_t>(::sideaware_malloc_async(reinterpret_cast<void**>(dev_ptr), bytes, stream));
}
template <typename T>
static inline cudaError_t sideaware_free(T* ptr) {
    return static_cast<cudaError_t>(::sideaware_free(const_cast<void*>(static_cast<const void*>(ptr))));
}
template <typename T>
static inline cudaError_t sideaware_free_async(T* ptr, cudaStream_t stream = 0) {
    return static_cast<cudaError_t>(::sideaware_free_async(const_cast<void*>(static_cast<const void*>(ptr)), stream));
}
#endif
