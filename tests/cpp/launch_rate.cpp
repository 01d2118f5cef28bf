// How fast short sideaware_memcpy calls follow one another when a C++ program issues them in a loop
// (a Python loop cannot: its own call overhead is several microseconds).  Works for any library with the
// reference's C ABI (sideaware.cu:1292, :1414); the path comes from the command line.  One line per size:
//   RATE <KiB> <host microseconds per call while issuing> <microseconds per call until the stream is empty>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>

typedef int (*malloc_fn)(void**, size_t);
typedef int (*free_fn)(void*);
typedef void (*memcpy_fn)(void*, const void*, size_t, int, cudaStream_t);

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    void* lib = dlopen(argv[1], RTLD_NOW);
    if (!lib) {
        std::printf("dlopen: %s\n", dlerror());
        return 1;
    }
    malloc_fn sa_malloc = (malloc_fn)dlsym(lib, "sideaware_malloc");
    free_fn sa_free = (free_fn)dlsym(lib, "sideaware_free");
    memcpy_fn sa_memcpy = (memcpy_fn)dlsym(lib, "sideaware_memcpy");
    if (!sa_malloc || !sa_free || !sa_memcpy) return 1;
    if (cudaSetDevice(0) != cudaSuccess || cudaFree(0) != cudaSuccess) return 1;
    void *a = nullptr, *b = nullptr;
    if (sa_malloc(&a, 64u << 20) || sa_malloc(&b, 64u << 20)) return 1;
    cudaStream_t s;
    cudaStreamCreate(&s);
    const size_t sizes[] = {size_t(64) << 10, size_t(1) << 20, size_t(4) << 20, size_t(16) << 20};
    for (size_t bytes : sizes) {
        for (int i = 0; i < 200; ++i) sa_memcpy(b, a, bytes, 0, s);
        cudaStreamSynchronize(s);
        const int n = 20000;
        auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < n; ++i) sa_memcpy(b, a, bytes, 0, s);
        auto t1 = std::chrono::steady_clock::now();
        cudaStreamSynchronize(s);
        auto t2 = std::chrono::steady_clock::now();
        std::printf("RATE %zu %.3f %.3f\n", bytes >> 10, std::chrono::duration<double, std::micro>(t1 - t0).count() / n,
                    std::chrono::duration<double, std::micro>(t2 - t0).count() / n);
    }
    cudaStreamDestroy(s);
    sa_free(a);
    sa_free(b);
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : 1;
}
