// A timeline of the decode kernels, for profiling builds only (compiled in with -DLLM_TIMELINE, which the build
// adds when the environment variable LLMSERVE_B200_TIMELINE is set; absent otherwise).  Thread 0 of every CTA
// stamps the global timer at up to six points of a kernel and leaves one record per CTA in a buffer of the
// translation unit; the host reads and clears the buffer through the reader that TL_DEFINE_READER exports.
#pragma once

#ifdef LLM_TIMELINE
#include "common.cuh"

namespace tl {
constexpr unsigned CAP = 1u << 16;
struct Rec {
    unsigned long long t[6];
    int kernel, launch, block, sm, a, b;
};
static __device__ Rec g_recs[CAP];
static __device__ unsigned g_count;
__device__ __forceinline__ unsigned long long now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ int smid() {
    int s;
    asm volatile("mov.u32 %0, %%smid;\n" : "=r"(s));
    return s;
}
struct Marks {
    unsigned long long t[6];
    __device__ __forceinline__ Marks() {
#pragma unroll
        for (int i = 0; i < 6; ++i) t[i] = 0;
        t[0] = now();
    }
    __device__ __forceinline__ void mark(int i) { t[i] = now(); }
    __device__ __forceinline__ void write(int kernel, int launch, int block, int a, int b) {
        const unsigned at = atomicAdd(&g_count, 1u);
        if (at >= CAP) return;
        Rec r;
#pragma unroll
        for (int i = 0; i < 6; ++i) r.t[i] = t[i];
        r.kernel = kernel; r.launch = launch; r.block = block; r.sm = smid(); r.a = a; r.b = b;
        g_recs[at] = r;
    }
};
}  // namespace tl

// Exports `name(void* host_buffer, unsigned capacity_records) -> records copied`; clears the buffer.
#define TL_DEFINE_READER(name)                                                                          \
    LLM_EXPORT int name(void* out, unsigned capacity) {                                                 \
        unsigned n = 0;                                                                                 \
        cudaDeviceSynchronize();                                                                        \
        cudaMemcpyFromSymbol(&n, tl::g_count, sizeof(n));                                               \
        if (n > tl::CAP) n = tl::CAP;                                                                   \
        if (n > capacity) n = capacity;                                                                 \
        if (n && out) cudaMemcpyFromSymbol(out, tl::g_recs, (size_t)n * sizeof(tl::Rec));               \
        const unsigned zero = 0;                                                                        \
        cudaMemcpyToSymbol(tl::g_count, &zero, sizeof(zero));                                           \
        return (int)n;                                                                                  \
    }
#define TL(...) __VA_ARGS__
#else
#define TL(...)
#define TL_DEFINE_READER(name)
#endif
