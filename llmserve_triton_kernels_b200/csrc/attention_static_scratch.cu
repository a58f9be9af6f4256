// The split-key attention with its scratch memory in a fixed device array, for callers that must
// not allocate (see attention_static_scratch.h for who they are, the limits and the rules).
#include "attention_static_scratch.h"

#include <stdio.h>

#include <mutex>

#include "common.cuh"

// The usual entry point (attention_mma.cu); this file only hands it other scratch pointers.
extern "C" int llm_attention_mma(const void* q, int q_stride, void* out, int out_stride, const void* pool,
                                 const int* page_table, int table_width, const int* token_request, const int* cu_tokens,
                                 const int* ctx_lens, int requests, int n_tokens, int H, int KV, int D, int page_size,
                                 int window, float scale, int max_rows_large, int have_small, int splits_small,
                                 int splits_large, float* scratch_o, float* scratch_ml, int* counters,
                                 cudaStream_t stream);

namespace {

// In host code these names are stand-ins, not device addresses: a kernel must be given what
// cudaGetSymbolAddress returns for them.
static __device__ __align__(256) float static_scratch_o[(size_t)LLM_STATIC_SCRATCH_MAX_ROWS * LLM_STATIC_SCRATCH_MAX_HEAD_DIM];
static __device__ __align__(256) float static_scratch_ml[(size_t)LLM_STATIC_SCRATCH_MAX_ROWS * 2];
static __device__ __align__(256) int static_counters[LLM_STATIC_SCRATCH_MAX_COUNTERS];

constexpr int MAX_DEVICES = 64;
struct DeviceScratch {
    float* o = nullptr;
    float* ml = nullptr;
    int* counters = nullptr;
    bool ready = false;
};
DeviceScratch per_device[MAX_DEVICES];
std::mutex setup_lock;
thread_local char last_error[256] = "";

// Once per device, with that device current: the arrays' addresses on it.
int scratch_of_current_device(DeviceScratch** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) {
        snprintf(last_error, sizeof last_error, "device %d is beyond the %d devices this entry point keeps track of", dev, MAX_DEVICES);
        return LLM_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> guard(setup_lock);
    DeviceScratch& s = per_device[dev];
    if (!s.ready) {
        if ((e = cudaGetSymbolAddress((void**)&s.o, static_scratch_o)) != cudaSuccess ||
            (e = cudaGetSymbolAddress((void**)&s.ml, static_scratch_ml)) != cudaSuccess ||
            (e = cudaGetSymbolAddress((void**)&s.counters, static_counters)) != cudaSuccess) {
            snprintf(last_error, sizeof last_error, "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return (int)e;
        }
        s.ready = true;
    }
    *out = &s;
    return 0;
}

}  // namespace

LLM_EXPORT const char* llm_attention_static_scratch_error(void) { return last_error; }

LLM_EXPORT int llm_attention_mma_static_scratch(const void* q, int q_stride, void* out, int out_stride, const void* pool,
                                                const int* page_table, int table_width, const int* token_request,
                                                const int* cu_tokens, const int* ctx_lens, int requests, int n_tokens,
                                                int H, int KV, int D, int page_size, int window, float scale,
                                                int max_rows_large, int have_small, int splits_small, int splits_large,
                                                cudaStream_t stream) {
    last_error[0] = 0;
    if (n_tokens <= 0 || requests <= 0) return 0;
    const long long rows = (long long)n_tokens * H * (splits_small > 0 ? splits_small : 1);
    if (splits_large != 1) {
        snprintf(last_error, sizeof last_error, "splits_large must be 1 with the fixed scratch array, got %d", splits_large);
        return LLM_STATIC_SCRATCH_TOO_LARGE;
    }
    if (rows > LLM_STATIC_SCRATCH_MAX_ROWS) {
        snprintf(last_error, sizeof last_error, "n_tokens * H * splits_small = %lld exceeds the fixed scratch array's %d rows", rows,
                 LLM_STATIC_SCRATCH_MAX_ROWS);
        return LLM_STATIC_SCRATCH_TOO_LARGE;
    }
    if (D > LLM_STATIC_SCRATCH_MAX_HEAD_DIM) {
        snprintf(last_error, sizeof last_error, "head size %d exceeds the fixed scratch array's %d", D, LLM_STATIC_SCRATCH_MAX_HEAD_DIM);
        return LLM_STATIC_SCRATCH_TOO_LARGE;
    }
    if ((long long)requests * KV > LLM_STATIC_SCRATCH_MAX_COUNTERS) {
        snprintf(last_error, sizeof last_error, "requests * KV = %lld exceeds the %d fixed counters", (long long)requests * KV,
                 LLM_STATIC_SCRATCH_MAX_COUNTERS);
        return LLM_STATIC_SCRATCH_TOO_LARGE;
    }
    DeviceScratch* s = nullptr;
    int code = scratch_of_current_device(&s);
    if (code) return code;
    // the counters must start at zero whatever an earlier (perhaps failed) call left in them
    cudaError_t e = cudaMemsetAsync(s->counters, 0, (size_t)requests * KV * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    return llm_attention_mma(q, q_stride, out, out_stride, pool, page_table, table_width, token_request, cu_tokens, ctx_lens,
                             requests, n_tokens, H, KV, D, page_size, window, scale, max_rows_large, have_small, splits_small,
                             splits_large, s->o, s->ml, s->counters, stream);
}
