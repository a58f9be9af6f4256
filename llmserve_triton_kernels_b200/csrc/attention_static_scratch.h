/* A second way into the split-key attention for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference project: it exists for the programs that
 * embed this library and are not allowed to call cudaMalloc on their hot path — a serving loop
 * that has handed all device memory to its own pool, code running inside a region where the
 * allocator is locked (a stream capture owned by someone else, a real-time thread), or a host
 * language binding that can pass pointers but has no allocator to offer.  The usual entry point,
 * llm_attention_mma, takes its scratch memory (the splits' partial results, their running
 * maxima and sums, and the counters that tell which split finished last) from the caller, who
 * has to get it from somewhere.  This one brings its own: a fixed array that lives in the
 * library's device image.
 *
 * What to know before using it:
 *   - Limits.  n_tokens * H * splits_small <= LLM_STATIC_SCRATCH_MAX_ROWS (16384),
 *     D <= LLM_STATIC_SCRATCH_MAX_HEAD_DIM (128), requests * KV <= LLM_STATIC_SCRATCH_MAX_COUNTERS
 *     (4096), splits_large == 1.  Beyond them the call returns LLM_STATIC_SCRATCH_TOO_LARGE and
 *     launches nothing; llm_attention_static_scratch_error() then says which limit it was.
 *   - Cost.  About 8.3 MB of device memory on every GPU that loads the library, held until the
 *     process exits, whether or not this entry point is ever called.
 *   - First call.  The first call on a device looks the array's device address up
 *     (cudaGetSymbolAddress) with that device current.  Make that call before any stream capture
 *     begins; later calls on the device do no set-up.
 *   - Sharing.  All calls on a device share the one array.  Two calls whose kernels overlap on
 *     the GPU (different streams, or graphs replayed side by side) race on it and give wrong
 *     results; calls on one stream are safe.  The array keeps what the last call left in it; the
 *     counters, which must start at zero, are cleared on the given stream before every launch.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine.
 *
 * Arguments and result are those of llm_attention_mma without the three scratch pointers. */
#pragma once

#include <cuda_runtime.h>

#define LLM_STATIC_SCRATCH_MAX_ROWS 16384
#define LLM_STATIC_SCRATCH_MAX_HEAD_DIM 128
#define LLM_STATIC_SCRATCH_MAX_COUNTERS 4096
#define LLM_STATIC_SCRATCH_TOO_LARGE 10003

#ifdef __cplusplus
extern "C" {
#endif

int llm_attention_mma_static_scratch(const void* q, int q_stride, void* out, int out_stride, const void* pool,
                                     const int* page_table, int table_width, const int* token_request,
                                     const int* cu_tokens, const int* ctx_lens, int requests, int n_tokens, int H, int KV,
                                     int D, int page_size, int window, float scale, int max_rows_large, int have_small,
                                     int splits_small, int splits_large, cudaStream_t stream);

/* The reason of the last LLM_STATIC_SCRATCH_TOO_LARGE (or set-up failure) on this thread, as text. */
const char* llm_attention_static_scratch_error(void);

#ifdef __cplusplus
}
#endif
