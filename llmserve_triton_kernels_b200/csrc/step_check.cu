// Checked mode: the integer arrays of a step, looked over ON THE DEVICE before the kernels that index with them.
//
// A wrong entry of a page table or a slot map makes an attention kernel read, or a cache write land in, memory that is
// not the request's; the tools that would show it (a memory checker) are not always at hand.  In checked mode every step
// starts with these kernels: they only read the step's arrays (never the cache or a weight), compare every index with its
// limit and every slot with the page table it must agree with, record the FIRST violation in a status record in pinned
// host memory, and overwrite the bad entry with a harmless one (index 0) so that the kernels after them touch nothing out
// of bounds.  The host reads the record after the step and raises.  The arrays are checked where the kernels read them:
// after their copy to the device, inside a captured graph too, and with token ids that a sampler left on the device
// and the host never saw.  The reference's guard is on the host only (src/llmserve/kvcache/paged.py:59-60).
#include "common.cuh"

namespace {

// status: [0] code of the first violation (0 = none), [1] page group or -1, [2] index into the array, [3] the value
// found, [4] the limit it broke, [5] number of violations seen
__device__ __forceinline__ void report(int* status, int code, int group, int index, int value, int limit) {
    atomicAdd(&status[5], 1);
    if (atomicCAS(&status[0], 0, code) == 0) {
        status[1] = group;
        status[2] = index;
        status[3] = value;
        status[4] = limit;
    }
}

enum {
    BAD_TOKEN_ID = 1, BAD_POSITION = 2, BAD_TOKEN_REQUEST = 3, BAD_CU_TOKENS = 4, BAD_CONTEXT_LEN = 5, BAD_LOGIT_ROW = 6,
    BAD_STATE_SLOT = 7, BAD_PAGE = 8, BAD_SLOT = 9, TABLE_TOO_NARROW = 10,
};

__global__ void check_step_arrays_kernel(int* token_ids, int* positions, int* token_request, const int* cu_tokens, int* ctx_lens,
                                         int* logit_rows, int* state_slots, int N, int R, int P, int vocab, int max_positions,
                                         int state_slot_count, int* status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) {
        if ((unsigned)token_ids[i] >= (unsigned)vocab) { report(status, BAD_TOKEN_ID, -1, i, token_ids[i], vocab); token_ids[i] = 0; }
        if ((unsigned)positions[i] >= (unsigned)max_positions) { report(status, BAD_POSITION, -1, i, positions[i], max_positions); positions[i] = 0; }
        int r = token_request[i];
        if ((unsigned)r >= (unsigned)R) { report(status, BAD_TOKEN_REQUEST, -1, i, r, R); token_request[i] = r = 0; }
        if (i < cu_tokens[r] || i >= cu_tokens[r + 1]) report(status, BAD_TOKEN_REQUEST, -1, i, r, R);
    }
    if (i < R) {
        const int q = cu_tokens[i + 1] - cu_tokens[i];
        if (q < 1 || cu_tokens[i] < 0 || cu_tokens[i + 1] > N) report(status, BAD_CU_TOKENS, -1, i, cu_tokens[i + 1], N);
        if (ctx_lens[i] < q || ctx_lens[i] > max_positions) { report(status, BAD_CONTEXT_LEN, -1, i, ctx_lens[i], max_positions); ctx_lens[i] = q > 0 ? q : 1; }
        if (state_slot_count > 0 && (unsigned)state_slots[i] >= (unsigned)state_slot_count) { report(status, BAD_STATE_SLOT, -1, i, state_slots[i], state_slot_count); state_slots[i] = 0; }
        if (i == 0 && (cu_tokens[0] != 0 || cu_tokens[R] != N)) report(status, BAD_CU_TOKENS, -1, R, cu_tokens[R], N);
    }
    if (i < P && (unsigned)logit_rows[i] >= (unsigned)N) { report(status, BAD_LOGIT_ROW, -1, i, logit_rows[i], N); logit_rows[i] = 0; }
}

// One block per request: the entries of its row that the step may read.
__global__ void check_pages_kernel(int* page_table, int table_width, const int* cu_tokens, const int* ctx_lens, int R, int page_size,
                                   int num_pages, int window, int group, int* status) {
    const int r = blockIdx.x;
    const int len = ctx_lens[r], q = cu_tokens[r + 1] - cu_tokens[r];
    const int pages = (len + page_size - 1) / page_size;
    if (pages > table_width) {
        if (threadIdx.x == 0) report(status, TABLE_TOO_NARROW, group, r, pages, table_width);
        return;
    }
    const int oldest = window > 0 ? max(0, len - q - window + 1) : 0;  // the oldest key that a token of this step may look at
    for (int pg = oldest / page_size + threadIdx.x; pg < pages; pg += blockDim.x) {
        int* e = page_table + (size_t)r * table_width + pg;
        if ((unsigned)*e >= (unsigned)num_pages) { report(status, BAD_PAGE, group, r * table_width + pg, *e, num_pages); *e = 0; }
    }
}

// Every new token's slot against the (repaired) page table.
__global__ void check_slots_kernel(const int* page_table, int table_width, int* slot_map, const int* positions, const int* token_request,
                                   int N, int R, int page_size, int num_pages, int group, int* status) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= N) return;
    const int r = token_request[t], pos = positions[t];
    const int slot = slot_map[t], slots = num_pages * page_size;
    if ((unsigned)r >= (unsigned)R || pos < 0 || pos / page_size >= table_width) {  // reported elsewhere; keep the slot inside the pool
        if ((unsigned)slot >= (unsigned)slots) { report(status, BAD_SLOT, group, t, slot, slots); slot_map[t] = 0; }
        return;
    }
    const int page = page_table[(size_t)r * table_width + pos / page_size];
    const bool page_ok = (unsigned)page < (unsigned)num_pages;
    const int want = page * page_size + pos % page_size;
    if ((unsigned)slot >= (unsigned)slots || (page_ok && slot != want)) {
        report(status, BAD_SLOT, group, t, slot, page_ok ? want : slots);
        slot_map[t] = page_ok ? want : 0;
    }
}

}  // namespace

LLM_EXPORT int llm_check_step_arrays(int* token_ids, int* positions, int* token_request, const int* cu_tokens, int* ctx_lens,
                                     int* logit_rows, int* state_slots, int N, int R, int P, int vocab, int max_positions,
                                     int state_slot_count, int* status, cudaStream_t stream) {
    if (N < 1 || R < 1 || P < 0 || !status) return LLM_ERR_BAD_ARGUMENT;
    const int most = max(N, max(R, P));
    check_step_arrays_kernel<<<(most + 255) / 256, 256, 0, stream>>>(token_ids, positions, token_request, cu_tokens, ctx_lens, logit_rows,
                                                                    state_slots, N, R, P, vocab, max_positions, state_slot_count, status);
    return (int)cudaGetLastError();
}

// To be launched after llm_check_step_arrays on the same stream (it trusts cu_tokens and repaired context lengths).
LLM_EXPORT int llm_check_page_group(int* page_table, int table_width, int* slot_map, const int* positions, const int* token_request,
                                    const int* cu_tokens, const int* ctx_lens, int N, int R, int page_size, int num_pages, int window,
                                    int group, int* status, cudaStream_t stream) {
    if (N < 1 || R < 1 || page_size < 1 || num_pages < 1 || table_width < 1 || !status) return LLM_ERR_BAD_ARGUMENT;
    check_pages_kernel<<<R, 128, 0, stream>>>(page_table, table_width, cu_tokens, ctx_lens, R, page_size, num_pages, window, group, status);
    check_slots_kernel<<<(N + 255) / 256, 256, 0, stream>>>(page_table, table_width, slot_map, positions, token_request, N, R, page_size,
                                                           num_pages, group, status);
    return (int)cudaGetLastError();
}
