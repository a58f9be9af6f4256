// Paged grouped-query attention on the tensor cores (bfloat16, head sizes 16/32/64/128) for
// prefill portions and decode tokens of one step.
//
// Work is cut by (request, key/value head): the query rows of a CTA are (token, member of the
// head group) pairs, so the G query heads that share a key/value head share every key and value
// that is loaded.  Two shapes of CTA, both 4 warps:
//   * ROWS: 64 rows (4 warps x 16); every warp walks the same keys.  Serves requests that bring
//     more than 16 rows (portions of prompts).
//   * KEYS: 16 rows; the 4 warps walk different keys of each tile and merge at the end.  Serves
//     decode tokens and very short portions.
// A launch of one shape skips the requests that belong to the other.  Keys and values are copied
// page by page into shared memory with cp.async (a ring of three or four tiles), the products are mma.sync
// m16n8k16 with 32-bit accumulation, the softmax is the running (max, sum) form in 32-bit in the
// base-2 domain.  Long contexts with few rows are cut over gridDim.x ("splits"); each split
// writes an unnormalised 32-bit partial and its (max, sum) to scratch memory, and the split that
// finishes last (a counter per request and key/value head tells) merges them.  A split's share of the keys is worked out on the device from the request's
// length, so the grid does not depend on the lengths (a CUDA graph replays it as captured).
#include "attention_tile.cuh"

#include <cstdlib>
#include "timeline.cuh"

namespace {

using namespace attn;

// D: head size.  ROW_WARPS x KEY_WARPS warps.  BN: keys per warp and tile.  blockIdx: (split, key/value
// head, request * tiles_per_request + row tile).
template <int D, int ROW_WARPS, int KEY_WARPS, int BN, int STAGES>
__global__ void __launch_bounds__(32 * ROW_WARPS * KEY_WARPS) attention_mma_kernel(const AttnParams p) {
    TL(tl::Marks marks;)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    attention_tile<D, ROW_WARPS, KEY_WARPS, BN, STAGES>(p, blockIdx.x, blockIdx.y, blockIdx.z / p.tiles_per_request,
                                                blockIdx.z % p.tiles_per_request, smem_raw, true TL(, &marks));
    TL(__syncthreads(); if (threadIdx.x == 0) {
        marks.mark(4);
        marks.write(100 + KEY_WARPS, 0, blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z), p.splits, 0);
    })
}

// Merges the splits of every (token, head) whose request went through a launch with splits > 1.
template <int D>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                       __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ token_request,
                                       const int* __restrict__ cu_tokens, int n_tokens, int H, int G, int merge_small,
                                       int merge_large) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tokens * H) return;
    const int tok = warp / H, head = warp - tok * H;
    const int r = token_request[tok];
    const bool small = (cu_tokens[r + 1] - cu_tokens[r]) * G <= SMALL_ROWS;
    if (small ? !merge_small : !merge_large) return;
    const size_t slot = ((size_t)tok * H + head) * splits;
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(slot + s) * 2]);
    const float m_use = m == -INFINITY ? 0.f : m;
    float l = 0.f;
    for (int s = 0; s < splits; ++s) l += part_ml[(slot + s) * 2 + 1] * exp2f(part_ml[(slot + s) * 2] - m_use);
    const float inv = 1.f / l;
    for (int d = lane; d < D; d += 32) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s) o += part_o[(slot + s) * D + d] * exp2f(part_ml[(slot + s) * 2] - m_use);
        out[(size_t)tok * out_stride + (size_t)head * D + d] = __float2bfloat16_rn(o * inv);
    }
}

template <int D, int ROW_WARPS, int KEY_WARPS, int BN, int STAGES>
int launch_shape(const AttnParams& p, int requests, cudaStream_t stream) {
    constexpr int BNC = BN * KEY_WARPS;
    size_t smem = (size_t)STAGES * 2 * BNC * attn::tile_pitch(D, ROW_WARPS, KEY_WARPS, BN) * sizeof(__nv_bfloat16);
    const size_t merge = ((size_t)KEY_WARPS * 16 * (attn::merge_pitch(D) + 2) + 16 * KEY_WARPS + 32) * sizeof(float);
    if (KEY_WARPS > 1 && merge > smem) smem = merge;
    auto kernel = attention_mma_kernel<D, ROW_WARPS, KEY_WARPS, BN, STAGES>;
    if (smem > 40 * 1024) {  // with the kernel's static shared memory beside it, more than the 48 KB that need no opt-in
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    static bool carved = false;  // per instantiation: all of the SM's memory as shared memory, so that this kernel's CTAs
    if (!carved) {               // may join those of the kernel in front on an SM, and the next kernel's may join them
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carved = true;
    }
    const long long z = (long long)requests * p.tiles_per_request;
    if (z > 65535 || p.KV > 65535) return LLM_ERR_UNSUPPORTED;
    dim3 grid(p.splits, p.KV, (unsigned)z);
    return launch_pdl(kernel, grid, dim3(32 * ROW_WARPS * KEY_WARPS), smem, stream, p);
}

template <int D>
int launch_all(AttnParams p, int requests, int n_tokens, const int* token_request, int max_rows_large, int splits_small,
               int splits_large, int have_small, cudaStream_t stream) {
    int code = 0;
    if (max_rows_large > 0) {
        p.splits = splits_large;
        p.tiles_per_request = (max_rows_large + 63) / 64;
        code = launch_shape<D, 4, 1, 64, stages_of(D, 1)>(p, requests, stream);
        if (code) return code;
    }
    if (have_small) {
        p.splits = splits_small;
        p.tiles_per_request = 1;
        // few rows: sixteen warps (eight for the largest head size) share the keys of a tile, 16 keys each, so that a
        // tile is a short step for every warp; the warps' shares are merged through shared memory at the end
        // More (request, kv head) pairs than SMs: eight warps and tiles of 128 keys, so that two CTAs share an SM and all
        // pairs run at once.
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        static const int forced = [] { const char* e = getenv("LLMSERVE_B200_ATTN_KEY_WARPS"); return e ? atoi(e) : 0; }();
        const bool many = forced ? forced == 8 : (long long)requests * p.KV > sms;
        if constexpr (D <= 64) code = many ? launch_shape<D, 1, 8, 16, 3>(p, requests, stream) : launch_shape<D, 1, 16, 16, 3>(p, requests, stream);
        else code = launch_shape<D, 1, 8, 16, 3>(p, requests, stream);
        if (code) return code;
    }
    const int merge_small = 0, merge_large = max_rows_large > 0 && splits_large > 1;  // the small shape merges in place
    if (merge_small || merge_large) {
        if (merge_small && merge_large && splits_small != splits_large) return LLM_ERR_BAD_ARGUMENT;
        const int splits = merge_small ? splits_small : splits_large;
        const long long warps = (long long)n_tokens * p.H;
        const int threads = 128;
        const long long blocks = (warps * 32 + threads - 1) / threads;
        attention_merge_kernel<D><<<(unsigned)blocks, threads, 0, stream>>>(p.part_o, p.part_ml, splits, p.out, p.out_stride,
                                                                            token_request, p.cu_tokens, n_tokens, p.H, p.G,
                                                                            merge_small, merge_large);
        code = launch_status();
    }
    return code;
}

}  // namespace

TL_DEFINE_READER(llm_timeline_read_attention)

// One step's attention in bfloat16.  max_rows_large: the most rows (tokens x group) of any request
// with more than 16 rows, 0 if there is none; have_small: some request has at most 16 rows.
// scratch_o / scratch_ml: float32 [tokens, H, splits, D] and [tokens, H, splits, 2], needed when a
// split count exceeds 1; counters: int32 [requests * KV], all zero before the launch and again
// after it, needed when splits_small exceeds 1.  Returns LLM_ERR_UNSUPPORTED for head sizes other than 16/32/64/128.
// skip_tokens_from: requests that bring at least this many tokens are left to another kernel (0: none are).
LLM_EXPORT int llm_attention_mma_routed(const void* q, int q_stride, void* out, int out_stride, const void* pool,
                                        const int* page_table, int table_width, const int* token_request, const int* cu_tokens,
                                        const int* ctx_lens, int requests, int n_tokens, int H, int KV, int D, int page_size,
                                        int window, float scale, int max_rows_large, int have_small, int splits_small,
                                        int splits_large, float* scratch_o, float* scratch_ml, int* counters,
                                        int skip_tokens_from, cudaStream_t stream) {
    if (n_tokens <= 0 || requests <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV || page_size <= 0 || table_width <= 0 || splits_small < 1 || splits_large < 1)
        return LLM_ERR_BAD_ARGUMENT;
    if ((q_stride & 1) || (out_stride & 1)) return LLM_ERR_BAD_ARGUMENT;
    if ((splits_small > 1 || splits_large > 1) && (!scratch_o || !scratch_ml)) return LLM_ERR_BAD_ARGUMENT;
    if (splits_small > 1 && !counters) return LLM_ERR_BAD_ARGUMENT;
    if (splits_small > 32) return LLM_ERR_BAD_ARGUMENT;
    // the merge of the 64-row shape's splits walks every token of the step, also those that another kernel serves
    if (splits_large > 1 && skip_tokens_from > 0) return LLM_ERR_BAD_ARGUMENT;
    AttnParams p;
    p.q = (const __nv_bfloat16*)q;
    p.q_stride = q_stride;
    p.out = (__nv_bfloat16*)out;
    p.out_stride = out_stride;
    p.pool = (const __nv_bfloat16*)pool;
    p.page_table = page_table;
    p.table_width = table_width;
    p.cu_tokens = cu_tokens;
    p.ctx_lens = ctx_lens;
    p.H = H;
    p.KV = KV;
    p.G = H / KV;
    p.page_size = page_size;
    p.window = window;
    p.tiles_per_request = 1;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.splits = 1;
    p.part_o = scratch_o;
    p.part_ml = scratch_ml;
    p.counters = counters;
    p.skip_tokens_from = skip_tokens_from;
    p.error_flag = library_error_flag();
    switch (D) {
        case 16: return launch_all<16>(p, requests, n_tokens, token_request, max_rows_large, splits_small, splits_large, have_small, stream);
        case 32: return launch_all<32>(p, requests, n_tokens, token_request, max_rows_large, splits_small, splits_large, have_small, stream);
        case 64: return launch_all<64>(p, requests, n_tokens, token_request, max_rows_large, splits_small, splits_large, have_small, stream);
        case 128: return launch_all<128>(p, requests, n_tokens, token_request, max_rows_large, splits_small, splits_large, have_small, stream);
        default: return LLM_ERR_UNSUPPORTED;
    }
}

LLM_EXPORT int llm_attention_mma(const void* q, int q_stride, void* out, int out_stride, const void* pool,
                                 const int* page_table, int table_width, const int* token_request, const int* cu_tokens,
                                 const int* ctx_lens, int requests, int n_tokens, int H, int KV, int D, int page_size,
                                 int window, float scale, int max_rows_large, int have_small, int splits_small,
                                 int splits_large, float* scratch_o, float* scratch_ml, int* counters,
                                 cudaStream_t stream) {
    return llm_attention_mma_routed(q, q_stride, out, out_stride, pool, page_table, table_width, token_request, cu_tokens, ctx_lens,
                                    requests, n_tokens, H, KV, D, page_size, window, scale, max_rows_large, have_small,
                                    splits_small, splits_large, scratch_o, scratch_ml, counters, 0, stream);
}
