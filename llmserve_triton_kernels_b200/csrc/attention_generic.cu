// Paged grouped-query attention for any mix of query lengths, any head size up to 256 and any
// group size: one warp per (token, query head).
//
// This is the attention of the true 32-bit path and the fallback of the bfloat16 path for
// shapes its faster kernels refuse.  Scores, the running maximum, the exponentials and the
// weighted sum are 32-bit.  Keys are visited in chunks of 32 that start at multiples of 32 of
// the absolute key position, so the order of every addition depends only on the query's
// position (and the window), never on how the tokens were cut into steps or batched.
//
// q rows hold the query heads first (row stride q_stride elements); out is [tokens, H * D].
// pool plane: [pages, 2, KV, page_size, D].  A query at position p of request r sees keys
// max(0, p - window + 1) .. p (window <= 0: from 0).
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ pool, const int* __restrict__ page_table, int table_width,
                         const int* __restrict__ token_request, const int* __restrict__ cu_tokens,
                         const int* __restrict__ ctx_lens, int n_tokens, int H, int KV, int D, int page_size,
                         int window, float scale) {
    __shared__ float q_s[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const int r = token_request[t];
    const int q_begin = cu_tokens[r], q_len = cu_tokens[r + 1] - q_begin;
    const int pos = ctx_lens[r] - q_len + (t - q_begin);
    const int kvh = h / (H / KV);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    const T* qp = q + (size_t)t * q_stride + (size_t)h * D;
    for (int d = lane; d < D; d += 32) q_s[warp][d] = to_float(qp[d]);
    __syncwarp();

    const int* table = page_table + (size_t)r * table_width;
    const size_t head_stride = (size_t)page_size * D;
    constexpr int ACC = MAX_D / 32;
    float acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int c = (lo / 32) * 32; c <= pos; c += 32) {
        const int j = c + lane;
        const bool visible = j >= lo && j <= pos;
        float s = -INFINITY;
        if (visible) {
            const int page = table[j / page_size], off = j % page_size;
            const T* kp = pool + ((size_t)(page * 2 + 0) * KV + kvh) * head_stride + (size_t)off * D;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot = fmaf(q_s[warp][d], to_float(kp[d]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));  // finite: the chunk holds at least one visible key
        const float p = visible ? expf(s - m_new) : 0.f;
        const float rescale = expf(m - m_new);  // 0 on the first chunk (m = -inf)
        l = l * rescale + warp_sum(p);
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] *= rescale;
        m = m_new;
        const int count = min(32, pos - c + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            if (pj == 0.f) continue;  // uniform across the warp
            const int key = c + jj;
            const int page = table[key / page_size], off = key % page_size;
            const T* vp = pool + ((size_t)(page * 2 + 1) * KV + kvh) * head_stride + (size_t)off * D;
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(pj, to_float(vp[d]), acc[i]);
            }
        }
    }
    const float inv = 1.f / l;
    T* op = out + (size_t)t * out_stride + (size_t)h * D;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < D) op[d] = from_float<T>(acc[i] * inv);
    }
}

}  // namespace

LLM_EXPORT int llm_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* pool,
                                     int dtype, const int* page_table, int table_width, const int* token_request,
                                     const int* cu_tokens, const int* ctx_lens, int n_tokens, int H, int KV, int D,
                                     int page_size, int window, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || D > MAX_D || H <= 0 || KV <= 0 || H % KV || page_size <= 0 || table_width <= 0)
        return LLM_ERR_BAD_ARGUMENT;
    const long long items = (long long)n_tokens * H;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 0x7fffffffLL) return LLM_ERR_UNSUPPORTED;
    if (dtype == LLM_F32)
        attention_generic_kernel<float><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
            (const float*)q, q_stride, (float*)out, out_stride, (const float*)pool, page_table, table_width,
            token_request, cu_tokens, ctx_lens, n_tokens, H, KV, D, page_size, window, scale);
    else if (dtype == LLM_BF16)
        attention_generic_kernel<__nv_bfloat16><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)pool, page_table,
            table_width, token_request, cu_tokens, ctx_lens, n_tokens, H, KV, D, page_size, window, scale);
    else
        return LLM_ERR_BAD_ARGUMENT;
    return launch_status();
}
