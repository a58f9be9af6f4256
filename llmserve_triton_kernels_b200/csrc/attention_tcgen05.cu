// Causal (optionally windowed) grouped-query attention over the paged cache for prompt portions, on the
// fifth-generation tensor cores: both products of a key tile (scores = Q K^T, output += P V) are
// tcgen05.mma with their accumulators in tensor memory; queries, keys and values come into shared
// memory by TMA (128-byte swizzle), page by page through the request's page table.
//
// One CTA computes 128 query tokens of one head against the keys they may see, 64 keys at a time:
//   warps 0-3 : softmax.  Thread i owns query row i, which is lane i of tensor memory: it reads its 64
//               scores with tcgen05.ld, keeps the running maximum and sum of the row (no shuffles: the
//               whole row is the thread's), writes the probabilities as bfloat16 into shared memory in
//               the layout the next product reads, and folds the product's result into the 64 output
//               values it keeps in registers (rescaled by the change of the maximum).
//   warp 4    : producer.  Looks up pages (32 entries of the page table per load, handed round by
//               shuffles) and issues one TMA box per page for keys and one for values into a ring of
//               STAGES tiles.
//   warp 5    : one thread issues the products; the warp owns the allocation of tensor memory.
// The scores of tile j+1 are computed while the softmax of tile j runs (the issuer needs only to know
// that the scores of tile j have been read); two CTAs share an SM, so that one's softmax overlaps the
// other's products.  Softmax, running sums and the output are 32-bit; probabilities are rounded to
// bfloat16 for the second product, as in the mma.sync kernel.
//
// Keys past a request's length inside its last page, and pages outside the range a CTA needs, are
// never looked at: a score outside [window start, position] is -inf before the exponential, and the
// producer loads a page of the needed range in place of one outside it, so that no stale or released
// page is touched.  Values of masked keys meet a probability of exactly zero; the cache pool holds only
// finite numbers (it starts as zeros and is written by the projection kernels).
//
// Every mbarrier wait is bounded; a wait that gives up sets *error_flag, the roles leave their loops,
// tensor memory is freed and the kernel returns.
#include "attention_tile.cuh"
#include "umma.cuh"

namespace {

using attn::AttnParams;

constexpr int BM = 128, BN = 64, HD = 64, STAGES = 4, THREADS = 192;
constexpr int Q_BYTES = BM * HD * 2, P_BYTES = BM * BN * 2, K_BYTES = BN * HD * 2, STAGE_BYTES = 2 * K_BYTES;
constexpr int TMEM_COLS = 128;  // scores in columns [0, 64), the second product's result in [64, 128)

struct TcParams {
    AttnParams a;
    int min_tokens;         // requests with fewer tokens are other kernels'
    int tiles_per_request;  // 128-token tiles of the longest request
    int* error_flag;
};

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) { tma::mbar_arrive(bar); }

__global__ void __launch_bounds__(THREADS, 2)
attention_tcgen05_kernel(const TcParams tp, const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kvmap) {
    const AttnParams& p = tp.a;
    const int head = blockIdx.x, kvh = head / p.G;
    const int r = blockIdx.y / tp.tiles_per_request;
    const int tile = tp.tiles_per_request - 1 - (int)(blockIdx.y % tp.tiles_per_request);  // long tiles first
    const int q_begin = p.cu_tokens[r], q_len = p.cu_tokens[r + 1] - q_begin;
    if (q_len < tp.min_tokens) return;
    const int row0 = tile * BM;
    if (row0 >= q_len) return;
    const int rows_here = min(BM, q_len - row0);
    const int pos0 = p.ctx_lens[r] - q_len;
    const int key_hi = pos0 + row0 + rows_here - 1;
    const int key_lo = p.window > 0 ? max(0, pos0 + row0 - p.window + 1) : 0;
    const int t_begin = key_lo / BN, n_tiles = key_hi / BN + 1 - t_begin;
    // a key tile needs no mask if every row of the CTA sees all of it
    const int tile_pos_min = pos0 + row0;
    const int tile_lo_max = p.window > 0 ? max(0, pos0 + row0 + rows_here - 1 - p.window + 1) : 0;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* p_s = base + Q_BYTES;
    unsigned char* kv_s = p_s + P_BYTES;  // [STAGES][keys | values]
    __shared__ __align__(8) unsigned long long q_full, kv_full[STAGES], kv_empty[STAGES], s_full, s_empty, p_full, o_full;
    __shared__ unsigned tmem_base;
    __shared__ int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        tma::mbar_init(&q_full, 1);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            tma::mbar_init(&kv_full[s], 1);
            tma::mbar_init(&kv_empty[s], 1);
        }
        tma::mbar_init(&s_full, 1);
        tma::mbar_init(&s_empty, 4);
        tma::mbar_init(&p_full, 4);
        tma::mbar_init(&o_full, 1);
        gave_up = 0;
        tma::mbar_fence_init();
        tma::prefetch_map(&qmap);
        tma::prefetch_map(&kvmap);
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma::smem_addr(&tmem_base)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    pdl_trigger();
    pdl_wait();  // the queries and the step's keys and values come from the kernels before

    auto fail = [&]() {
        gave_up = 1;
        if (tp.error_flag) atomicExch(tp.error_flag, 1);
    };

    if (warp == 4) {
        // ---- producer ----
        const int ps = p.page_size, pages_per_tile = BN / ps;
        const int lp_lo = key_lo / ps, lp_hi = key_hi / ps;
        const int* table = p.page_table + (size_t)r * p.table_width;
        if (lane == 0) {
            tma::mbar_expect_tx(&q_full, Q_BYTES);
            tma::load_2d(q_s, &qmap, head * HD, q_begin + row0, &q_full);
        }
        const int first_page = t_begin * pages_per_tile, total_pages = n_tiles * pages_per_tile;
        bool alive = true;
        for (int pg0 = 0; pg0 < total_pages && alive; pg0 += 32) {
            // 32 entries of the page table at once; a page outside the needed range is replaced by one inside it
            const int lp = min(max(first_page + pg0 + lane, lp_lo), lp_hi);
            const int my_page = table[lp];
            const int n_here = min(32, total_pages - pg0);
            for (int i = 0; i < n_here && alive; ++i) {
                const int page = __shfl_sync(0xffffffffu, my_page, i);
                const int idx = pg0 + i, j = idx / pages_per_tile, in_tile = idx - j * pages_per_tile, s = j % STAGES;
                if (lane == 0) {
                    if (in_tile == 0) {
                        if (gave_up || (j >= STAGES && !tma::mbar_wait(&kv_empty[s], ((j / STAGES) - 1) & 1))) {
                            if (!gave_up) fail();
                            alive = false;
                        } else {
                            tma::mbar_expect_tx(&kv_full[s], STAGE_BYTES);
                        }
                    }
                    if (alive) {
                        unsigned char* k_dst = kv_s + (size_t)s * STAGE_BYTES + (size_t)in_tile * ps * (HD * 2);
                        const int row_k = ((page * 2) * p.KV + kvh) * ps, row_v = ((page * 2 + 1) * p.KV + kvh) * ps;
                        tma::load_2d(k_dst, &kvmap, 0, row_k, &kv_full[s]);
                        tma::load_2d(k_dst + K_BYTES, &kvmap, 0, row_v, &kv_full[s]);
                    }
                }
                alive = __shfl_sync(0xffffffffu, (int)alive, 0) != 0;
            }
        }
    } else if (warp == 5) {
        // ---- issuer of the products ----
        if (lane == 0) {
            constexpr unsigned IDESC_QK = umma::idesc_bf16(BM, BN, false), IDESC_PV = umma::idesc_bf16(BM, HD, true);
            const unsigned s_tmem = tmem_base, o_tmem = tmem_base + BN;
            const unsigned long long q_desc = umma::desc_sw128(q_s), p_desc = umma::desc_sw128(p_s);
            auto scores = [&](int j) {  // S = Q K_j^T
                const unsigned long long k_desc = umma::desc_sw128(kv_s + (size_t)(j % STAGES) * STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) umma::mma_bf16(s_tmem, q_desc + 2 * k, k_desc + 2 * k, IDESC_QK, k != 0);
                umma::commit(&s_full);
            };
            bool ok = tma::mbar_wait(&q_full, 0) && tma::mbar_wait(&kv_full[0], 0);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                scores(0);
            }
            for (int j = 0; j < n_tiles && ok && !gave_up; ++j) {
                const int s = j % STAGES;
                if (j + 1 < n_tiles) {
                    // the scores of the next tile, as soon as those of this one have been read
                    ok = tma::mbar_wait(&s_empty, j & 1) && tma::mbar_wait(&kv_full[(j + 1) % STAGES], ((j + 1) / STAGES) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    scores(j + 1);
                }
                ok = tma::mbar_wait(&p_full, j & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // the values lie [key][d]: B with N contiguous; 16 keys are two atoms of 8 rows, 2048 bytes further per step
                const unsigned long long v_desc = umma::desc_sw128(kv_s + (size_t)s * STAGE_BYTES + K_BYTES, 1024 >> 4);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) umma::mma_bf16(o_tmem, p_desc + 2 * k, v_desc + (2048 >> 4) * k, IDESC_PV, k != 0);
                umma::commit(&o_full);
                umma::commit(&kv_empty[s]);
            }
            if (!ok) fail();
        }
    } else {
        // ---- softmax: thread = query row = lane of tensor memory ----
        const int row = warp * 32 + lane, tok = row0 + row;
        const bool row_ok = tok < q_len;
        const int pos = pos0 + tok;
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const unsigned lane_base = tmem_base + ((unsigned)(warp * 32) << 16);
        float o[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int key_base = (t_begin + j) * BN;
            ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&s_full, j & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const bool whole = key_base + BN - 1 <= tile_pos_min && key_base >= tile_lo_max && rows_here == BM;
            // the keys of this tile that the row sees are those with index (within the tile) in [see_lo, see_hi]
            const int see_lo = row_ok ? lo - key_base : BN, see_hi = row_ok ? pos - key_base : -1;
            // first pass over the scores: the row's maximum (four chains, so that the comparisons do not wait for
            // one another; the scale is positive and is applied to the maximum alone)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int h = 0; h < BN / 32; ++h) {
                float v[32];
                umma::tmem_ld32(lane_base + h * 32, v);
                if (whole) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], v[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const bool visible = h * 32 + i >= see_lo && h * 32 + i <= see_hi;
                        mx4[i & 3] = fmaxf(mx4[i & 3], visible ? v[i] : -INFINITY);
                    }
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            const float m_new = fmaxf(m_run, mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = attn::fast_exp2(m_run - m_use);
            m_run = m_new;
            // second pass: the probabilities, into shared memory as the second product's A (K-major, 128-byte
            // swizzle: row `row`, 16-byte piece c at c ^ (row % 8))
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            const float shift = -m_use;
#pragma unroll
            for (int h = 0; h < BN / 32; ++h) {
                float v[32];
                umma::tmem_ld32(lane_base + h * 32, v);
                if (whole) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = attn::fast_exp2(fmaf(v[i], p.scale_log2, shift));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const bool visible = h * 32 + i >= see_lo && h * 32 + i <= see_hi;
                        v[i] = visible ? attn::fast_exp2(fmaf(v[i], p.scale_log2, shift)) : 0.f;
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) sum4[i & 3] += v[i];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint4 u;
                    u.x = attn::pack_bf16(v[c * 8], v[c * 8 + 1]);
                    u.y = attn::pack_bf16(v[c * 8 + 2], v[c * 8 + 3]);
                    u.z = attn::pack_bf16(v[c * 8 + 4], v[c * 8 + 5]);
                    u.w = attn::pack_bf16(v[c * 8 + 6], v[c * 8 + 7]);
                    *reinterpret_cast<uint4*>(p_s + row * 128 + (((h * 4 + c) ^ (row & 7)) << 4)) = u;
                }
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l_run = l_run * alpha + sum;
            // the scores have been read (the next tile's may overwrite them) and the probabilities are written
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s_empty);
                mbar_arrive(&p_full);
            }
            ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&o_full, j & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int h = 0; h < HD / 32; ++h) {
                float v[32];
                umma::tmem_ld32(lane_base + BN + h * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[h * 32 + i] = o[h * 32 + i] * alpha + v[i];
            }
        }
        if (!ok) {
            if (lane == 0) fail();
        } else if (row_ok) {
            const float inv = 1.f / l_run;
            __nv_bfloat16* dst = p.out + (size_t)(q_begin + tok) * p.out_stride + (size_t)head * HD;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                uint4 u;
                u.x = attn::pack_bf16(o[c * 8] * inv, o[c * 8 + 1] * inv);
                u.y = attn::pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
                u.z = attn::pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
                u.w = attn::pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
                *reinterpret_cast<uint4*>(dst + c * 8) = u;
            }
        }
    }
    // after a failed wait, copies may still be on their way into this CTA's shared memory: wait for them (bounded)
    if (gave_up && threadIdx.x == 0) {
        tma::mbar_wait(&q_full, 0);
        for (int j = max(0, n_tiles - STAGES); j < n_tiles; ++j) tma::mbar_wait(&kv_full[j % STAGES], (j / STAGES) & 1);
    }
    // everyone is done with tensor memory: the allocating warp gives it back
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
    }
}

}  // namespace

// The fewest tokens a request must bring for this kernel to take it (its CTAs are 128 tokens of one head).
LLM_EXPORT int llm_attention_tcgen05_min_tokens() { return 128; }

// Attention of the requests that bring at least min_tokens tokens (others are left untouched: another kernel's).
// q: bfloat16 rows of q_stride elements that start with the H query heads; out: [tokens, H * 64] with row stride
// out_stride; pool: one layer's plane [pool_pages, 2, KV, page_size, 64]; max_tokens: the most tokens of any request.
// Takes head size 64, pages of 8, 16, 32 or 64 keys, 16-byte aligned rows; else LLM_ERR_UNSUPPORTED (nothing ran).
LLM_EXPORT int llm_attention_tcgen05(const void* q, int q_stride, void* out, int out_stride, const void* pool, long long pool_pages,
                                     const int* page_table, int table_width, const int* cu_tokens, const int* ctx_lens,
                                     int requests, int n_tokens, int H, int KV, int D, int page_size, int window, float scale,
                                     int min_tokens, int max_tokens, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0 || requests <= 0 || max_tokens < min_tokens) return 0;
    if (D != HD || (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64)) return LLM_ERR_UNSUPPORTED;
    if (H <= 0 || KV <= 0 || H % KV || table_width <= 0 || min_tokens < 1 || !(scale > 0.f)) return LLM_ERR_BAD_ARGUMENT;
    if ((q_stride & 7) || (out_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)pool & 127) || q_stride < H * HD)
        return LLM_ERR_UNSUPPORTED;
    const long long kv_rows = pool_pages * 2 * KV * page_size;
    if (kv_rows <= 0 || kv_rows > 0x7fffffffLL) return LLM_ERR_UNSUPPORTED;
    const CUtensorMap* qmap = tma::cached_map_2d_bf16(q, (uint64_t)n_tokens, (uint64_t)H * HD, (uint64_t)q_stride, BM, HD, CU_TENSOR_MAP_SWIZZLE_128B);
    const CUtensorMap* kvmap = tma::cached_map_2d_bf16(pool, (uint64_t)kv_rows, HD, HD, (uint32_t)page_size, HD, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!qmap || !kvmap) return LLM_ERR_UNSUPPORTED;
    TcParams tp = {};
    tp.a.out = (__nv_bfloat16*)out;
    tp.a.out_stride = out_stride;
    tp.a.page_table = page_table;
    tp.a.table_width = table_width;
    tp.a.cu_tokens = cu_tokens;
    tp.a.ctx_lens = ctx_lens;
    tp.a.H = H;
    tp.a.KV = KV;
    tp.a.G = H / KV;
    tp.a.page_size = page_size;
    tp.a.window = window;
    tp.a.scale_log2 = scale * 1.4426950408889634f;
    tp.min_tokens = min_tokens;
    tp.tiles_per_request = (max_tokens + BM - 1) / BM;
    tp.error_flag = error_flag;
    const long long y = (long long)requests * tp.tiles_per_request;
    if (y > 65535) return LLM_ERR_UNSUPPORTED;
    constexpr size_t smem = 1024 + Q_BYTES + P_BYTES + (size_t)STAGES * STAGE_BYTES;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_pdl(attention_tcgen05_kernel, dim3((unsigned)H, (unsigned)y), dim3(THREADS), smem, stream, tp, *qmap, *kvmap);
}
