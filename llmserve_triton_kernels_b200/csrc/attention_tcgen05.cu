// Causal (optionally windowed) grouped-query attention over the paged cache for prompt portions, on the
// fifth-generation tensor cores: both products of a key tile (scores = Q K^T, output += P V) are
// tcgen05.mma with their accumulators AND their A operands (queries, probabilities) in tensor memory; keys and
// values come into shared memory by TMA (128-byte swizzle), page by page through the request's page table.
//
// One CTA computes 128 query tokens of one head against the keys they may see, 64 keys at a time:
//   warps 0-3 : softmax.  Thread i owns query row i, which is lane i of tensor memory: it puts its queries there
//               once, reads its 64 scores with tcgen05.ld, keeps the running maximum and sum of the row (no
//               shuffles: the whole row is the thread's) and stores the probabilities as bfloat16 into its lane,
//               where the second product reads them.  The output accumulates in tensor memory over all key
//               tiles; a row's shift follows its maximum only when the maximum has risen by more than 2^8, and
//               only then does the warp rescale its 32 rows of the output (load, multiply, store).
//   warps 4, 6: producers of keys and of values.  Each looks up pages (32 entries of the page table per load,
//               handed round by shuffles) and issues one TMA box per page, each from a lane of its own, into
//               rings of STAGES tiles; a stage of keys is free as soon as its scores are computed.
//   warps 5, 7: one thread of each issues a product (5 the scores, 7 the output); warp 5 owns the allocation of
//               tensor memory.
// Scores have two buffers: those of tile j+1 are computed while the softmax of tile j runs, and the second
// product of tile j runs while the softmax of tile j+1 does.  Two CTAs share an SM.  Softmax, running sums and
// the output are 32-bit; probabilities are rounded to bfloat16 for the second product, as in the mma.sync kernel.
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
#ifdef ATT_PROF
#include <cstdio>
#endif
#include "umma.cuh"

namespace {

using attn::AttnParams;

constexpr int BM = 128, BN = 64, HD = 64, STAGES = 3, THREADS = 256;
constexpr int K_BYTES = BN * HD * 2, STAGE_BYTES = 2 * K_BYTES;
constexpr float LAZY = 8.f;  // log2 of how far a row's maximum may rise before its shift follows
// Tensor memory: two tiles of scores in columns [0, 64) and [64, 128); the output in [128, 192); the queries in
// [192, 224) and a tile's probabilities in [224, 256), two bfloat16 to a column.
constexpr int TMEM_COLS = 256, O_COL = 2 * BN, Q_COL = 2 * BN + HD, P_COL = Q_COL + HD / 2;

struct TcParams {
    AttnParams a;
    int min_tokens;         // requests with fewer tokens are other kernels'
    int tiles_per_request;  // 128-token tiles of the longest request
    int* error_flag;
};

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) { tma::mbar_arrive(bar); }

__global__ void __launch_bounds__(THREADS, 2)
attention_tcgen05_kernel(const TcParams tp, const __grid_constant__ CUtensorMap kvmap) {
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
    unsigned char* kv_s = base;  // [STAGES][keys | values]
    __shared__ __align__(8) unsigned long long q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES], s_full[2], s_empty[2], p_full, o_full;
    __shared__ unsigned tmem_base;
    __shared__ int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        tma::mbar_init(&q_full, 4);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            tma::mbar_init(&k_full[s], 1);
            tma::mbar_init(&k_empty[s], 1);
            tma::mbar_init(&v_full[s], 1);
            tma::mbar_init(&v_empty[s], 1);
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            tma::mbar_init(&s_full[b], 1);
            tma::mbar_init(&s_empty[b], 4);
        }
        tma::mbar_init(&p_full, 4);
        tma::mbar_init(&o_full, 1);
        gave_up = 0;
        tma::mbar_fence_init();
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

    if (warp == 4 || warp == 6) {
        // ---- producers: warp 4 brings the queries and the keys, warp 6 the values ----
        // Keys and values have rings of their own: a stage of keys is free again as soon as its scores are computed,
        // which is more than a tile before the values of the same tile have been used, so the keys of three tiles on
        // are requested that much earlier (with one ring for both, the scores waited for their keys).
        const bool is_v = warp == 6;
        unsigned long long* full = is_v ? v_full : k_full;
        unsigned long long* empty = is_v ? v_empty : k_empty;
        const int ps = p.page_size, pages_per_tile = BN / ps;
        const int lp_lo = key_lo / ps, lp_hi = key_hi / ps;
        const int* table = p.page_table + (size_t)r * p.table_width;
        // One box per page, each issued by a lane of its own (a thread's TMA instructions follow one another slowly;
        // several threads' overlap).  The page table is read 32 entries at a time; a page outside the needed range is
        // replaced by one inside it.
        const int first_page = t_begin * pages_per_tile;
        int my_page = 0, loaded_from = -32;
        bool alive = true;
        for (int j = 0; j < n_tiles && alive; ++j) {
            const int s = j % STAGES, idx0 = j * pages_per_tile;
            if (idx0 >= loaded_from + 32) {  // pages_per_tile divides 32: a tile's pages lie in one batch
                loaded_from = idx0;
                my_page = table[min(max(first_page + idx0 + lane, lp_lo), lp_hi)];
            }
            if (lane == 0) {
                if (gave_up || (j >= STAGES && !tma::mbar_wait(&empty[s], ((j / STAGES) - 1) & 1))) {
                    if (!gave_up) fail();
                    alive = false;
                } else {
                    tma::mbar_expect_tx(&full[s], K_BYTES);
                }
            }
            alive = __shfl_sync(0xffffffffu, (int)alive, 0) != 0;
            const int page = __shfl_sync(0xffffffffu, my_page, (idx0 - loaded_from + lane) & 31);
            if (alive && lane < pages_per_tile) {
                unsigned char* dst = kv_s + (size_t)s * STAGE_BYTES + (size_t)is_v * K_BYTES + (size_t)lane * ps * (HD * 2);
                tma::load_2d(dst, &kvmap, 0, ((page * 2 + (int)is_v) * p.KV + kvh) * ps, &full[s]);
            }
        }
    } else if (warp == 5) {
        // ---- issuer of the scores: S[j % 2] = Q K_j^T, as soon as the keys are there and the buffer has been read ----
        // One thread spends about a hundred cycles on every tcgen05.mma it issues and sixty on a commit, so the two
        // products of a tile have an issuing thread each: together in one thread they, not the softmax, set the pace.
        // Both products take their A operand (queries, probabilities) from tensor memory: read from shared memory, a
        // 128 x 64 x 16 step would want 6 KB in 32 cycles, more than shared memory gives.
        if (lane == 0) {
            constexpr unsigned IDESC_QK = umma::idesc_bf16(BM, BN, false);
            const unsigned q_tmem = tmem_base + Q_COL;
            bool ok = tma::mbar_wait(&q_full, 0);
            for (int j = 0; j < n_tiles && ok && !gave_up; ++j) {
                ok = tma::mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1) && (j < 2 || tma::mbar_wait(&s_empty[j & 1], ((j >> 1) - 1) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned long long k_desc = umma::desc_sw128(kv_s + (size_t)(j % STAGES) * STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) umma::mma_bf16_ts(tmem_base + (j & 1) * BN, q_tmem + 8 * k, k_desc + 2 * k, IDESC_QK, k != 0);
                umma::commit(&s_full[j & 1]);
                umma::commit(&k_empty[j % STAGES]);
            }
            if (!ok) fail();
        }
    } else if (warp == 7) {
        // ---- issuer of the second product: O += P_j V_j, as soon as the probabilities and the values are there ----
        if (lane == 0) {
            constexpr unsigned IDESC_PV = umma::idesc_bf16(BM, HD, true);
            const unsigned o_tmem = tmem_base + O_COL, p_tmem = tmem_base + P_COL;
            bool ok = true;
            for (int j = 0; j < n_tiles && ok && !gave_up; ++j) {
                const int s = j % STAGES;
                ok = tma::mbar_wait(&v_full[s], (j / STAGES) & 1) && tma::mbar_wait(&p_full, j & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // the values lie [key][d]: B with N contiguous; 16 keys are two atoms of 8 rows, 2048 bytes further per step
                const unsigned long long v_desc = umma::desc_sw128(kv_s + (size_t)s * STAGE_BYTES + K_BYTES, 1024 >> 4);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)  // the output accumulates over the tiles
                    umma::mma_bf16_ts(o_tmem, p_tmem + 8 * k, v_desc + (2048 >> 4) * k, IDESC_PV, k != 0 || j != 0);
                umma::commit(&o_full);
                umma::commit(&v_empty[s]);
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
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        const unsigned o_taddr = lane_base + O_COL;
        {   // the row's queries, as they lie in memory (two to a word), into the row's lane of tensor memory
            unsigned qw[32];
            const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)(q_begin + tok) * p.q_stride + (size_t)head * HD);
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                const uint4 u = row_ok ? src[c] : make_uint4(0, 0, 0, 0);
                qw[4 * c] = u.x; qw[4 * c + 1] = u.y; qw[4 * c + 2] = u.z; qw[4 * c + 3] = u.w;
            }
            umma::tmem_st32(lane_base + Q_COL, qw);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_full);
        }
#ifdef ATT_PROF
        long long pc[6] = {0, 0, 0, 0, 0, 0}, c0 = clock64(), c1;
#define PH(i) { c1 = clock64(); pc[i] += c1 - c0; c0 = c1; }
#else
#define PH(i)
#endif
        for (int j = 0; j < n_tiles; ++j) {
            const int key_base = (t_begin + j) * BN;
            ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&s_full[j & 1], (j >> 1) & 1));
            PH(0)
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const bool whole = key_base + BN - 1 <= tile_pos_min && key_base >= tile_lo_max && rows_here == BM;
            // the keys of this tile that the row sees are those with index (within the tile) in [see_lo, see_hi]
            const int see_lo = row_ok ? lo - key_base : BN, see_hi = row_ok ? pos - key_base : -1;
            // the row's 64 scores in one load; once they are in registers the buffer may take the scores two tiles on
            static_assert(BN == 64, "the softmax reads a tile's scores with one 64-column load");
            float v[BN];
            umma::tmem_ld64(lane_base + (j & 1) * BN, v);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[j & 1]);  // the buffer may take the scores two tiles on
            PH(1)
            // the row's maximum (four chains, so that the comparisons do not wait for one another; the scale is
            // positive and is applied to the maximum alone)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (whole) {
#pragma unroll
                for (int i = 0; i < BN; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], v[i]);
            } else {
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    const bool visible = i >= see_lo && i <= see_hi;
                    v[i] = visible ? v[i] : -INFINITY;
                    mx4[i & 3] = fmaxf(mx4[i & 3], v[i]);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            // The output accumulates in tensor memory, scaled by 2^-m_run.  The row keeps its old shift while the new
            // maximum is less than 2^LAZY above it (any shift gives the same quotient in the end; probabilities then
            // reach 2^LAZY at most, which bfloat16 holds with its usual relative error), so the accumulated output
            // has to be rescaled only on the few tiles where a row's maximum jumps.
            const float m_cand = fmaxf(m_run, mx);
            const bool grow = m_cand > m_run + LAZY || m_run == -INFINITY;
            const float m_new = grow ? m_cand : m_run;
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = attn::fast_exp2(m_run - m_use);  // 1 where the shift stays
            const bool rescale = grow && m_run != -INFINITY;  // (a row that has seen no key yet has an output of zeros)
            m_run = m_new;
            PH(2)
            // the probabilities (a masked score is -inf: its probability is exactly 0), two to a word: the second
            // product's A operand, stored into the row's lane of tensor memory once the product before has read its own
            unsigned pw[BN / 2];
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};  // four chains, two per packed add
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-m_use, -m_use);
#pragma unroll
            for (int c = 0; c < BN / 8; ++c) {
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const float2 x = __ffma2_rn(make_float2(v[c * 8 + i], v[c * 8 + i + 1]), scale2, shift2);
                    v[c * 8 + i] = attn::fast_exp2(x.x);
                    v[c * 8 + i + 1] = attn::fast_exp2(x.y);
                    sum2[(i >> 1) & 1] = __fadd2_rn(sum2[(i >> 1) & 1], make_float2(v[c * 8 + i], v[c * 8 + i + 1]));
                }
                pw[4 * c] = attn::pack_bf16(v[c * 8], v[c * 8 + 1]);
                pw[4 * c + 1] = attn::pack_bf16(v[c * 8 + 2], v[c * 8 + 3]);
                pw[4 * c + 2] = attn::pack_bf16(v[c * 8 + 4], v[c * 8 + 5]);
                pw[4 * c + 3] = attn::pack_bf16(v[c * 8 + 6], v[c * 8 + 7]);
            }
            l_run = l_run * alpha + ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y));
            PH(3)
            // The product of the tile before has had this tile's softmax to finish in.  Its barrier is waited for at
            // every tile, needed or not: a phase is told from the one two before it only by its parity, and a warp
            // that skipped phases could take an old one for the one it wants.
            // It has also read the probabilities of the tile before, whose place this tile's take below.
            if (j > 0) {
                ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&o_full, (j - 1) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            }
            if (__any_sync(0xffffffffu, rescale)) {
                // this tile's product must not start before the rows are rescaled: the issuer learns of the
                // probabilities only below
                float o[HD];
                umma::tmem_ld64(o_taddr, o);
                const float a = rescale ? alpha : 1.f;
                const float2 a2 = make_float2(a, a);
#pragma unroll
                for (int i = 0; i < HD; i += 2) {
                    const float2 r = __fmul2_rn(make_float2(o[i], o[i + 1]), a2);
                    o[i] = r.x;
                    o[i + 1] = r.y;
                }
                umma::tmem_st64(o_taddr, o);
            }
            PH(4)
            umma::tmem_st32(lane_base + P_COL, pw);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full);
            PH(5)
        }
#ifdef ATT_PROF
        if (threadIdx.x == 0 && blockIdx.x == 3 && (blockIdx.y % 5) == 0)
            printf("tile %d n_tiles %d: per tile wait_s %lld ld %lld max %lld exp+store %lld o_wait %lld arrive %lld total %lld\n", tile, n_tiles,
                   pc[0] / n_tiles, pc[1] / n_tiles, pc[2] / n_tiles, pc[3] / n_tiles, pc[4] / n_tiles, pc[5] / n_tiles,
                   (pc[0] + pc[1] + pc[2] + pc[3] + pc[4] + pc[5]) / n_tiles);
#endif
        float o[HD];
        if (ok && n_tiles > 0) {
            ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&o_full, (n_tiles - 1) & 1));
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                static_assert(HD == 64, "the output is read with one 64-column load");
                umma::tmem_ld64(o_taddr, o);
            }
        }
        if (!ok) {
            if (lane == 0) fail();
        } else if (row_ok && n_tiles > 0) {
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
        for (int j = max(0, n_tiles - STAGES); j < n_tiles; ++j) {
            tma::mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1);
            tma::mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1);
        }
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
    const CUtensorMap* kvmap = tma::cached_map_2d_bf16(pool, (uint64_t)kv_rows, HD, HD, (uint32_t)page_size, HD, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!kvmap) return LLM_ERR_UNSUPPORTED;
    TcParams tp = {};
    tp.a.q = (const __nv_bfloat16*)q;
    tp.a.q_stride = q_stride;
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
    constexpr size_t smem = 1024 + (size_t)STAGES * STAGE_BYTES;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_pdl(attention_tcgen05_kernel, dim3((unsigned)H, (unsigned)y), dim3(THREADS), smem, stream, tp, *kvmap);
}
