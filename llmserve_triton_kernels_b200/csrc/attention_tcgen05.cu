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

constexpr int BM = 128, BN = 64, THREADS = 256, TMEM_COLS = 256;
constexpr float LAZY = 8.f;  // log2 of how far a row's maximum may rise before its shift follows

// What differs between the head sizes.  256 columns of tensor memory a CTA (two CTAs share an SM's 512), two
// bfloat16 to a column where an A operand lies:
//   head size 64 : two tiles of scores [0, 64), [64, 128); the output [128, 192); the queries [192, 224); a tile's
//                  probabilities [224, 256).  Three stages of keys and of values (16 KB a stage): 49 KB of shared memory.
//   head size 128: one tile of scores [0, 64); the output [64, 192); probabilities [192, 224).  The queries do not fit
//                  and stay in shared memory (32 KB, the first product's A operand from there); two stages of keys
//                  and of values (32 KB a stage): 97 KB.  With one buffer of scores the product of tile j+1 starts when
//                  the softmax has read tile j; the other CTA of the SM fills the gap.
template <int HD>
struct Shape {
    static constexpr bool Q_IN_TMEM = HD == 64;
    static constexpr int S_BUFFERS = HD == 64 ? 2 : 1, STAGES = HD == 64 ? 3 : 2;
    static constexpr int O_COL = S_BUFFERS * BN, Q_COL = O_COL + HD, P_COL = Q_IN_TMEM ? Q_COL + HD / 2 : O_COL + HD;
    static constexpr int HALVES = HD / 64;                // 64-wide pieces of a row of keys, values, queries: one TMA box each
    static constexpr int K_BYTES = BN * HD * 2, STAGE_BYTES = 2 * K_BYTES, Q_BYTES = Q_IN_TMEM ? 0 : BM * HD * 2;
    static constexpr size_t SMEM = 1024 + (size_t)Q_BYTES + (size_t)STAGES * STAGE_BYTES;
    static_assert(P_COL + BN / 2 <= TMEM_COLS, "tensor memory");
};

struct TcParams {
    AttnParams a;
    int min_tokens;         // requests with fewer tokens are other kernels'
    int tiles_per_request;  // 128-token tiles of the longest request
    int* error_flag;
};

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) { tma::mbar_arrive(bar); }

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attention_tcgen05_kernel(const TcParams tp, const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kvmap) {
    using Sh = Shape<HD>;
    constexpr int STAGES = Sh::STAGES, NBUF = Sh::S_BUFFERS, K_BYTES = Sh::K_BYTES, STAGE_BYTES = Sh::STAGE_BYTES, HALVES = Sh::HALVES;
    constexpr int O_COL = Sh::O_COL, Q_COL = Sh::Q_COL, P_COL = Sh::P_COL;
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
    unsigned char* q_s = base;                // [halves][128 rows][64]: head size 128 only
    unsigned char* kv_s = base + Sh::Q_BYTES;  // [STAGES][keys | values], each [halves][64 keys][64]
    __shared__ __align__(8) unsigned long long q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES], s_full[NBUF], s_empty[NBUF], p_full, o_full;
    __shared__ unsigned tmem_base;
    __shared__ int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        tma::mbar_init(&q_full, Sh::Q_IN_TMEM ? 4 : 1);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            tma::mbar_init(&k_full[s], 1);
            tma::mbar_init(&k_empty[s], 1);
            tma::mbar_init(&v_full[s], 1);
            tma::mbar_init(&v_empty[s], 1);
        }
#pragma unroll
        for (int b = 0; b < NBUF; ++b) {
            tma::mbar_init(&s_full[b], 1);
            tma::mbar_init(&s_empty[b], 4);
        }
        tma::mbar_init(&p_full, 4);
        tma::mbar_init(&o_full, 1);
        gave_up = 0;
        tma::mbar_fence_init();
        tma::prefetch_map(&kvmap);
        if (!Sh::Q_IN_TMEM) tma::prefetch_map(&qmap);
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
        if (!Sh::Q_IN_TMEM && !is_v && lane == 0) {
            tma::mbar_expect_tx(&q_full, Sh::Q_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h) tma::load_2d(q_s + (size_t)h * (BM * 128), &qmap, head * HD + h * 64, q_begin + row0, &q_full);
        }
        // One box per page and 64-wide piece, each issued by a lane of its own (a thread's TMA instructions follow one another slowly;
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
            const int in_tile = lane / HALVES, half = lane % HALVES;
            const int page = __shfl_sync(0xffffffffu, my_page, (idx0 - loaded_from + in_tile) & 31);
            if (alive && in_tile < pages_per_tile) {
                unsigned char* dst = kv_s + (size_t)s * STAGE_BYTES + (size_t)is_v * K_BYTES + (size_t)half * (BN * 128) + (size_t)in_tile * ps * 128;
                tma::load_2d(dst, &kvmap, half * 64, ((page * 2 + (int)is_v) * p.KV + kvh) * ps, &full[s]);
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
                ok = tma::mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1) &&
                     (j < NBUF || tma::mbar_wait(&s_empty[j % NBUF], ((j / NBUF) - 1) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* k_tile = kv_s + (size_t)(j % STAGES) * STAGE_BYTES;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {  // 16 of the head's lanes a step: piece k / 4 of the tile, 32 bytes further per step
                    const unsigned long long k_desc = umma::desc_sw128(k_tile + (size_t)(k / 4) * (BN * 128)) + 2 * (k % 4);
                    if constexpr (Sh::Q_IN_TMEM) {
                        umma::mma_bf16_ts(tmem_base + (j % NBUF) * BN, q_tmem + 8 * k, k_desc, IDESC_QK, k != 0);
                    } else {
                        const unsigned long long q_desc = umma::desc_sw128(q_s + (size_t)(k / 4) * (BM * 128)) + 2 * (k % 4);
                        umma::mma_bf16(tmem_base + (j % NBUF) * BN, q_desc, k_desc, IDESC_QK, k != 0);
                    }
                }
                umma::commit(&s_full[j % NBUF]);
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
                // (a head of 128 lanes is two such pieces side by side, BN * 128 bytes apart: the leading offset)
                const unsigned long long v_desc = umma::desc_sw128(kv_s + (size_t)s * STAGE_BYTES + K_BYTES, (HALVES > 1 ? BN * 128 : 1024) >> 4);
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
        if constexpr (Sh::Q_IN_TMEM) {  // the row's queries, as they lie in memory (two to a word), into the row's lane of tensor memory
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
            ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&s_full[j % NBUF], (j / NBUF) & 1));
            PH(0)
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const bool whole = key_base + BN - 1 <= tile_pos_min && key_base >= tile_lo_max && rows_here == BM;
            // the keys of this tile that the row sees are those with index (within the tile) in [see_lo, see_hi]
            const int see_lo = row_ok ? lo - key_base : BN, see_hi = row_ok ? pos - key_base : -1;
            // the row's 64 scores in one load; once they are in registers the buffer may take the scores two tiles on
            static_assert(BN == 64, "the softmax reads a tile's scores with one 64-column load");
            float v[BN];
            umma::tmem_ld64(lane_base + (j % NBUF) * BN, v);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[j % NBUF]);  // the buffer may take the scores of a later tile
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
                const float a = rescale ? alpha : 1.f;
                const float2 a2 = make_float2(a, a);
#pragma unroll 1
                for (int h = 0; h < HALVES; ++h) {
                    float o[64];
                    umma::tmem_ld64(o_taddr + 64 * h, o);
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        const float2 r = __fmul2_rn(make_float2(o[i], o[i + 1]), a2);
                        o[i] = r.x;
                        o[i + 1] = r.y;
                    }
                    umma::tmem_st64(o_taddr + 64 * h, o);
                }
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
        if (ok && n_tiles > 0) ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&o_full, (n_tiles - 1) & 1));
        if (!ok) {
            if (lane == 0) fail();
        } else if (n_tiles > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = 1.f / l_run;
            __nv_bfloat16* dst = p.out + (size_t)(q_begin + tok) * p.out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int h = 0; h < HALVES; ++h) {
                float o[64];
                umma::tmem_ld64(o_taddr + 64 * h, o);  // (by all lanes of the warp: the load is the warp's)
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint4 u;
                        u.x = attn::pack_bf16(o[c * 8] * inv, o[c * 8 + 1] * inv);
                        u.y = attn::pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
                        u.z = attn::pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
                        u.w = attn::pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + 64 * h + c * 8) = u;
                    }
                }
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

namespace {
template <int HD>
int launch_tcgen05(const TcParams& tp, const void* q, int q_stride, int n_tokens, const void* pool, long long kv_rows, int page_size,
                   unsigned grid_y, cudaStream_t stream) {
    using Sh = Shape<HD>;
    // one box of keys or values: a page's rows, 64 of the head's lanes; one box of queries: 128 tokens, 64 lanes of a head
    const CUtensorMap* kvmap = tma::cached_map_2d_bf16(pool, (uint64_t)kv_rows, HD, HD, (uint32_t)page_size, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    const CUtensorMap* qmap = Sh::Q_IN_TMEM ? kvmap
                                            : tma::cached_map_2d_bf16(q, (uint64_t)n_tokens, (uint64_t)tp.a.H * HD, (uint64_t)q_stride, BM, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!kvmap || !qmap) return LLM_ERR_UNSUPPORTED;
    static bool configured = false;  // per head size
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sh::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_pdl(attention_tcgen05_kernel<HD>, dim3((unsigned)tp.a.H, grid_y), dim3(THREADS), Sh::SMEM, stream, tp, *qmap, *kvmap);
}
}  // namespace

// Attention of the requests that bring at least min_tokens tokens (others are left untouched: another kernel's).
// q: bfloat16 rows of q_stride elements that start with the H query heads; out: [tokens, H * D] with row stride
// out_stride; pool: one layer's plane [pool_pages, 2, KV, page_size, D]; max_tokens: the most tokens of any request.
// Takes head sizes 64 and 128, pages of 8, 16, 32 or 64 keys, 16-byte aligned rows; else LLM_ERR_UNSUPPORTED (nothing ran).
LLM_EXPORT int llm_attention_tcgen05(const void* q, int q_stride, void* out, int out_stride, const void* pool, long long pool_pages,
                                     const int* page_table, int table_width, const int* cu_tokens, const int* ctx_lens,
                                     int requests, int n_tokens, int H, int KV, int D, int page_size, int window, float scale,
                                     int min_tokens, int max_tokens, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0 || requests <= 0 || max_tokens < min_tokens) return 0;
    if ((D != 64 && D != 128) || (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64)) return LLM_ERR_UNSUPPORTED;
    if (H <= 0 || KV <= 0 || H % KV || table_width <= 0 || min_tokens < 1 || !(scale > 0.f)) return LLM_ERR_BAD_ARGUMENT;
    if ((q_stride & 7) || (out_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)pool & 127) || q_stride < H * D)
        return LLM_ERR_UNSUPPORTED;
    const long long kv_rows = pool_pages * 2 * KV * page_size;
    if (kv_rows <= 0 || kv_rows > 0x7fffffffLL) return LLM_ERR_UNSUPPORTED;
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
    return D == 64 ? launch_tcgen05<64>(tp, q, q_stride, n_tokens, pool, kv_rows, page_size, (unsigned)y, stream)
                   : launch_tcgen05<128>(tp, q, q_stride, n_tokens, pool, kv_rows, page_size, (unsigned)y, stream);
}
