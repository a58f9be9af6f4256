// The tensor-core attention over the paged cache as a device function: one CTA of 4 warps computes
// one (request, key/value head, row tile, split of the keys).  Used by the attention kernels of
// attention_mma.cu.
#pragma once

#include "common.cuh"
#include "timeline.cuh"
#include "tma.cuh"

namespace attn {


constexpr int SMALL_ROWS = 16;  // requests with at most this many rows go to the KEYS shape
constexpr int SMALL_MIN_KEYS = 768;  // keys a split of that shape takes at least (three tiles of 256): measured best of 512, 768, 1024, 2048

// The threads that compute a tile meet here.  A named barrier, not __syncthreads: inside the fused decode
// kernel the tile is computed by four of the CTA's eight warps.
template <int THREADS>
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 9, %0;\n" ::"n"(THREADS) : "memory"); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {  // 2^x by the special-function unit: exp2(-inf) = 0, relative error about 2^-22
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

struct AttnParams {
    const __nv_bfloat16* q;
    int q_stride;
    __nv_bfloat16* out;
    int out_stride;
    const __nv_bfloat16* pool;
    const int* page_table;
    int table_width;
    const int* cu_tokens;
    const int* ctx_lens;
    int H, KV, G, page_size, window;
    int tiles_per_request;  // gridDim.z = requests * tiles_per_request
    float scale_log2;       // softmax scale * log2(e)
    int splits;             // gridDim.x
    float* part_o;          // [tokens, H, splits, D], relative to the split's max
    float* part_ml;         // [tokens, H, splits, 2]: (max in the base-2 domain, sum)
    int* counters;          // [requests * KV] zeros: how many splits of a (request, kv head) have finished
    int skip_tokens_from;   // requests that bring at least this many tokens are another kernel's (0: none are)
    int* error_flag;        // host-visible word set to 1 if a bounded wait gave up, or null
};

// Floats between the rows of a warp's share where the split-key shape merges its warps through shared memory.
__host__ __device__ constexpr int merge_pitch(int D) { return D + 8; }

// Whether a shape brings its keys row by row with bulk copies (see attention_tile), and the elements between the rows of a
// tile in shared memory.
// Rows of 256 bytes and more only: with 128-byte rows (head size 64) the bulk copies themselves were the slower way
// (35.0 against 22.4 us for 64 requests of 1,600 keys), with 256-byte rows the faster (41 against 50 us at head size 128).
__host__ __device__ constexpr bool bulk_rows(int D, int row_warps, int key_warps, int bn) { return row_warps == 1 && key_warps > 1 && bn == 16 && D >= 128; }
__host__ __device__ constexpr int tile_pitch(int D, int row_warps, int key_warps, int bn) { return bulk_rows(D, row_warps, key_warps, bn) ? D + 8 : D; }

__device__ __forceinline__ void bulk_copy_row(void* smem, const void* gmem, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(bytes), "r"((unsigned)__cvta_generic_to_shared(bar)) : "memory");
}

constexpr float LAZY_RISE = 8.f;  // log2 of how far a row's maximum may rise before the split-key shape moves the row's shift

// Stages of the key/value ring: four where shared memory allows, three for the largest tiles.
__host__ __device__ constexpr int stages_of(int D, int key_warps) { return D <= 64 ? 4 : 3; }

// D: head size.  ROW_WARPS x KEY_WARPS warps.  BN: keys per warp and tile.
template <int D, int ROW_WARPS, int KEY_WARPS, int BN, int STAGES = stages_of(D, KEY_WARPS)>
__device__ __forceinline__ void attention_tile(const AttnParams& p, int split, int kvh, int r, int tile, unsigned char* smem_raw,
                                               bool use_pdl TL(, tl::Marks* marks = nullptr)) {
    constexpr int THREADS = 32 * ROW_WARPS * KEY_WARPS;
    constexpr int BM = 16 * ROW_WARPS;   // rows of the CTA
    constexpr int BNC = BN * KEY_WARPS;  // keys of one CTA tile
    constexpr int CHUNKS = D / 8;        // 16-byte pieces of a key row
    constexpr int SWZ = CHUNKS >= 8 ? 7 : CHUNKS - 1;
    constexpr int KSTEPS = D / 16;
    constexpr int NT_S = BN / 8;  // 8-key tiles of a warp's scores
    constexpr int NT_O = D / 8;   // 8-wide tiles of the output
    constexpr bool SMALL = KEY_WARPS > 1;
    // The split-key shape with 16 keys a warp: a warp's 32 lanes bring exactly the 16 key rows and 16 value rows that
    // the warp itself reads, so no meeting of the CTA is needed between tiles (WARP_PRIVATE).  At head size 128 and more
    // each lane brings its row as ONE bulk copy (cp.async.bulk, completion counted on a barrier of the warp's own) instead
    // of D / 8 sixteen-byte copies: the copies' instructions, not their bytes, were what this shape waited for (the
    // load/store unit's queue).  A bulk copy cannot swizzle, so rows then lie PITCH = D + 8 elements apart: eight rows'
    // 16-byte pieces fall into eight different groups of four banks.
    constexpr bool BULK = bulk_rows(D, ROW_WARPS, KEY_WARPS, BN);
    constexpr int PITCH = tile_pitch(D, ROW_WARPS, KEY_WARPS, BN);
    // STAGES tiles in flight: a tile's latency is a page lookup plus a trip to HBM
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [STAGES][BNC][PITCH]
    __nv_bfloat16* v_s = k_s + STAGES * BNC * PITCH;                  // [STAGES][BNC][PITCH]
    __shared__ __align__(8) unsigned long long rows_full[BULK ? KEY_WARPS : 1][STAGES];  // per warp and stage

    const int q_begin = p.cu_tokens[r], q_len = p.cu_tokens[r + 1] - q_begin;
    const int G = p.G, rows_total = q_len * G;
    if ((rows_total <= SMALL_ROWS) != SMALL) return;
    if (p.skip_tokens_from > 0 && q_len >= p.skip_tokens_from) return;
    const int row0 = tile * BM;
    if (row0 >= rows_total) return;
    const int ctx = p.ctx_lens[r], pos0 = ctx - q_len;
    const int tid = threadIdx.x & (THREADS - 1), warp = tid >> 5, lane = tid & 31;
    const int row_warp = warp % ROW_WARPS, key_warp = warp / ROW_WARPS;
    const int qr = lane >> 2, qc = lane & 3;

    // the two rows this thread holds pieces of
    int row_tok[2], row_pos[2], row_lo[2], row_head[2];
    bool row_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int rho = row0 + row_warp * 16 + qr + 8 * i;
        row_ok[i] = rho < rows_total;
        const int tok = row_ok[i] ? rho / G : 0;
        row_tok[i] = q_begin + tok;
        row_head[i] = kvh * G + (row_ok[i] ? rho - tok * G : 0);
        row_pos[i] = row_ok[i] ? pos0 + tok : -1;
        row_lo[i] = p.window > 0 ? max(0, row_pos[i] - p.window + 1) : 0;
    }
    // keys this CTA needs: from the window's start of its first token to its last token's position
    const int tok_first = row0 / G, tok_last = (min(rows_total, row0 + BM) - 1) / G;
    const int key_hi = pos0 + tok_last;
    const int key_lo = p.window > 0 ? max(0, pos0 + tok_first - p.window + 1) : 0;
    // a key tile needs no mask if every row of the CTA sees all of it (rows past the end are never written)
    const int tile_pos_min = pos0 + tok_first;
    const int tile_lo_max = p.window > 0 ? max(0, pos0 + tok_last - p.window + 1) : 0;
    const int tile_first = key_lo / BNC, tile_last = key_hi / BNC;
    // a split of the small shape takes at least SMALL_MIN_KEYS keys, so contexts up to that many keys are not
    // split however many splits the grid has (merging splits costs more than a few more tiles in a row); splits
    // beyond the last active one do nothing
    const int n_tiles = tile_last - tile_first + 1;
    const int per_split = max(SMALL ? (SMALL_MIN_KEYS + BNC - 1) / BNC : 1, (n_tiles + p.splits - 1) / p.splits);
    const int active_splits = (n_tiles + per_split - 1) / per_split;
    const int t_begin = tile_first + split * per_split;
    const int t_end = min(tile_last + 1, t_begin + per_split);
    if (SMALL && split >= active_splits) return;

    const int* table = p.page_table + (size_t)r * p.table_width;
    const size_t head_stride = (size_t)p.page_size * D;

    // one key row (or a fixed part of it) per thread: one page lookup and a few 16-byte copies per tile
    constexpr int TPK = THREADS / BNC;        // threads per key
    constexpr int CPT = CHUNKS / TPK;         // 16-byte pieces per thread
    static_assert(THREADS % BNC == 0 && CHUNKS % TPK == 0, "a key row must split evenly over its threads");
    const int load_key = tid / TPK, load_c0 = (tid % TPK) * CPT;
    constexpr bool WARP_PRIVATE = ROW_WARPS == 1 && TPK * BN == 32;  // thread tid copies key tid / TPK: warp w the keys [w BN, (w + 1) BN)
    // the page of this thread's key row in tile t (-1: the row lies outside the piece's keys and reads as zeros);
    // looked up one tile ahead of the copies that use it, so that a tile's latency is one trip to memory, not two
    auto page_of = [&](int t) -> int {
        const int j = t * BNC + load_key;
        return t < t_end && j >= key_lo && j <= key_hi ? table[j / p.page_size] : -1;
    };
    // ---- the bulk loader of the split-key shape: lane l < 16 brings key row l of the warp's sixteen, lane 16 + l value row l
    const int my_row = lane & 15, is_v = lane >> 4;
    unsigned long long* my_full = rows_full[BULK ? key_warp : 0];
    bool waits_ok = true;
    if constexpr (BULK) {
        if (lane == 0) {
#pragma unroll
            for (int s2 = 0; s2 < STAGES; ++s2) tma::mbar_init(&my_full[s2], 1);
            tma::mbar_fence_init();
        }
        __syncwarp();
    }
    auto bulk_page_of = [&](int t) -> int {  // the page of this lane's row in tile t, -1 if the row is not among the piece's keys
        const int j = t * BNC + key_warp * BN + my_row;
        return t < t_end && j >= key_lo && j <= key_hi ? table[j / p.page_size] : -1;
    };
    auto bulk_expect = [&](int t, int stage) {  // lane 0: the bytes that the warp's rows of tile t will bring
        const int lo = max(t * BNC + key_warp * BN, key_lo), hi = min(t * BNC + key_warp * BN + BN - 1, key_hi);
        const int rows = t < t_end && hi >= lo ? hi - lo + 1 : 0;
        tma::mbar_expect_tx(&my_full[stage], (unsigned)(rows * 2 * D * 2));
    };
    auto bulk_row = [&](int t, int stage, int page) {  // this lane's row of tile t: copied, or zeros where there is no such key
        const int j = t * BNC + key_warp * BN + my_row;
        __nv_bfloat16* dst = (is_v ? v_s : k_s) + (size_t)(stage * BNC + key_warp * BN + my_row) * PITCH;
        if (page >= 0) {
            const size_t off = ((size_t)(page * 2 + is_v) * p.KV + kvh) * head_stride + (size_t)(j % p.page_size) * D;
            bulk_copy_row(dst, p.pool + off, D * 2, &my_full[stage]);
        } else {
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // (a later tile's copy may land on these bytes)
        }
    };
    auto load_tile = [&](int t, int stage, int page) {
        const int j = t * BNC + load_key;
        const bool valid = page >= 0;
        size_t off = 0;
        if (valid) off = ((size_t)(page * 2) * p.KV + kvh) * head_stride + (size_t)(j % p.page_size) * D;
        const int dst_row = (stage * BNC + load_key) * D;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = load_c0 + i;
            const int dst = dst_row + ((c ^ (load_key & SWZ)) * 8);
            cp_async16(k_s + dst, p.pool + off + c * 8, valid);
            cp_async16(v_s + dst, p.pool + off + (size_t)p.KV * head_stride + c * 8, valid);
        }
    };

    // the pages of the first tiles: the page table is the step's own, written by no kernel, so the lookups go out
    // before the wait for the kernel in front
    int first_pages[STAGES - 1];
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) first_pages[i] = BULK ? bulk_page_of(t_begin + i) : page_of(t_begin + i);
    int page_next = BULK ? bulk_page_of(t_begin + STAGES - 1) : page_of(t_begin + STAGES - 1);

    // One commit group per tile, empty past the end, so that the wait in the loop counts tiles.  A tile whose keys
    // all lie before the step's first position was written by earlier steps: its copies go out before the wait for
    // the kernel in front too (such tiles are the first ones, so the groups stay in the order of the tiles).
    bool asked[STAGES - 1];
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if constexpr (BULK) {
            // row by row: a row that earlier steps wrote (or that does not exist) goes out now, the step's own rows behind the wait
            const int j = (t_begin + i) * BNC + key_warp * BN + my_row;
            if (lane == 0) bulk_expect(t_begin + i, i);
            asked[i] = use_pdl && (j < pos0 || first_pages[i] < 0);
            if (asked[i]) bulk_row(t_begin + i, i, first_pages[i]);
        } else {
            asked[i] = use_pdl && t_begin + i < t_end && (t_begin + i + 1) * BNC <= pos0;
            if (asked[i]) {
                load_tile(t_begin + i, i, first_pages[i]);
                cp_async_commit();
            }
        }
    }
    // up to here only the step's descriptor arrays and keys of earlier steps were read, which no kernel of this step
    // writes; the queries and the step's own keys come from the kernels before this one
    if (use_pdl) {
        pdl_trigger();
        TL(if (marks) marks->mark(1);)
        pdl_wait();
        TL(if (marks) marks->mark(2);)
    }
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (asked[i]) continue;
        if constexpr (BULK) {
            bulk_row(t_begin + i, i, first_pages[i]);
        } else {
            if (t_begin + i < t_end) load_tile(t_begin + i, i, first_pages[i]);
            cp_async_commit();
        }
    }

    // query fragments, straight from global memory
    unsigned qa[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int which = i & 1;
            const __nv_bfloat16* src = p.q + (size_t)row_tok[which] * p.q_stride + (size_t)row_head[which] * D +
                                       ks * 16 + (i >> 1) * 8 + qc * 2;
            qa[ks][i] = row_ok[which] ? *reinterpret_cast<const unsigned*>(src) : 0u;
        }

    float oacc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int t = t_begin; t < t_end; ++t) {
        const int stage = (t - t_begin) % STAGES;
        if constexpr (BULK) {
            // the warp's rows of tile t have landed (every lane looks at the warp's barrier: bounded); the zeros that lanes
            // stored themselves are shown to the warp by __syncwarp, which also says that the stage refilled next (the
            // one read in the round before) is no longer read
            if (waits_ok && !tma::mbar_wait(&my_full[stage], ((t - t_begin) / STAGES) & 1)) {
                waits_ok = false;
                if (p.error_flag) atomicExch(p.error_flag, 1);
            }
            __syncwarp();
            const int ahead = t + STAGES - 1, ahead_stage = (t - t_begin + STAGES - 1) % STAGES;
            if (ahead < t_end) {
                if (lane == 0) bulk_expect(ahead, ahead_stage);
                bulk_row(ahead, ahead_stage, page_next);
            }
            page_next = bulk_page_of(t + STAGES);
        } else {
            cp_async_wait<STAGES - 2>();  // tile t has landed (this thread's copies) ...
            // ... everyone's; and the stage refilled next is no longer read.  Where a warp's threads copy exactly the
            // keys that the warp itself reads, "everyone" is the warp: its tiles follow one another without a meeting of
            // the CTA, and a warp whose keys include the step's own (copied after the wait for the kernel in front) does
            // not hold up the others
            if constexpr (WARP_PRIVATE) __syncwarp();
            else cta_sync<THREADS>();
            if (t + STAGES - 1 < t_end) load_tile(t + STAGES - 1, (t - t_begin + STAGES - 1) % STAGES, page_next);
            cp_async_commit();
            page_next = page_of(t + STAGES);
        }
        const __nv_bfloat16* ks_tile = k_s + (stage * BNC + key_warp * BN) * PITCH;
        const __nv_bfloat16* vs_tile = v_s + (stage * BNC + key_warp * BN) * PITCH;
        // where 16-byte piece `chunk` of row `key` of the warp's part of the tile lies: swizzled, or rows PITCH apart
        auto piece = [&](int key, int chunk) { return BULK ? key * PITCH + chunk * 8 : key * D + ((chunk ^ (key & SWZ)) * 8); };
        const int key_base = t * BNC + key_warp * BN;

        // scores: S = Q K^T
        float sacc[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
        const int mi = lane >> 3, ri = lane & 7;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int np = 0; np < NT_S / 2; ++np) {
                const int key = np * 16 + (mi >> 1) * 8 + ri;  // row of the tile; key_warp*BN is a multiple of 8
                const int chunk = ks * 2 + (mi & 1);
                unsigned b[4];
                ldmatrix_x4(b, ks_tile + piece(key, chunk));
                mma_bf16(sacc[2 * np], qa[ks], b[0], b[1]);
                mma_bf16(sacc[2 * np + 1], qa[ks], b[2], b[3]);
            }
        }
        // mask (only in tiles that some row does not see whole), running max and sum
        float mx[2] = {-INFINITY, -INFINITY};
        const bool whole = key_base + BN - 1 <= tile_pos_min && key_base >= tile_lo_max;
        if (whole) {
#pragma unroll
            for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sacc[nt][e] *= p.scale_log2;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sacc[nt][e]);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int j = key_base + nt * 8 + qc * 2 + (e & 1);
                    const bool visible = j <= row_pos[i] && j >= row_lo[i];
                    sacc[nt][e] = visible ? sacc[nt][e] * p.scale_log2 : -INFINITY;
                    mx[i] = fmaxf(mx[i], sacc[nt][e]);
                }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            // the row keeps its shift while its maximum has risen by less than 2^LAZY_RISE since the shift was set (any
            // shift gives the same quotient in the end; probabilities then reach 2^LAZY_RISE at most): the sums so far
            // are rescaled on few tiles only
            const float m_cand = fmaxf(m_run[i], mx[i]);
            const bool grow = SMALL && m_run[i] != -INFINITY ? m_cand > m_run[i] + LAZY_RISE : true;
            const float m_new = grow ? m_cand : m_run[i];
            m_use[i] = m_new == -INFINITY ? 0.f : m_new;
            alpha[i] = fast_exp2(m_run[i] - m_use[i]);  // exactly 1 where the shift stays
            m_run[i] = m_new;
            l_run[i] *= alpha[i];
        }
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = fast_exp2(sacc[nt][e] - m_use[e >> 1]);
                sacc[nt][e] = pv;
                l_run[e >> 1] += pv;
            }
        if (!SMALL || __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) {
                oacc[nt][0] *= alpha[0];
                oacc[nt][1] *= alpha[0];
                oacc[nt][2] *= alpha[1];
                oacc[nt][3] *= alpha[1];
            }
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            unsigned pa[4];
            pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
            pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
            pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
            pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < NT_O / 2; ++dp) {
                const int key = kk * 16 + (mi & 1) * 8 + ri;
                const int chunk = dp * 2 + (mi >> 1);
                unsigned b[4];
                ldmatrix_x4_trans(b, vs_tile + piece(key, chunk));
                mma_bf16(oacc[2 * dp], pa, b[0], b[1]);
                mma_bf16(oacc[2 * dp + 1], pa, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    cta_sync<THREADS>();  // the ring is free (the small shape merges its warps through it)
    TL(if (marks) marks->mark(3);)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }

    if constexpr (!SMALL) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!row_ok[i]) continue;
            if (p.splits == 1) {
                const float inv = 1.f / l_run[i];
                __nv_bfloat16* dst = p.out + (size_t)row_tok[i] * p.out_stride + (size_t)row_head[i] * D + qc * 2;
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt)
                    *reinterpret_cast<unsigned*>(dst + nt * 8) = pack_bf16(oacc[nt][2 * i] * inv, oacc[nt][2 * i + 1] * inv);
            } else {
                const size_t slot = ((size_t)row_tok[i] * p.H + row_head[i]) * p.splits + split;
                float* dst = p.part_o + slot * D + qc * 2;
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    dst[nt * 8] = oacc[nt][2 * i];
                    dst[nt * 8 + 1] = oacc[nt][2 * i + 1];
                }
                if (qc == 0) {
                    p.part_ml[slot * 2] = m_run[i];
                    p.part_ml[slot * 2 + 1] = l_run[i];
                }
            }
        }
    } else {
        // merge the warps' shares of the keys through shared memory (the key tiles are done with).  A row of a share
        // is MERGE_PITCH floats long: with D, the eight rows that a warp stores at once would meet in one bank (their
        // places are 64 or 128 floats apart), eight times over for every one of the 2 x D / 8 stores; with D + 8 and
        // two values a store, each half warp's sixteen stores fall into sixteen different pairs of banks.
        constexpr int DP = merge_pitch(D);
        float* o_sm = reinterpret_cast<float*>(smem_raw);    // [KEY_WARPS][16][DP]
        float* ml_sm = o_sm + KEY_WARPS * 16 * DP;           // [KEY_WARPS][16][2]
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = qr + 8 * i;
            if (row >= rows_total) continue;  // (a decode step has no more rows than the group has heads)
            float* dst = o_sm + (key_warp * 16 + row) * DP + qc * 2;
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(oacc[nt][2 * i], oacc[nt][2 * i + 1]);
            if (qc == 0) {
                ml_sm[(key_warp * 16 + row) * 2] = m_run[i];
                ml_sm[(key_warp * 16 + row) * 2 + 1] = l_run[i];
            }
        }
        cta_sync<THREADS>();
        // each row's weights of the warps' shares first (one thread per (row, warp): a few exponentials in all, not one per
        // element), then the weighted sums, an element per thread, over the rows that exist only
        float* f_sm = ml_sm + KEY_WARPS * 16 * 2;  // [16][KEY_WARPS] weight of a warp's share; then [16] max, [16] sum
        float* row_m = f_sm + 16 * KEY_WARPS;
        float* row_l = row_m + 16;
        for (int idx = tid; idx < rows_total * KEY_WARPS; idx += THREADS) {
            const int row = idx / KEY_WARPS, w = idx - row * KEY_WARPS;
            float m = -INFINITY;
#pragma unroll
            for (int w2 = 0; w2 < KEY_WARPS; ++w2) m = fmaxf(m, ml_sm[(w2 * 16 + row) * 2]);
            const float m_use = m == -INFINITY ? 0.f : m;
            f_sm[row * KEY_WARPS + w] = exp2f(ml_sm[(w * 16 + row) * 2] - m_use);
            if (w == 0) row_m[row] = m;
        }
        cta_sync<THREADS>();
        for (int idx = tid; idx < rows_total * D; idx += THREADS) {
            const int row = idx / D, d = idx - row * D;
            float o = 0.f, l = 0.f;
#pragma unroll
            for (int w = 0; w < KEY_WARPS; ++w) {  // a fixed order
                const float f = f_sm[row * KEY_WARPS + w];
                o += o_sm[(w * 16 + row) * DP + d] * f;
                l += ml_sm[(w * 16 + row) * 2 + 1] * f;
            }
            const int tok = row / G, head = kvh * G + (row - tok * G);
            if (active_splits == 1) {
                p.out[(size_t)(q_begin + tok) * p.out_stride + (size_t)head * D + d] = __float2bfloat16_rn(o / l);
            } else {
                const size_t slot = ((size_t)(q_begin + tok) * p.H + head) * p.splits + split;
                p.part_o[slot * D + d] = o;
                if (d == 0) {
                    p.part_ml[slot * 2] = row_m[row];
                    p.part_ml[slot * 2 + 1] = l;
                }
            }
        }
        if (active_splits > 1) {
            // the split that finishes last merges all of them: no second launch
            __shared__ int ticket;
            __threadfence();
            cta_sync<THREADS>();
            if (tid == 0) ticket = atomicAdd(&p.counters[r * p.KV + kvh], 1);
            cta_sync<THREADS>();
            if (ticket != active_splits - 1) return;
            __threadfence();
            // factors of every (row, split) first, side by side, then the weighted sums
            float* f_sm = reinterpret_cast<float*>(smem_raw);  // [rows][splits] factor, then [rows] 1 / sum
            float* inv_sm = f_sm + SMALL_ROWS * 32;
            for (int row = tid; row < rows_total; row += THREADS) {
                const int tok = row / G, head = kvh * G + (row - tok * G);
                const size_t slot = ((size_t)(q_begin + tok) * p.H + head) * p.splits;
                float m = -INFINITY;
                for (int s2 = 0; s2 < active_splits; ++s2) m = fmaxf(m, __ldcg(&p.part_ml[(slot + s2) * 2]));
                const float m_use = m == -INFINITY ? 0.f : m;
                float l = 0.f;
                for (int s2 = 0; s2 < active_splits; ++s2) {
                    const float f = exp2f(__ldcg(&p.part_ml[(slot + s2) * 2]) - m_use);
                    f_sm[row * 32 + s2] = f;
                    l += __ldcg(&p.part_ml[(slot + s2) * 2 + 1]) * f;
                }
                inv_sm[row] = 1.f / l;
            }
            cta_sync<THREADS>();
            for (int idx = tid; idx < rows_total * D; idx += THREADS) {
                const int row = idx / D, d = idx - row * D;
                const int tok = row / G, head = kvh * G + (row - tok * G);
                const size_t slot = ((size_t)(q_begin + tok) * p.H + head) * p.splits;
                float o = 0.f;
#pragma unroll 4
                for (int s2 = 0; s2 < active_splits; ++s2) o += __ldcg(&p.part_o[(slot + s2) * D + d]) * f_sm[row * 32 + s2];
                p.out[(size_t)(q_begin + tok) * p.out_stride + (size_t)head * D + d] = __float2bfloat16_rn(o * inv_sm[row]);
            }
            if (tid == 0) p.counters[r * p.KV + kvh] = 0;  // ready for the next launch
        }
    }
}

}  // namespace attn
