// The weight-streaming matrix product for few rows as device functions, used by the kernels of
// linear_decode.cu.
//
// A CTA of 8 warps; each warp streams tiles of 16 output features of its own through a private ring
// of TMA boxes (16 rows x 128 k, completion counted by the warp's own mbarriers).  The caller owns
// shared memory and the mbarriers (initialised once per kernel) and keeps, per warp, the count of
// boxes the ring has carried so far (`base`): slots and mbarrier phases go on from one product to
// the next.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "timeline.cuh"

namespace lin {


constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_RESIDUAL = 2, MODE_QKV = 3;

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Which row of a box (of eight, or of each eight of sixteen) holds the weights of MMA row g: rows g and g + 1 of the
// MMA are read by the same quarter of a warp, and in the swizzled box rows r and r + 4 use different banks.  The
// features of a tile are therefore numbered so: the thread that holds MMA row g holds feature feature_row(g).
__device__ __forceinline__ int feature_row(int g) { return ((g & 1) << 2) | (g >> 1); }

struct LinearParams {
    const __nv_bfloat16* x;
    const __nv_bfloat16* w;
    void* out;
    int M, N, K, ldx, ldo;
    const float* in_ss;  // [in_parts, M] partial sums of squares of the input's source rows, or null
    int in_parts;
    float in_eps;
    int up_offset;          // MODE_SWIGLU: row of w where the up matrix starts
    float* resid;           // MODE_RESIDUAL: [M, N] float32, updated in place
    const float* norm_w;    // MODE_RESIDUAL: [N] weight of the next norm
    __nv_bfloat16* xw_out;  // MODE_RESIDUAL: [M, N] = resid * norm_w
    float* ss_out;          // MODE_RESIDUAL: [tiles of 16 features, M]
    int* error_flag;        // set to 1 if a wait for a copy gave up (host-visible memory), or null
    int group;              // warps that share a tile: 1, 2, 4 or 8
    int slots;              // boxes of a warp's ring: 2 to SLOTS
    int ring_warps;         // warps that have a ring: the first ones of the CTA, those whose teams have tiles
    int red_floats;         // floats of shared memory for the teams' partial sums (red_floats() below)
    // MODE_QKV: w rows are [H query heads | KV key heads | KV value heads] x D; out is [M, H * D]
    const int* positions;   // [M]
    const float* rotary;    // [positions, D] = cos | sin halves, or null (no rotation)
    int rotary_rows;
    const int* slot_map;    // [M] page * page_size + offset of each token
    __nv_bfloat16* pool;    // [pages, 2, KV, page_size, D]
    int H, KV, D, page_size;
    int tl_launch;          // profiling builds: which launch this is
};

constexpr int SLOTS = 4;   // most boxes per warp, all in flight but for the moment in which one is read into registers;
                           // a product whose warps never have more than two boxes is given two (LinearParams::slots)
constexpr int BOXK = 128;  // k per box: a slot is 16 rows x 128 k = 4 KB
constexpr int SLOT_ELEMS = 16 * BOXK;
// elements of a slot: the box of weights and, where x rides with the boxes, the same 128 k of the MT token tiles of x
__host__ __device__ constexpr int slot_elems(int MT, bool ride) { return SLOT_ELEMS + (ride ? MT * 8 * BOXK : 0); }
constexpr int PIECES = BOXK / 32;
constexpr int X_PAD = 32;  // elements between the rows of x in shared memory: 8 tokens x 64 bytes hit 8 bank groups


constexpr int MT_MAX = 2;  // 8-token tiles a product may carry

// How many warps share a tile (1, 2, 4 or 8, splitting its k-blocks): the choice that leaves the busiest warp the
// fewest boxes to stream.  The warps of a CTA form WARPS / g teams, team j of CTA b takes tiles b + j grid,
// b + (j + WARPS / g) grid, ...; a team's warps put their partial sums into shared memory and meet once, when all of
// the team's tiles are done; a shared tile is counted as SHARE_COST boxes more.
constexpr float SHARE_COST = 1.0f;  // measured: 8 x 11264 x 2048 takes 10.8 us unshared, 10.9 us shared by 4 warps, 11.4 us by 8

inline int choose_group(int tiles, int kblocks, int grid, int max_shared_tiles_each = 1 << 30) {
    int best = 1;
    float best_cost = 1e30f;
    for (int g = 1; g <= WARPS; g *= 2) {
        const int teams = grid * (WARPS / g);
        const int tiles_each = (tiles + teams - 1) / teams, boxes_each = (kblocks + g - 1) / g;
        if (g > 1 && tiles_each > max_shared_tiles_each) continue;  // the partial sums' place in shared memory is limited
        const float cost = (float)tiles_each * ((float)boxes_each + (g > 1 ? SHARE_COST : 0.f));
        if (cost < best_cost) {
            best_cost = cost;
            best = g;
        }
    }
    return best;
}

// Floats of shared memory the teams' partial sums need: a place per (tile of a team, warp) when tiles are shared.
inline size_t red_floats(int tiles, int grid, int group, int MT) {
    if (group <= 1) return 0;
    const int teams = grid * (WARPS / group);
    return (size_t)((tiles + teams - 1) / teams) * WARPS * MT * 4 * 32;
}

struct StreamState {
    int group, member, tiles, kblocks, first, stride, my_tiles, units;
    int slots;              // boxes of this warp's ring
    int arm_slot;           // the slot the next box asked for goes to
    int my_kblocks;         // k-blocks of a tile that this warp multiplies
    const CUtensorMap* xmap;  // x rides with the boxes and may be read (the kernel in front has ended): its map; else null
    int tl_sec[5];
    int tl_loop, tl_sync, tl_all;  // profiling builds: cycles from the start of stream_run to the end of the boxes, of the team's meeting, of all
    int a_ti, a_kb, armed;
    int mode, up_offset, D;  // what arm_next needs of the product: which rows a box takes
    unsigned base;  // boxes this warp's ring carried before this product
    // What the end of this warp's FIRST tile needs besides the product, fetched together with the first weights
    // (none of it depends on the product's input), so that the end is not a chain of trips to memory:
    bool early;                                  // the values below are there
    float e_cos[MT_MAX][2], e_sin[MT_MAX][2];    // MODE_QKV: the rotation of this thread's pair, per token
    int e_slot[MT_MAX][2];                       // MODE_QKV: the tokens' cache slots
    bool have_resid;                             // MODE_RESIDUAL: e_resid holds the stream's values of the first tile
    float e_resid[MT_MAX][4];                    // MODE_RESIDUAL: fetched by stream_fetch_resid once the kernel in front has ended
    float e_norm[2];                             // MODE_RESIDUAL: the next norm's weights of this thread's features
};

// Asks for the next box of the product whose state is `st` (lane 0 only).  The slot and its mbarrier phase follow
// from the number of boxes the ring has carried, so a product's boxes may be asked for while the product before
// it is still being computed.
template <int MT = 1, bool RIDE = false>
__device__ __forceinline__ void arm_next(StreamState& st, const CUtensorMap* wmap, __nv_bfloat16* my_ring, unsigned long long* my_full) {
    constexpr int SLOT = slot_elems(MT, RIDE);
    const int tile = st.first + st.a_ti * st.stride, sl = st.arm_slot;
    __nv_bfloat16* dst = my_ring + (size_t)sl * SLOT;
    tma::mbar_expect_tx(&my_full[sl], (unsigned)(SLOT * 2));  // the weights, and x where it rides
    const int piece = st.a_kb * (BOXK / 64);  // the box's two 64-k pieces of its rows (see tma::make_map_row_pieces_bf16)
    if (st.mode == MODE_SWIGLU) {  // the map's box is 8 rows: gate rows, then up rows
        tma::load_3d(dst, wmap, 0, tile * 8, piece, &my_full[sl]);
        tma::load_3d(dst + 8 * BOXK, wmap, 0, st.up_offset + tile * 8, piece, &my_full[sl]);
    } else if (st.mode == MODE_QKV) {  // 8 lanes of a head's first half, then their partners in the second half
        const int per_head = st.D >> 4, head = tile / per_head, y = head * st.D + (tile - head * per_head) * 8;
        tma::load_3d(dst, wmap, 0, y, piece, &my_full[sl]);
        tma::load_3d(dst + 8 * BOXK, wmap, 0, y + (st.D >> 1), piece, &my_full[sl]);
    } else {
        tma::load_3d(dst, wmap, 0, tile * 16, piece, &my_full[sl]);
    }
    // the same k of every row of x behind the weights (before x may be read, stream_ride_x sends it after the box)
    if constexpr (RIDE)
        if (st.xmap) tma::load_3d(dst + SLOT_ELEMS, st.xmap, 0, 0, piece, &my_full[sl]);
    if (++st.arm_slot == st.slots) st.arm_slot = 0;
    ++st.armed;
    st.a_kb += st.group;
    if (st.a_kb >= st.kblocks) {
        st.a_kb = st.member;
        ++st.a_ti;
    }
}

// Splits the work and fetches what the end of the first tile needs.  Touches nothing that depends on the product's
// input: it may run before that is ready.  Asks for no box yet (stream_arm does).
template <int MODE, int MT = 1>
__device__ __forceinline__ void stream_plan(StreamState& st, const LinearParams& p, unsigned base) {
    static_assert(MT <= MT_MAX, "too many token tiles");
    constexpr int FEATURES = MODE == MODE_SWIGLU ? 8 : 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    st.group = p.group;
    st.slots = p.slots;
    st.arm_slot = (int)(base % (unsigned)p.slots);
    st.xmap = nullptr;
    st.member = warp % st.group;
    st.tiles = (p.N + FEATURES - 1) / FEATURES;
    st.kblocks = (p.K + BOXK - 1) / BOXK;
    st.first = blockIdx.x + (warp / st.group) * gridDim.x;
    st.stride = gridDim.x * (WARPS / st.group);
    st.my_tiles = st.tiles > st.first ? (st.tiles - 1 - st.first) / st.stride + 1 : 0;
    st.my_kblocks = st.kblocks > st.member ? (st.kblocks - 1 - st.member) / st.group + 1 : 0;
    st.units = st.my_tiles * st.my_kblocks;
    st.a_ti = 0;
    st.a_kb = st.member;
    st.armed = 0;
    st.base = base;
    st.mode = MODE;
    st.up_offset = p.up_offset;
    st.D = p.D;
    st.early = false;
    st.have_resid = false;
    if (st.member == 0 && st.my_tiles > 0) {
        const int qr = feature_row(lane >> 2), qc = lane & 3, tile = st.first;
        if constexpr (MODE == MODE_QKV) {
            const int D = p.D, half = D >> 1, per_head = D >> 4;
            const int head = tile / per_head, j = (tile - head * per_head) * 8 + qr;
            const bool rotate = head < p.H + p.KV && p.rotary;
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int m = 8 * t + 2 * qc + i;
                    st.e_cos[t][i] = 1.f;
                    st.e_sin[t][i] = 0.f;
                    st.e_slot[t][i] = 0;
                    if (m >= p.M) continue;
                    if (rotate) {
                        const int pos = min(max(p.positions[m], 0), p.rotary_rows - 1);
                        st.e_cos[t][i] = p.rotary[(size_t)pos * D + j];
                        st.e_sin[t][i] = p.rotary[(size_t)pos * D + half + j];
                    }
                    if (head >= p.H) st.e_slot[t][i] = p.slot_map[m];
                }
            st.early = true;
        } else if constexpr (MODE == MODE_RESIDUAL) {
            const int n0 = tile * 16;
#pragma unroll
            for (int h = 0; h < 2; ++h) st.e_norm[h] = n0 + qr + 8 * h < p.N ? p.norm_w[n0 + qr + 8 * h] : 0.f;
            st.early = true;
        }
    }
}

// MODE_RESIDUAL: the residual stream's values that the end of this warp's first tile adds to, asked for as soon as
// the kernel in front has ended (its writes, and those of every kernel before it, are visible then) instead of at the
// end of the tile, where the trip to memory would stand between the last product and the kernel's end.
template <int MT>
__device__ __forceinline__ void stream_fetch_resid(StreamState& st, const LinearParams& p) {
    if (st.member != 0 || st.my_tiles <= 0) return;
    const int lane = threadIdx.x & 31, qr = feature_row(lane >> 2), qc = lane & 3, n0 = st.first * 16;
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int n = n0 + qr + 8 * (e >> 1), m = 8 * t + 2 * qc + (e & 1);
            st.e_resid[t][e] = m < p.M && n < p.N ? p.resid[(size_t)m * p.N + n] : 0.f;
        }
    st.have_resid = true;
}

// Fills the free slots of the ring with the product's next boxes; `consumed`: how many of its boxes have been used.
template <int MT = 1, bool RIDE = false>
__device__ __forceinline__ void stream_arm(StreamState& st, const CUtensorMap* wmap, __nv_bfloat16* my_ring, unsigned long long* my_full,
                                           int consumed) {
    if ((threadIdx.x & 31) == 0)
        while (st.armed < st.units && st.armed < consumed + st.slots) arm_next<MT, RIDE>(st, wmap, my_ring, my_full);
}

template <int MODE, int MT = 1, bool RIDE = false>
__device__ __forceinline__ void stream_begin(StreamState& st, const LinearParams& p, const CUtensorMap* wmap,
                                             __nv_bfloat16* my_ring, unsigned long long* my_full, unsigned base) {
    stream_plan<MODE, MT>(st, p, base);
    stream_arm<MT, RIDE>(st, wmap, my_ring, my_full, 0);
}

// Where x rides with the boxes: sends x after the boxes that were asked for before x could be read (none of them has been
// used yet), and lets every later box bring its x along.  Lane 0 of the warp asks, as for the boxes.
template <int MT>
__device__ __forceinline__ void stream_ride_x(StreamState& st, const CUtensorMap* xmap, __nv_bfloat16* my_ring,
                                              unsigned long long* my_full) {
    constexpr int SLOT = slot_elems(MT, true);
    st.xmap = xmap;
    if ((threadIdx.x & 31) != 0) return;
    int sl = (int)(st.base % (unsigned)st.slots), j = 0;
    for (int u = 0; u < st.armed; ++u) {
        const int kb = st.member + j * st.group;
        tma::load_3d(my_ring + (size_t)sl * SLOT + SLOT_ELEMS, xmap, 0, 0, kb * (BOXK / 64), &my_full[sl]);
        if (++sl == st.slots) sl = 0;
        if (++j == st.my_kblocks) j = 0;
    }
}

// A product whose k is short (at most XREG_KB boxes a warp when its eight warps share every tile) keeps x in REGISTERS:
// a warp multiplies the same k-blocks in every one of its tiles, so the B fragments of those blocks are loaded once,
// straight from L2 by the lanes that use them, and no shared memory, no copy into it and no meeting of the CTA stands
// between the wait for the kernel in front and the first product; the CTA is then small enough (its rings and the
// partial sums) to sit beside the kernel in front also with two token tiles.
constexpr int XREG_KB = 2;

template <int MT>
__device__ __forceinline__ void stream_fetch_x(const LinearParams& p, const StreamState& st, uint4 (&xb)[XREG_KB][PIECES][MT]) {
    const int lane = threadIdx.x & 31, qr = lane >> 2, qc = lane & 3;
#pragma unroll
    for (int j = 0; j < XREG_KB; ++j) {
        const int kb = st.member + j * st.group;
#pragma unroll
        for (int i = 0; i < PIECES; ++i)
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                const int m = 8 * t + qr, k = kb * BOXK + i * 32 + qc * 8;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (m < p.M && kb < st.kblocks && k < p.K) v = __ldcg(reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + k));
                xb[j][i][t] = v;
            }
    }
}

// The input rows' RMS scales into row_scale (visible to the CTA after its next barrier): row m = warp + 8 t by warp `warp`.
template <int MT>
__device__ __forceinline__ void stream_row_scales(const LinearParams& p, float* row_scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        const int m = warp + WARPS * t;
        float s = 1.f;
        if (p.in_ss && m < p.M) {
            float sum = 0.f;
            for (int i = lane; i < p.in_parts; i += 32) sum += __ldcg(p.in_ss + (size_t)i * p.M + m);  // a fixed order: parts lane, lane + 32, ...
            s = rsqrtf(warp_sum(sum) / (float)p.K + p.in_eps);
        }
        if (lane == 0) row_scale[m] = s;
    }
}

// x into shared memory (rows beyond M as zeros) and the input rows' RMS scales; the caller synchronises the CTA.
// Every load is asked for before the first is used: one trip to memory, not one per loop.
template <int MT>
__device__ __forceinline__ void stream_stage_x(const LinearParams& p, __nv_bfloat16* x_s, float* row_scale) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int M = p.M, K = p.K, x_pitch = K + X_PAD;
    // the partial sums of squares of this warp's rows (row m = warp + 8 t; lanes take the parts in strides of 32)
    constexpr int SS_AHEAD = 4;
    float ss[MT][SS_AHEAD];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int j = 0; j < SS_AHEAD; ++j) {
            const int m = warp + WARPS * t, i = lane + 32 * j;
            ss[t][j] = p.in_ss && m < M && i < p.in_parts ? p.in_ss[(size_t)i * M + m] : 0.f;
        }
    {
        // asynchronous 16-byte copies straight into shared memory: all of them in flight at once
        const int per_row = K >> 3, total = 8 * MT * per_row;
        for (int idx = tid; idx < total; idx += THREADS) {
            const int m = idx / per_row, c = idx - m * per_row;
            __nv_bfloat16* dst = x_s + (size_t)m * x_pitch + c * 8;
            if (m < M) {
                const unsigned d32 = (unsigned)__cvta_generic_to_shared(dst);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d32), "l"(p.x + (size_t)m * p.ldx + c * 8) : "memory");
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        const int m = warp + WARPS * t;
        float s = 1.f;
        if (p.in_ss && m < M) {
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < SS_AHEAD; ++j) sum += ss[t][j];  // a fixed order: parts lane, lane + 32, ...
            for (int i = lane + 32 * SS_AHEAD; i < p.in_parts; i += 32) sum += p.in_ss[(size_t)i * M + m];
            s = rsqrtf(warp_sum(sum) / (float)K + p.in_eps);
        }
        if (lane == 0) row_scale[m] = s;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");  // this thread's copies have landed; the caller's barrier shows them to all
}

// The products of every box of this warp's tiles and the tiles' epilogues.  Returns false if a wait gave up.
template <int MT, int MODE, typename TO, bool XREG = false, bool RIDE = false>
__device__ __forceinline__ bool stream_run(StreamState& st, const LinearParams& p, const CUtensorMap* wmap, __nv_bfloat16* my_ring,
                                           unsigned long long* my_full, float* red, const __nv_bfloat16* x_s,
                                           const float* row_scale, const uint4 (*xb)[PIECES][MT] = nullptr) {
    constexpr int FEATURES = MODE == MODE_SWIGLU ? 8 : 16;
    constexpr int CHAINS = MT == 1 ? 4 : 2;
    constexpr int SLOT = slot_elems(MT, RIDE);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qr = lane >> 2, qc = lane & 3;  // MMA row (a feature of the tile) and column pair (tokens) of this thread
    const int fr = feature_row(qr);           // the feature of the tile that MMA row qr stands for
    const int M = p.M, N = p.N, K = p.K, x_pitch = K + X_PAD;
    const int group = st.group, member = st.member, kblocks = st.kblocks, first = st.first, stride = st.stride;
    const int my_tiles = st.my_tiles, units = st.units;
    bool gave_up = false;
    (void)tid; (void)N;
    const __nv_bfloat16* xrow[MT];  // this thread's x rows: token 8 t + qr
#pragma unroll
    for (int t = 0; t < MT; ++t) xrow[t] = x_s + (size_t)(8 * t + qr) * x_pitch + qc * 8;

    // what happens to a complete tile
    auto finish = [&](int ti, float (&acc)[MT][4]) {
    const int tile = first + ti * stride, n0 = tile * FEATURES;
    if constexpr (MODE == MODE_QKV) {
        // this thread: lanes j (e = 0, 1) and j + D/2 (e = 2, 3) of one head for tokens 8 t + 2 qc and + 1:
        // a rotation pair.  Query heads go to `out` rotated, key heads rotated into their page, value heads as
        // they are into theirs.
        const int D = p.D, half = D >> 1, per_head = D >> 4;
        const int head = tile / per_head, j = (tile - head * per_head) * 8 + fr;
#pragma unroll
        for (int t = 0; t < MT; ++t)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int m = 8 * t + 2 * qc + i;
                if (m >= M) continue;
                float a = acc[t][i] * row_scale[m], b = acc[t][2 + i] * row_scale[m];
                if (head < p.H + p.KV && p.rotary) {
                    float c, sn;
                    if (ti == 0 && st.early) {
                        c = st.e_cos[t][i];
                        sn = st.e_sin[t][i];
                    } else {
                        const int pos = min(max(p.positions[m], 0), p.rotary_rows - 1);
                        c = p.rotary[(size_t)pos * D + j];
                        sn = p.rotary[(size_t)pos * D + half + j];
                    }
                    const float ra = a * c - b * sn, rb = b * c + a * sn;
                    a = ra;
                    b = rb;
                }
                __nv_bfloat16* dst;
                if (head < p.H) {
                    dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + head * D + j;
                } else {
                    const int slot = ti == 0 && st.early ? st.e_slot[t][i] : p.slot_map[m];
                    const int page = slot / p.page_size, off = slot - page * p.page_size;
                    const int is_v = head >= p.H + p.KV, kvh = head - p.H - (is_v ? p.KV : 0);
                    dst = p.pool + (((size_t)(page * 2 + is_v) * p.KV + kvh) * p.page_size + off) * D + j;
                }
                dst[0] = __float2bfloat16_rn(a);
                dst[half] = __float2bfloat16_rn(b);
            }
    } else if constexpr (MODE == MODE_SWIGLU) {
        // this thread: gate (e = 0, 1) and up (e = 2, 3) sums of feature fr for tokens 8 t + 2 qc and + 1
        const int n = n0 + fr;
#pragma unroll
        for (int t = 0; t < MT; ++t)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int m = 8 * t + 2 * qc + j;
                const float g = acc[t][j] * row_scale[m], u = acc[t][2 + j] * row_scale[m];
                if (m < M && n < N) reinterpret_cast<TO*>(p.out)[(size_t)m * p.ldo + n] = from_float<TO>(g / (1.f + expf(-g)) * u);
            }
    } else {
        // this thread: features fr (e = 0, 1) and fr + 8 (e = 2, 3) of tokens 8 t + 2 qc and + 1
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            float sq[2] = {0.f, 0.f};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int n = n0 + fr + 8 * (e >> 1), m = 8 * t + 2 * qc + (e & 1);
                const bool live = m < M && n < N;
                const float s = acc[t][e] * row_scale[m];
                if constexpr (MODE == MODE_RESIDUAL) {
                    if (live) {
                        const bool have = ti == 0 && st.early;
                        const float before = ti == 0 && st.have_resid ? st.e_resid[t][e] : p.resid[(size_t)m * N + n];
                        const float v = before + s;
                        p.resid[(size_t)m * N + n] = v;
                        p.xw_out[(size_t)m * N + n] = __float2bfloat16_rn(v * (have ? st.e_norm[e >> 1] : p.norm_w[n]));
                        sq[e & 1] += v * v;
                    }
                } else {
                    if (live) reinterpret_cast<TO*>(p.out)[(size_t)m * p.ldo + n] = from_float<TO>(s);
                }
            }
            if constexpr (MODE == MODE_RESIDUAL) {
                // sum of v^2 over the tile's 16 features of a token: over the 8 lanes that share qc
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float v = sq[j];
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 16);
                    const int m = 8 * t + 2 * qc + j;
                    if (qr == 0 && m < M) p.ss_out[(size_t)tile * M + m] = v;
                }
            }
        }
    }
    };

    int unit = 0;
    int sl = (int)(st.base % (unsigned)st.slots);            // the slot of the next box and the phase of its mbarrier
    unsigned phase = (st.base / (unsigned)st.slots) & 1u;
    TL(const long long tl0 = clock64(); long long tl_loop = 0, tl_sync = 0, tl_w = 0, tl_l = 0, tl_a = 0, tl_m = 0; int tl_n = 0, tl_dummy = 0;)
    for (int ti = 0; ti < my_tiles; ++ti) {
        // CHAINS independent sums per token tile, joined when the tile is complete: an MMA waits for the one before it
        // on the same accumulator, and one chain of eight per box would leave the tensor pipe idle most of the time
        float part[MT][CHAINS][4];
#pragma unroll
        for (int t = 0; t < MT; ++t)
#pragma unroll
            for (int c = 0; c < CHAINS; ++c)
#pragma unroll
                for (int e = 0; e < 4; ++e) part[t][c][e] = 0.f;
        auto box = [&](const int kb, auto jtag) {  // one box: k-block kb of this tile (jtag: which of the warp's k-blocks it is)
            constexpr int j = decltype(jtag)::value;
            (void)j;
            TL(const long long c0 = clock64();)
            if (!gave_up && !tma::mbar_wait(&my_full[sl], phase)) {
                gave_up = true;
                if (p.error_flag) atomicExch(p.error_flag, 1);
            }
            TL(const long long c1 = clock64(); tl_w += c1 - c0;)
            // the box lies as [2 pieces of 64 k][rows][64] with the 128-byte swizzle: chunk c of row r at chunk c ^ (r & 7)
            const __nv_bfloat16* slot = my_ring + (size_t)sl * SLOT + fr * 64;
            [[maybe_unused]] const __nv_bfloat16* xs = my_ring + (size_t)sl * SLOT + SLOT_ELEMS;  // RIDE: [2 pieces][8 MT rows][64]
            const int k0 = kb * BOXK;
            uint4 a[PIECES][2], b[PIECES][MT];
#pragma unroll
            for (int i = 0; i < PIECES; ++i) {
                constexpr bool SPLIT = MODE == MODE_SWIGLU || MODE == MODE_QKV;  // two loads of eight rows, else one of sixteen
                const int chunk = ((((i & 1) << 2) | qc) ^ fr) * 8, piece = (i >> 1) * (SPLIT ? 8 * 64 : 16 * 64);
                a[i][0] = *reinterpret_cast<const uint4*>(slot + piece + chunk);
                a[i][1] = *reinterpret_cast<const uint4*>(slot + piece + chunk + (SPLIT ? 8 * BOXK : 8 * 64));
                // beyond K the weights arrived as zeros and x is not read (its row ends there)
                [[maybe_unused]] const bool have = k0 + i * 32 + qc * 8 < K;
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    if constexpr (XREG) b[i][t] = xb[j][i][t];
                    else if constexpr (RIDE) {  // rows beyond M and k beyond K arrived as zeros
                        const int row = 8 * t + qr;
                        b[i][t] = *reinterpret_cast<const uint4*>(xs + (i >> 1) * (8 * MT * 64) + row * 64 + (((((i & 1) << 2) | qc) ^ (row & 7)) * 8));
                    } else b[i][t] = have ? *reinterpret_cast<const uint4*>(xrow[t] + k0 + i * 32) : make_uint4(0, 0, 0, 0);
                }
            }
            TL(if (a[PIECES - 1][1].w == 0x7fc12345u && b[PIECES - 1][0].w == 0x7fc12345u) ++tl_dummy; const long long c2 = clock64(); tl_l += c2 - c1;)
            TL(const long long c3 = c2;)
#pragma unroll
            for (int i = 0; i < PIECES; ++i)
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    mma_bf16(part[t][(2 * i) % CHAINS], a[i][0].x, a[i][1].x, a[i][0].y, a[i][1].y, b[i][t].x, b[i][t].y);
                    mma_bf16(part[t][(2 * i + 1) % CHAINS], a[i][0].z, a[i][1].z, a[i][0].w, a[i][1].w, b[i][t].z, b[i][t].w);
                }
            TL(if (part[0][0][0] + part[0][1][0] + part[0][CHAINS - 1][0] == -1.2345e30f) ++tl_dummy; const long long c4 = clock64(); tl_m += c4 - c3; ++tl_n;)
            // The slot takes the next box only now, when the products above have been issued and so have read every
            // lane's pieces of it out of the registers: a load from shared memory is complete when its first user is
            // issued, not when the lanes meet.  (Asked for between the loads and the products, the next box was seen
            // to land in the slot before the loads had read it, when loads from global memory stood in the way.)
            __syncwarp();
            if (lane == 0 && st.armed < units) arm_next<MT, RIDE>(st, wmap, my_ring, my_full);
            TL(__syncwarp(); tl_a += clock64() - c4;)
            ++unit;
            if (++sl == st.slots) {
                sl = 0;
                phase ^= 1u;
            }
        };
        if constexpr (XREG) {  // unrolled, so that xb[j] is a register
            if (member < kblocks) box(member, std::integral_constant<int, 0>{});
            if (member + group < kblocks) box(member + group, std::integral_constant<int, 1>{});
            static_assert(XREG_KB == 2, "one call per k-block of a warp");
        } else {
            for (int kb = member; kb < kblocks; kb += group) box(kb, std::integral_constant<int, 0>{});
        }
        float acc[MT][4];
#pragma unroll
        for (int t = 0; t < MT; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sum = part[t][0][e];
#pragma unroll
                for (int c = 1; c < CHAINS; ++c) sum += part[t][c][e];  // a fixed order
                acc[t][e] = sum;
            }
        if (group == 1) {
            finish(ti, acc);
        } else {
            // the members' partial sums wait in shared memory, a place per (tile of the team, warp), until all of the
            // team's tiles are done: the warps of a team meet once, not once per tile
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[(((size_t)ti * WARPS + warp) * (MT * 4) + t * 4 + e) * 32 + lane] = acc[t][e];
        }
    }
    TL(tl_loop = clock64() - tl0;)
    if (group > 1) {
        asm volatile("bar.sync %0, %1;\n" ::"r"(1 + warp / group), "r"(group * 32) : "memory");
        TL(tl_sync = clock64() - tl0;)
        // the team's tiles are ended by its members in turn (tile ti by member ti mod group), not all by one warp while
        // the others have nothing left to do; the first tile, whose end has values fetched early, is member 0's
        for (int ti = member; ti < my_tiles; ti += group) {
            float acc[MT][4];
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
            for (int w2 = warp - member; w2 < warp - member + group; ++w2)  // a fixed order
#pragma unroll
                for (int t = 0; t < MT; ++t)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[t][e] += red[(((size_t)ti * WARPS + w2) * (MT * 4) + t * 4 + e) * 32 + lane];
            finish(ti, acc);
        }
    }
    // nothing of this warp's is in flight: every armed unit was waited for above (after a failed wait, once
    // more here, bounded, so that no copy lands in shared memory after the CTA has left)
    if (gave_up && lane == 0)
        for (unit = max(0, units - st.slots); unit < units; ++unit)
            tma::mbar_wait(&my_full[(st.base + unit) % (unsigned)st.slots], ((st.base + unit) / (unsigned)st.slots) & 1u);
    TL(if (threadIdx.x == 0) { st.tl_loop = (int)tl_loop; st.tl_sync = (int)tl_sync; st.tl_all = (int)(clock64() - tl0) + (tl_dummy & 1);
       st.tl_sec[0] = (int)tl_w; st.tl_sec[1] = (int)tl_l; st.tl_sec[2] = (int)tl_a; st.tl_sec[3] = (int)tl_m; st.tl_sec[4] = tl_n; })
    return !gave_up;
}

}  // namespace lin
