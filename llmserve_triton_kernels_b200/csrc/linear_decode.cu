// y[M, N] = x[M, K] * w[N, K]^T for few rows (M <= 16, a decode batch): a weight-streaming kernel
// with the neighbouring row-wise work fused into its ends.
//
// Every weight is read from HBM exactly once, with 16-byte loads that go straight into tensor-core
// fragments; the batch rides along as the narrow side of the product ("swap A and B": the 16 rows of
// an mma.sync m16n8k16 tile are 16 output features, its 8 columns are 8 tokens).  One CTA per SM
// stays resident; each of its 8 warps streams tiles of 16 output features of its own through a
// private ring of TMA boxes (16 rows x 128 k through a tensor map, completion counted by the
// warp's own mbarriers), so about 100 KB per SM are in flight and no warp waits for another.
//
// Fragment trick: a thread's 16-byte read of weight row r at k = 8 q .. 8 q + 7 (q = lane % 4) holds
// the A elements of TWO k16 steps if the product's k-order is permuted the same way on the x
// side — a sum over k does not care about the order — so the fragments need no shuffles and no
// ldmatrix.
//
// Where x lives is chosen per launch (see launch()): in the registers of the lanes that multiply with it
// (k <= 2048, few tiles a CTA), riding with the weight boxes (one tile a CTA, or x too long for shared
// memory), or copied into shared memory once (x reused over many tiles).  The first two have no barrier of
// the CTA before the first product.
//
// Fused ends (decode steps are bound by launches as much as by bytes):
//   * input in factored normalised form: x holds v * norm_weight (v the residual stream) and
//     in_ss holds partial sums of v^2 per row; the product is scaled by rsqrt(sum / K + eps) at the
//     end, which is the RMS norm of the input without a pass of its own.
//   * MODE_SWIGLU: w is [gate rows | up rows]; the CTA computes both for its features and writes
//     silu(gate) * up.
//   * MODE_RESIDUAL: the result is added to the 32-bit residual stream in place, and the stream's
//     next factored normalised form (v * next_norm_weight in bfloat16, partial sums of v^2 per CTA)
//     is written for the next product.
#include "linear_stream.cuh"
#include "timeline.cuh"

#include <mutex>
#include <unordered_map>

namespace {

using namespace lin;

enum { X_STAGED = 0, X_REGISTERS = 1, X_RIDES = 2 };  // where a kernel keeps x

// One product: MT 8-token tiles (M <= 8 MT); see linear_stream.cuh for how a CTA streams.

template <int MT, int MODE, typename TO, int XWHERE>
__device__ __forceinline__ void linear_decode_body(const LinearParams& p, const CUtensorMap& wmap, const CUtensorMap* xmap = nullptr) {
    constexpr bool XREG = XWHERE == X_REGISTERS, RIDE = XWHERE == X_RIDES;
    constexpr int SLOT = slot_elems(MT, RIDE);
    TL(tl::Marks marks;)
    extern __shared__ __align__(1024) unsigned char smem_all[];
    unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_all + 1023) & ~(uintptr_t)1023);  // the swizzle's period
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);                    // [warps that have tiles][slots][SLOT]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)p.ring_warps * p.slots * SLOT * 2);  // [tiles of a team][WARPS][MT * 4][32]
    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(red + p.red_floats);  // [8 MT][K + X_PAD]
    __shared__ float row_scale[8 * MT];
    __shared__ __align__(8) unsigned long long full[WARPS][SLOTS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl) tma::mbar_init(&full[warp][sl], 1);
        tma::mbar_fence_init();
        if (warp == 0) tma::prefetch_map(&wmap);
    }
    __syncwarp();
    __nv_bfloat16* my_ring = ring + (size_t)warp * p.slots * SLOT;
    StreamState st;
    // the weights do not depend on what ran before: their first boxes are asked for at once, while the
    // kernel before this one may still be running; everything else waits for it
    stream_begin<MODE, MT, RIDE>(st, p, &wmap, my_ring, full[warp], 0u);
    pdl_trigger();
    TL(marks.mark(1);)
    pdl_wait();
    TL(marks.mark(2);)
    if constexpr (MODE == MODE_RESIDUAL) stream_fetch_resid<MT>(st, p);
    bool ok;
    if constexpr (XREG) {
        // x straight into the registers of the lanes that multiply with it; the rows' scales are shown to the warps that
        // end the tiles by the meeting of the team (all eight warps) that comes before any tile's end
        uint4 xb[XREG_KB][PIECES][MT];
        stream_fetch_x<MT>(p, st, xb);
        stream_row_scales<MT>(p, row_scale);
        TL(marks.mark(3);)
        ok = stream_run<MT, MODE, TO, true>(st, p, &wmap, my_ring, full[warp], red, nullptr, row_scale, xb);
    } else if constexpr (RIDE) {
        // every box brings its 128 k of x along: no copy of x as a whole and, when the CTA's warps are one team (whose
        // meeting also shows the rows' scales), no barrier of the CTA
        stream_ride_x<MT>(st, xmap, my_ring, full[warp]);
        stream_row_scales<MT>(p, row_scale);
        if (p.group < WARPS) __syncthreads();
        TL(marks.mark(3);)
        ok = stream_run<MT, MODE, TO, false, true>(st, p, &wmap, my_ring, full[warp], red, nullptr, row_scale);
    } else {
        stream_stage_x<MT>(p, x_s, row_scale);
        __syncthreads();  // the only CTA-wide barrier
        TL(marks.mark(3);)
        ok = stream_run<MT, MODE, TO, false>(st, p, &wmap, my_ring, full[warp], red, x_s, row_scale);
    }
    if (!ok && lane == 0 && p.error_flag) atomicExch(p.error_flag, 1);
    TL(__syncthreads(); if (threadIdx.x == 0) { marks.mark(4); marks.t[1] = ((unsigned long long)(unsigned)st.tl_sec[0] << 48) | ((unsigned long long)(unsigned)(st.tl_sec[1] & 0xffff) << 32) | ((unsigned long long)(unsigned)(st.tl_sec[2] & 0xffff) << 16) | (unsigned)(st.tl_sec[3] & 0xffff); marks.t[3] = (marks.t[3] & ~0xffull) | (unsigned)st.tl_sec[4]; marks.t[5] = ((unsigned long long)(unsigned)st.tl_loop << 40) | ((unsigned long long)(unsigned)st.tl_sync << 20) | (unsigned)st.tl_all; marks.write(MODE, p.tl_launch, blockIdx.x, p.N, p.K); })
}

// Up to 8 tokens: at most 120 registers a thread, so that two CTAs of 256 threads share an SM's registers with room to
// spare (two CTAs of 128 registers a thread fill the file to the last register, and were then seen to run one after
// the other); 9 to 16 tokens carry twice the accumulators and fragments and take what they need.
template <int MODE, typename TO>
__global__ void __maxnreg__(120) linear_decode_kernel_8(const LinearParams p, const __grid_constant__ CUtensorMap wmap) {
    linear_decode_body<1, MODE, TO, X_STAGED>(p, wmap);
}
template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1) linear_decode_kernel_16(const LinearParams p, const __grid_constant__ CUtensorMap wmap) {
    linear_decode_body<2, MODE, TO, X_STAGED>(p, wmap);
}
// The same with x in registers (short k, every tile shared by the CTA's eight warps): see stream_fetch_x.
template <int MODE, typename TO>
__global__ void __maxnreg__(120) linear_decode_xreg_kernel_8(const LinearParams p, const __grid_constant__ CUtensorMap wmap) {
    linear_decode_body<1, MODE, TO, X_REGISTERS>(p, wmap);
}
template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1) linear_decode_xreg_kernel_16(const LinearParams p, const __grid_constant__ CUtensorMap wmap) {
    linear_decode_body<2, MODE, TO, X_REGISTERS>(p, wmap);
}
// The same with x riding with the boxes (any k: x takes no shared memory of its own): see stream_ride_x.
template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1) linear_decode_ride_kernel_8(const LinearParams p, const __grid_constant__ CUtensorMap wmap,
                                                                          const __grid_constant__ CUtensorMap xmap) {
    linear_decode_body<1, MODE, TO, X_RIDES>(p, wmap, &xmap);
}
template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1) linear_decode_ride_kernel_16(const LinearParams p, const __grid_constant__ CUtensorMap wmap,
                                                                           const __grid_constant__ CUtensorMap xmap) {
    linear_decode_body<2, MODE, TO, X_RIDES>(p, wmap, &xmap);
}

int sm_count() {
    static int count = 0;
    if (count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0) count = 148;
    }
    return count;
}

// Tensor maps of row-major matrices [rows, K] (ld elements from row to row), made once per (address, shape, box): of
// weight matrices, which live as long as the model, and of x where it rides with the boxes (activations of a shape come
// back to the same addresses from a caching allocator, and a captured step keeps its buffers).
// The map is handed out by value: an entry may be dropped by the next call.
bool weight_map(CUtensorMap* out, const void* w, int rows, int K, int box_rows, int ld = 0) {
    struct Key {
        const void* w;
        int rows, K, box, ld;
        bool operator==(const Key& o) const { return w == o.w && rows == o.rows && K == o.K && box == o.box && ld == o.ld; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return std::hash<const void*>()(k.w) ^ ((size_t)k.rows << 20) ^ ((size_t)k.K << 4) ^ (size_t)k.box ^ ((size_t)k.ld << 36);
        }
    };
    static std::unordered_map<Key, CUtensorMap, Hash> maps;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    const Key key{w, rows, K, box_rows, ld};
    auto it = maps.find(key);
    if (it != maps.end()) {
        *out = it->second;
        return true;
    }
    if (maps.size() > 8192) maps.clear();  // (activations that never came back to the same address)
    if (!tma::make_map_row_pieces_bf16(out, w, rows, K, box_rows, ld)) return false;
    maps.emplace(key, *out);
    return true;
}

constexpr size_t SMEM_LIMIT = 227 * 1024;

// x rides with the boxes (stream_ride_x): a slot holds the box of weights and the same 128 k of x, and x as a whole takes no
// shared memory, so any k is taken.  Chosen where x does not fit beside the rings, and where no CTA has more than one tile
// (x would be read from its copy once: the copy and the barrier behind it are saved).
template <int MT, int MODE, typename TO>
int launch_ride(const LinearParams& p, cudaStream_t stream) {
    constexpr int FEATURES = MODE == MODE_SWIGLU ? 8 : 16;
    constexpr size_t SLOT_BYTES = (size_t)slot_elems(MT, true) * 2, RED_BYTES = (size_t)WARPS * MT * 4 * 32 * sizeof(float);
    constexpr int RIDE_SLOTS = MT == 1 ? SLOTS : 3;  // 192 KB of rings either way
    const int tiles = (p.N + FEATURES - 1) / FEATURES, kblocks = (p.K + BOXK - 1) / BOXK, sms = sm_count();
    const int grid = tiles < sms ? tiles : sms;
    LinearParams q = p;
    TL(static int tl_launches = 1000; q.tl_launch = tl_launches++;)
    const int room = (int)((SMEM_LIMIT - 1024 - (size_t)WARPS * RIDE_SLOTS * SLOT_BYTES) / RED_BYTES);
    q.group = choose_group(tiles, kblocks, grid, room);
    const int teams = grid * (WARPS / q.group);
    const int boxes_each = ((tiles + teams - 1) / teams) * ((kblocks + q.group - 1) / q.group);
    q.slots = boxes_each <= 2 ? 2 : RIDE_SLOTS;
    q.red_floats = (int)red_floats(tiles, grid, q.group, MT);
    const int busy_teams = (tiles + grid - 1) / grid < WARPS / q.group ? (tiles + grid - 1) / grid : WARPS / q.group;
    q.ring_warps = busy_teams * q.group;
    const size_t smem = (size_t)q.ring_warps * q.slots * SLOT_BYTES + (size_t)q.red_floats * sizeof(float) + 1024;
    if (smem > SMEM_LIMIT) return LLM_ERR_UNSUPPORTED;
    void (*kernel)(const LinearParams, const CUtensorMap, const CUtensorMap);
    if constexpr (MT == 1) kernel = linear_decode_ride_kernel_8<MODE, TO>;
    else kernel = linear_decode_ride_kernel_16<MODE, TO>;
    static size_t configured = 0;  // per instantiation: the most dynamic shared memory asked for so far
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = smem;
    }
    CUtensorMap wmap, xmap;
    if (!weight_map(&wmap, p.w, MODE == MODE_SWIGLU ? p.up_offset + p.N : p.N, p.K, MODE == MODE_QKV ? 8 : FEATURES) ||
        !weight_map(&xmap, p.x, p.M, p.K, 8 * MT, p.ldx))
        return LLM_ERR_UNSUPPORTED;
    return launch_pdl(kernel, dim3(grid), dim3(THREADS), smem, stream, q, wmap, xmap);
}

template <int MT, int MODE, typename TO>
int launch(const LinearParams& p, cudaStream_t stream) {
    constexpr int FEATURES = MODE == MODE_SWIGLU ? 8 : 16;
    const int tiles = (p.N + FEATURES - 1) / FEATURES, kblocks = (p.K + BOXK - 1) / BOXK, sms = sm_count();
    int grid = tiles < sms ? tiles : sms;
    LinearParams q = p;
    TL(static int tl_launches = 0; q.tl_launch = tl_launches++;)
    // x in registers: k short enough for XREG_KB boxes a warp when eight warps share a tile, few enough tiles a CTA for
    // their partial sums, and not the output matrix's many tiles (their ends would all wait for one meeting)
    static const bool xreg_on = [] { const char* e = getenv("LLMSERVE_B200_XREG"); return !e || atoi(e) != 0; }();
    const bool xreg = xreg_on && kblocks <= XREG_KB * WARPS && (tiles + sms - 1) / sms <= 6;
    const size_t x_bytes = xreg ? 0 : (size_t)8 * MT * (p.K + X_PAD) * 2;
    auto ring_bytes = [](int slots, int warps = WARPS) { return (size_t)warps * slots * SLOT_ELEMS * 2; };
    // A product of a few more tiles than SMs whose k is short (the stacked projection of a small model): one tile per
    // CTA, shared by its eight warps, on as many CTAs as tiles.  Each CTA then needs two boxes per warp, two such
    // CTAs fit an SM, and none has twice the work of the others.
    const size_t pair_limit = (SMEM_LIMIT + 1024) / 2 - 1024;
    const bool one_each = (MT == 1 || xreg) && tiles > sms && tiles <= 2 * sms && (kblocks + WARPS - 1) / WARPS <= 2 &&
                          ring_bytes(2) + x_bytes + (size_t)WARPS * MT * 4 * 32 * sizeof(float) <= pair_limit;
    static const bool ride_on = [] { const char* e = getenv("LLMSERVE_B200_RIDE"); return !e || atoi(e) != 0; }();
    if (one_each) {
        grid = tiles;
        q.group = WARPS;
    } else if (xreg) {
        q.group = WARPS;
    } else {
        const bool fits = ring_bytes(SLOTS) + x_bytes <= SMEM_LIMIT;  // x beside the rings
        if (ride_on && (!fits || tiles <= sms)) return launch_ride<MT, MODE, TO>(p, stream);
        if (!fits) return LLM_ERR_UNSUPPORTED;
        // as many tiles of a team may be shared as their partial sums find room for
        const int room = (int)((SMEM_LIMIT - ring_bytes(SLOTS) - x_bytes) / ((size_t)WARPS * MT * 4 * 32 * sizeof(float)));
        q.group = choose_group(tiles, kblocks, grid, room);
    }
    // a warp that never has more than two boxes needs no more than two slots: the CTA is then small enough for the
    // CTA of the kernel behind it (launched early) to sit beside it and do what it can before its turn
    const int teams = grid * (WARPS / q.group);
    const int boxes_each = ((tiles + teams - 1) / teams) * ((kblocks + q.group - 1) / q.group);
    q.slots = boxes_each <= 2 ? 2 : SLOTS;
    q.red_floats = (int)red_floats(tiles, grid, q.group, MT);
    // rings only for the warps that have tiles (those of the teams j with j grid < tiles: the first warps of a CTA)
    const int busy_teams = (tiles + grid - 1) / grid < WARPS / q.group ? (tiles + grid - 1) / grid : WARPS / q.group;
    q.ring_warps = busy_teams * q.group;
    const size_t smem = ring_bytes(q.slots, q.ring_warps) + x_bytes + (size_t)q.red_floats * sizeof(float) + 1024;  // and room to align
    if (smem > SMEM_LIMIT) return LLM_ERR_UNSUPPORTED;
    void (*kernel)(const LinearParams, const CUtensorMap);
    if constexpr (MT == 1) kernel = xreg ? linear_decode_xreg_kernel_8<MODE, TO> : linear_decode_kernel_8<MODE, TO>;
    else kernel = xreg ? linear_decode_xreg_kernel_16<MODE, TO> : linear_decode_kernel_16<MODE, TO>;
    static size_t configured_of[2] = {0, 0};  // per instantiation and kernel: the most dynamic shared memory asked for so far
    size_t& configured = configured_of[xreg ? 1 : 0];
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // all of the SM's memory as shared memory whatever this launch needs, so that a CTA of the next kernel can join
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = smem;
    }
    CUtensorMap map;
    if (!weight_map(&map, p.w, MODE == MODE_SWIGLU ? p.up_offset + p.N : p.N, p.K, MODE == MODE_QKV ? 8 : FEATURES)) return LLM_ERR_UNSUPPORTED;
    return launch_pdl(kernel, dim3(grid), dim3(THREADS), smem, stream, q, map);
}

// MODE_QKV: the product for all heads, rotary encoding of query and key heads, and the write of keys and
// values into their pages, in one launch (see llm_linear_decode for the other arguments).
template <int MODE, typename TO>
int dispatch(const LinearParams& p, cudaStream_t stream) {
    return p.M <= 8 ? launch<1, MODE, TO>(p, stream) : launch<2, MODE, TO>(p, stream);
}

}  // namespace

LLM_EXPORT int llm_linear_decode_qkv(const void* x, const void* w, void* q_out, int M, int K, int ldx, const float* in_ss,
                                     int in_parts, float in_eps, const int* positions, const float* rotary, int rotary_rows,
                                     const int* slot_map, void* pool, int H, int KV, int D, int page_size, int* error_flag,
                                     cudaStream_t stream);

TL_DEFINE_READER(llm_timeline_read_linear)

// The most rows this kernel takes; more go to another matrix product.
LLM_EXPORT int llm_linear_decode_max_rows() { return 16; }

// How many partial sums of squares per row MODE_RESIDUAL writes for N features.
LLM_EXPORT int llm_linear_decode_parts(int N) { return (N + 15) / 16; }

// bfloat16 x [M, K] (row stride ldx) times w^T (w contiguous [N or 2 N, K]).
//   mode 0: out [M, N] (row stride ldo), bfloat16 or float32.
//   mode 1: w = [gate | up] with the up rows starting at row up_offset; out [M, N] = silu(gate) * up.
//   mode 2: resid [M, N] += product; xw_out [M, N] = resid * norm_w; ss_out [parts(N), M] = partial sums
//           of resid^2.  out is not used.
// in_ss (or null): [in_parts, M] partial sums of squares; the product is scaled by
// rsqrt(sum / K + in_eps) per row.  Needs M <= 16, K a multiple of 64 (the weights travel in pieces of 64 k), 16-byte aligned rows;
// otherwise it returns LLM_ERR_UNSUPPORTED and the caller takes another route.  error_flag (host-visible
// int, or null) is set to 1 if a bounded wait inside the kernel ever gives up.
LLM_EXPORT int llm_linear_decode(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int ldx,
                                 int ldo, const float* in_ss, int in_parts, float in_eps, int mode, int up_offset,
                                 float* resid, const float* norm_w, void* xw_out, float* ss_out, int* error_flag,
                                 cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K < 64 || (K & 63) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return LLM_ERR_UNSUPPORTED;
    LinearParams p = {};
    p.x = (const __nv_bfloat16*)x;
    p.w = (const __nv_bfloat16*)w;
    p.out = out;
    p.M = M;
    p.N = N;
    p.K = K;
    p.ldx = ldx;
    p.ldo = ldo;
    p.in_ss = in_ss;
    p.in_parts = in_parts;
    p.in_eps = in_eps;
    p.up_offset = up_offset;
    p.resid = resid;
    p.norm_w = norm_w;
    p.xw_out = (__nv_bfloat16*)xw_out;
    p.ss_out = ss_out;
    p.error_flag = error_flag;
    if (mode == MODE_RESIDUAL) {
        if (!resid || !norm_w || !xw_out || !ss_out) return LLM_ERR_BAD_ARGUMENT;
        return dispatch<MODE_RESIDUAL, __nv_bfloat16>(p, stream);
    }
    if (mode == MODE_SWIGLU) {
        if (out_dtype != LLM_BF16) return LLM_ERR_BAD_ARGUMENT;
        return dispatch<MODE_SWIGLU, __nv_bfloat16>(p, stream);
    }
    if (mode != MODE_PLAIN) return LLM_ERR_BAD_ARGUMENT;
    if (out_dtype == LLM_BF16) return dispatch<MODE_PLAIN, __nv_bfloat16>(p, stream);
    if (out_dtype == LLM_F32) return dispatch<MODE_PLAIN, float>(p, stream);
    return LLM_ERR_BAD_ARGUMENT;
}

// bfloat16 x [M, K] times the stacked projection w [(H + 2 KV) D, K]: query heads, rotated by each token's
// row of `rotary` ([positions, D] = cos | sin halves; null: no rotation), go to q_out [M, H D]; key heads,
// rotated, and value heads go into `pool` [pages, 2, KV, page_size, D] at slot_map[m].  KV = 0: w holds
// query heads only and nothing is written to the pool.  Needs M <= 16, K and D multiples of 64 and 16.
LLM_EXPORT int llm_linear_decode_qkv(const void* x, const void* w, void* q_out, int M, int K, int ldx, const float* in_ss,
                                     int in_parts, float in_eps, const int* positions, const float* rotary, int rotary_rows,
                                     const int* slot_map, void* pool, int H, int KV, int D, int page_size, int* error_flag,
                                     cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 16 || K < 64 || (K & 63) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || D < 16 || (D & 15) || H < 1 || KV < 0)
        return LLM_ERR_UNSUPPORTED;
    if (KV > 0 && (!slot_map || !pool || page_size < 1)) return LLM_ERR_BAD_ARGUMENT;
    if (rotary && (!positions || rotary_rows < 1)) return LLM_ERR_BAD_ARGUMENT;
    LinearParams p = {};
    p.x = (const __nv_bfloat16*)x;
    p.w = (const __nv_bfloat16*)w;
    p.out = q_out;
    p.M = M;
    p.N = (H + 2 * KV) * D;
    p.K = K;
    p.ldx = ldx;
    p.ldo = H * D;
    p.in_ss = in_ss;
    p.in_parts = in_parts;
    p.in_eps = in_eps;
    p.error_flag = error_flag;
    p.positions = positions;
    p.rotary = rotary;
    p.rotary_rows = rotary_rows;
    p.slot_map = slot_map;
    p.pool = (__nv_bfloat16*)pool;
    p.H = H;
    p.KV = KV;
    p.D = D;
    p.page_size = page_size;
    return dispatch<MODE_QKV, __nv_bfloat16>(p, stream);
}
