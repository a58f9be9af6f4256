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
// Fused ends (decode steps are bound by launches as much as by bytes):
//   * input in factored normalised form: x holds v * norm_weight (v the residual stream) and
//     in_ss holds partial sums of v^2 per row; the product is scaled by rsqrt(sum / K + eps) at the
//     end, which is the RMS norm of the input without a pass of its own.
//   * MODE_SWIGLU: w is [gate rows | up rows]; the CTA computes both for its features and writes
//     silu(gate) * up.
//   * MODE_RESIDUAL: the result is added to the 32-bit residual stream in place, and the stream's
//     next factored normalised form (v * next_norm_weight in bfloat16, partial sums of v^2 per CTA)
//     is written for the next product.
#include "common.cuh"
#include "tma.cuh"

#include <mutex>
#include <unordered_map>

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_RESIDUAL = 2, MODE_QKV = 3;

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

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
    // MODE_QKV: w rows are [H query heads | KV key heads | KV value heads] x D; out is [M, H * D]
    const int* positions;   // [M]
    const float* rotary;    // [positions, D] = cos | sin halves, or null (no rotation)
    int rotary_rows;
    const int* slot_map;    // [M] page * page_size + offset of each token
    __nv_bfloat16* pool;    // [pages, 2, KV, page_size, D]
    int H, KV, D, page_size;
    const void* prefetch;   // weights that a later product will stream: pulled into L2 meanwhile (or null)
    unsigned long long prefetch_bytes;
};

constexpr int SLOTS = 4;   // boxes per warp: three in flight while one is being used
constexpr int BOXK = 128;  // k per box: a slot is 16 rows x 128 k = 4 KB
constexpr int SLOT_ELEMS = 16 * BOXK;
constexpr int PIECES = BOXK / 32;
constexpr int X_PAD = 32;  // elements between the rows of x in shared memory: 8 tokens x 64 bytes hit 8 bank groups

// MT: 8-token tiles (M <= 8 MT).  A tile of work is 16 output features over the whole of K — in
// MODE_SWIGLU 8 features, whose gate rows fill rows 0-7 of the mma tile and whose up rows fill rows
// 8-15, so that one thread holds a feature's gate and up sums.  Every WARP streams tiles of its own:
// its first lane asks the TMA unit for the box (16 rows x 128 k) three boxes ahead while the warp
// multiplies the current one; nothing but the warp's own mbarriers orders the two, so no warp waits
// for another, and 8 warps x 3 boxes are in flight per SM.  With few tiles, 2, 4 or 8 warps of a CTA
// share a tile by k-blocks and add up through shared memory.  x lies in shared memory, copied once.
// Every wait on a copy is bounded: if it gives up, the kernel sets *error_flag and runs to its end.
template <int MT, int MODE, typename TO>
__global__ void __launch_bounds__(THREADS)
linear_decode_kernel(const LinearParams p, const __grid_constant__ CUtensorMap wmap) {
    constexpr int FEATURES = MODE == MODE_SWIGLU ? 8 : 16;  // output features of a tile
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);                    // [WARPS][SLOTS][SLOT_ELEMS]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)WARPS * SLOTS * SLOT_ELEMS * 2);  // [2][WARPS][MT * 4][32]
    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(red + 2 * WARPS * MT * 4 * 32);  // [8 MT][K + X_PAD]
    __shared__ float row_scale[8 * MT];
    __shared__ __align__(8) unsigned long long full[WARPS][SLOTS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qr = lane >> 2, qc = lane & 3;
    const int M = p.M, N = p.N, K = p.K;
    const int x_pitch = K + X_PAD;

    if (lane == 0) {
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl) tma::mbar_init(&full[warp][sl], 1);
        tma::mbar_fence_init();
        if (warp == 0) tma::prefetch_map(&wmap);
    }
    __syncwarp();

    // Work: `group` warps of a CTA (1, 2, 4 or 8: more when there are few tiles, so that every SM streams)
    // share a tile and take its k-blocks in turn; consecutive tiles go to different CTAs first.
    const int group = p.group, member = warp % group;
    const int tiles = (N + FEATURES - 1) / FEATURES, kblocks = (K + BOXK - 1) / BOXK;
    const int first = blockIdx.x + (warp / group) * gridDim.x, stride = gridDim.x * (WARPS / group);
    const int my_tiles = tiles > first ? (tiles - 1 - first) / stride + 1 : 0;
    const int my_kblocks = kblocks > member ? (kblocks - 1 - member) / group + 1 : 0;
    const int units = my_tiles * my_kblocks;
    __nv_bfloat16* my_ring = ring + (size_t)warp * SLOTS * SLOT_ELEMS;
    bool gave_up = false;

    int a_ti = 0, a_kb = member, armed = 0;  // the producer's cursor: the next unit to ask for
    auto arm = [&]() {                       // lane 0 only
        const int tile = first + a_ti * stride, sl = armed % SLOTS;
        __nv_bfloat16* dst = my_ring + (size_t)sl * SLOT_ELEMS;
        tma::mbar_expect_tx(&full[warp][sl], (unsigned)(SLOT_ELEMS * 2));
        if (MODE == MODE_SWIGLU) {  // the map's box is 8 rows: gate rows, then up rows
            tma::load_2d(dst, &wmap, a_kb * BOXK, tile * 8, &full[warp][sl]);
            tma::load_2d(dst + 8 * BOXK, &wmap, a_kb * BOXK, p.up_offset + tile * 8, &full[warp][sl]);
        } else if (MODE == MODE_QKV) {  // 8 lanes of a head's first half, then their partners in the second half
            const int per_head = p.D >> 4, head = tile / per_head, y = head * p.D + (tile - head * per_head) * 8;
            tma::load_2d(dst, &wmap, a_kb * BOXK, y, &full[warp][sl]);
            tma::load_2d(dst + 8 * BOXK, &wmap, a_kb * BOXK, y + (p.D >> 1), &full[warp][sl]);
        } else {
            tma::load_2d(dst, &wmap, a_kb * BOXK, tile * 16, &full[warp][sl]);
        }
        ++armed;
        a_kb += group;
        if (a_kb >= kblocks) {
            a_kb = member;
            ++a_ti;
        }
    };
    // the weights do not depend on what ran before: their first boxes are asked for at once, while the
    // kernel before this one may still be running; everything else waits for it
    if (lane == 0)
        while (armed < SLOTS - 1 && armed < units) arm();
    // and the weights of a later product start their way into L2, a slice per CTA, 4 KB per instruction
    if (p.prefetch && warp == WARPS - 1) {
        const unsigned long long per_cta = ((p.prefetch_bytes / gridDim.x) + 4095) & ~4095ull;
        const unsigned long long begin = per_cta * blockIdx.x;
        const unsigned long long end = begin + per_cta < p.prefetch_bytes ? begin + per_cta : p.prefetch_bytes;
        for (unsigned long long off = begin + (unsigned long long)lane * 4096; off < end; off += 32ull * 4096) {
            const unsigned bytes = (unsigned)((end - off < 4096 ? end - off : 4096) & ~15ull);
            if (bytes)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"((const char*)p.prefetch + off), "r"(bytes) : "memory");
        }
    }
    pdl_trigger();
    pdl_wait();

    // x into shared memory (rows beyond M as zeros), and the input rows' RMS scale from the partial sums of
    // squares: warp w sums rows w, w + 8, ...; its lanes take the parts in strides of 32 (a fixed order)
    {
        const int per_row = K >> 3;
        for (int idx = tid; idx < 8 * MT * per_row; idx += THREADS) {
            const int m = idx / per_row, c = idx - m * per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < M) v = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + c * 8);
            *reinterpret_cast<uint4*>(x_s + (size_t)m * x_pitch + c * 8) = v;
        }
    }
    for (int m = warp; m < 8 * MT; m += WARPS) {
        float s = 1.f;
        if (p.in_ss && m < M) {
            float sum = 0.f;
            for (int i = lane; i < p.in_parts; i += 32) sum += p.in_ss[(size_t)i * M + m];
            s = rsqrtf(warp_sum(sum) / (float)K + p.in_eps);
        }
        if (lane == 0) row_scale[m] = s;
    }
    __syncthreads();  // the only CTA-wide barrier

    const __nv_bfloat16* xrow[MT];  // this thread's x rows: token 8 t + qr
#pragma unroll
    for (int t = 0; t < MT; ++t) xrow[t] = x_s + (size_t)(8 * t + qr) * x_pitch + qc * 8;

    int unit = 0;
    for (int ti = 0; ti < my_tiles; ++ti) {
        float acc[MT][4];
#pragma unroll
        for (int t = 0; t < MT; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
        for (int kb = member; kb < kblocks; kb += group, ++unit) {
            // the slot used one unit ago is free (the __syncwarp below): ask for the box three units ahead
            if (lane == 0 && armed < units) arm();
            if (!gave_up && !tma::mbar_wait(&full[warp][unit % SLOTS], (unit / SLOTS) & 1)) {
                gave_up = true;
                if (p.error_flag) atomicExch(p.error_flag, 1);
            }
            const __nv_bfloat16* slot = my_ring + (size_t)(unit % SLOTS) * SLOT_ELEMS + qc * 8;
            const int k0 = kb * BOXK;
            uint4 a[PIECES][2], b[PIECES][MT];
#pragma unroll
            for (int i = 0; i < PIECES; ++i) {
                a[i][0] = *reinterpret_cast<const uint4*>(slot + qr * BOXK + i * 32);
                a[i][1] = *reinterpret_cast<const uint4*>(slot + (qr + 8) * BOXK + i * 32);
                // beyond K the weights arrived as zeros and x is not read (its row ends there)
                const bool have = k0 + i * 32 + qc * 8 < K;
#pragma unroll
                for (int t = 0; t < MT; ++t)
                    b[i][t] = have ? *reinterpret_cast<const uint4*>(xrow[t] + k0 + i * 32) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int i = 0; i < PIECES; ++i)
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    mma_bf16(acc[t], a[i][0].x, a[i][1].x, a[i][0].y, a[i][1].y, b[i][t].x, b[i][t].y);
                    mma_bf16(acc[t], a[i][0].z, a[i][1].z, a[i][0].w, a[i][1].w, b[i][t].z, b[i][t].w);
                }
            __syncwarp();  // every lane has read the slot: it may be refilled
        }
        if (group > 1) {
            // the members' partial sums meet in shared memory (two buffers by tile parity: the first member may
            // still be reading the tile before when the others write this one); the first member adds them up
            float* buf = red + (size_t)(ti & 1) * WARPS * (MT * 4) * 32;
            if (member != 0) {
#pragma unroll
                for (int t = 0; t < MT; ++t)
#pragma unroll
                    for (int e = 0; e < 4; ++e) buf[((size_t)warp * (MT * 4) + t * 4 + e) * 32 + lane] = acc[t][e];
            }
            asm volatile("bar.sync %0, %1;\n" ::"r"(1 + warp / group), "r"(group * 32) : "memory");
            if (member != 0) continue;
            for (int w2 = warp + 1; w2 < warp + group; ++w2)
#pragma unroll
                for (int t = 0; t < MT; ++t)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[t][e] += buf[((size_t)w2 * (MT * 4) + t * 4 + e) * 32 + lane];
        }
        // the tile is complete
        const int tile = first + ti * stride, n0 = tile * FEATURES;
        if constexpr (MODE == MODE_QKV) {
            // this thread: lanes j (e = 0, 1) and j + D/2 (e = 2, 3) of one head for tokens 8 t + 2 qc and + 1:
            // a rotation pair.  Query heads go to `out` rotated, key heads rotated into their page, value heads as
            // they are into theirs.
            const int D = p.D, half = D >> 1, per_head = D >> 4;
            const int head = tile / per_head, j = (tile - head * per_head) * 8 + qr;
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int m = 8 * t + 2 * qc + i;
                    if (m >= M) continue;
                    float a = acc[t][i] * row_scale[m], b = acc[t][2 + i] * row_scale[m];
                    if (head < p.H + p.KV && p.rotary) {
                        const int pos = min(max(p.positions[m], 0), p.rotary_rows - 1);
                        const float c = p.rotary[(size_t)pos * D + j], sn = p.rotary[(size_t)pos * D + half + j];
                        const float ra = a * c - b * sn, rb = b * c + a * sn;
                        a = ra;
                        b = rb;
                    }
                    __nv_bfloat16* dst;
                    if (head < p.H) {
                        dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + head * D + j;
                    } else {
                        const int slot = p.slot_map[m], page = slot / p.page_size, off = slot - page * p.page_size;
                        const int is_v = head >= p.H + p.KV, kvh = head - p.H - (is_v ? p.KV : 0);
                        dst = p.pool + (((size_t)(page * 2 + is_v) * p.KV + kvh) * p.page_size + off) * D + j;
                    }
                    dst[0] = __float2bfloat16_rn(a);
                    dst[half] = __float2bfloat16_rn(b);
                }
        } else if constexpr (MODE == MODE_SWIGLU) {
            // this thread: gate (e = 0, 1) and up (e = 2, 3) sums of feature qr for tokens 8 t + 2 qc and + 1
            const int n = n0 + qr;
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int m = 8 * t + 2 * qc + j;
                    const float g = acc[t][j] * row_scale[m], u = acc[t][2 + j] * row_scale[m];
                    if (m < M && n < N) reinterpret_cast<TO*>(p.out)[(size_t)m * p.ldo + n] = from_float<TO>(g / (1.f + expf(-g)) * u);
                }
        } else {
            // this thread: features qr (e = 0, 1) and qr + 8 (e = 2, 3) of tokens 8 t + 2 qc and + 1
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                float sq[2] = {0.f, 0.f};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int n = n0 + qr + 8 * (e >> 1), m = 8 * t + 2 * qc + (e & 1);
                    const bool live = m < M && n < N;
                    const float s = acc[t][e] * row_scale[m];
                    if constexpr (MODE == MODE_RESIDUAL) {
                        if (live) {
                            const float v = p.resid[(size_t)m * N + n] + s;
                            p.resid[(size_t)m * N + n] = v;
                            p.xw_out[(size_t)m * N + n] = __float2bfloat16_rn(v * p.norm_w[n]);
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
    }
    // nothing of this warp's is in flight: every armed unit was waited for above (after a failed wait, once
    // more here, bounded, so that no copy lands in shared memory after the CTA has left)
    if (gave_up && lane == 0)
        for (unit = max(0, units - SLOTS); unit < units; ++unit) tma::mbar_wait(&full[warp][unit % SLOTS], (unit / SLOTS) & 1);
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

// Tensor maps of weight matrices, made once per (address, shape, box).
const CUtensorMap* weight_map(const void* w, int rows, int K, int box_rows) {
    struct Key {
        const void* w;
        int rows, K, box;
        bool operator==(const Key& o) const { return w == o.w && rows == o.rows && K == o.K && box == o.box; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return std::hash<const void*>()(k.w) ^ ((size_t)k.rows << 20) ^ ((size_t)k.K << 4) ^ (size_t)k.box;
        }
    };
    static std::unordered_map<Key, CUtensorMap, Hash> maps;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    auto it = maps.find(Key{w, rows, K, box_rows});
    if (it != maps.end()) return &it->second;
    CUtensorMap map;
    if (!tma::make_map_2d_bf16(&map, w, rows, K, K, box_rows, BOXK, CU_TENSOR_MAP_SWIZZLE_NONE)) return nullptr;
    return &maps.emplace(Key{w, rows, K, box_rows}, map).first->second;
}

constexpr size_t SMEM_LIMIT = 227 * 1024;

template <int MT, int MODE, typename TO>
int launch(const LinearParams& p, cudaStream_t stream) {
    constexpr int FEATURES = MODE == MODE_SWIGLU ? 8 : 16;
    const size_t smem = (size_t)WARPS * SLOTS * SLOT_ELEMS * 2 + (size_t)2 * WARPS * MT * 4 * 32 * sizeof(float) +
                        (size_t)8 * MT * (p.K + X_PAD) * 2;
    if (smem > SMEM_LIMIT) return LLM_ERR_UNSUPPORTED;  // x does not fit beside the rings
    auto kernel = linear_decode_kernel<MT, MODE, TO>;
    static size_t configured = 0;  // per instantiation: the most dynamic shared memory asked for so far
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const CUtensorMap* map = weight_map(p.w, MODE == MODE_SWIGLU ? p.up_offset + p.N : p.N, p.K, MODE == MODE_QKV ? 8 : FEATURES);
    if (!map) return LLM_ERR_UNSUPPORTED;
    const int tiles = (p.N + FEATURES - 1) / FEATURES;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    LinearParams q = p;
    q.group = 1;  // the most warps per tile (a power of two) that still leaves every warp of the grid a tile
    while (q.group < WARPS && (long long)tiles * q.group * 2 <= (long long)grid * WARPS) q.group *= 2;
    return launch_pdl(kernel, dim3(grid), dim3(THREADS), smem, stream, q, *map);
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
// rsqrt(sum / K + in_eps) per row.  Needs M <= 16, K a multiple of 8, 16-byte aligned rows;
// otherwise it returns LLM_ERR_UNSUPPORTED and the caller takes another route.  error_flag (host-visible
// int, or null) is set to 1 if a bounded wait inside the kernel ever gives up.  prefetch (or null): 16-byte
// aligned weights of a later product, pulled into L2 while this one runs.
LLM_EXPORT int llm_linear_decode(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int ldx,
                                 int ldo, const float* in_ss, int in_parts, float in_eps, int mode, int up_offset,
                                 float* resid, const float* norm_w, void* xw_out, float* ss_out, int* error_flag,
                                 const void* prefetch, unsigned long long prefetch_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K < 8 || (K & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return LLM_ERR_UNSUPPORTED;
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
    p.prefetch = prefetch;
    p.prefetch_bytes = prefetch ? prefetch_bytes : 0;
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
// query heads only and nothing is written to the pool.  Needs M <= 16, K and D multiples of 8 and 16.
LLM_EXPORT int llm_linear_decode_qkv(const void* x, const void* w, void* q_out, int M, int K, int ldx, const float* in_ss,
                                     int in_parts, float in_eps, const int* positions, const float* rotary, int rotary_rows,
                                     const int* slot_map, void* pool, int H, int KV, int D, int page_size, int* error_flag,
                                     cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 16 || K < 8 || (K & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || D < 16 || (D & 15) || H < 1 || KV < 0)
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
