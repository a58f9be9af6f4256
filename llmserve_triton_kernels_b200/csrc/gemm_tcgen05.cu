// y[M, N] = x[M, K] * w[N, K]^T in bfloat16 on the fifth-generation tensor cores (tcgen05) for
// many rows (prompt portions): operands staged in shared memory by TMA, accumulators in tensor
// memory, read back with tcgen05.ld for the epilogue.
//
// One CTA per SM walks 128 x BN tiles of y (tile t, t + CTAs, ...).  Three roles, chosen by warp:
//   warp 0, one thread : TMA producer — fills a ring of STAGES slots with a 128 x 64 tile of x and a
//                        BN x 64 tile of w (two of them in MODE_SWIGLU: the gate's and the up's rows
//                        of the same features), 128-byte swizzled, and arms the slot's mbarrier;
//   warp 1, one thread : issues tcgen05.mma (M = 128, N = BN, K = 16, four per slot) into tensor
//                        memory and commits to the slot's "empty" mbarrier, so that the slot is
//                        refilled as soon as the tensor cores have read it; warp 1 also owns the
//                        allocation of tensor memory;
//   warps 2-5          : epilogue — each warp reads its 32 lanes of the accumulator, 32 columns at a
//                        time, and writes bfloat16 or float32 rows (MODE_SWIGLU: silu(gate) * up).
// Tensor memory holds two accumulators: the epilogue of a tile runs while the products of the CTA's next
// tile fill the other one, and the producer runs on into the next tile's k-blocks without a pause.
// Rows and columns beyond the matrices arrive as zeros from TMA and are masked at the store; K may
// be any multiple of 8.  Every mbarrier wait is bounded; a wait that gives up sets *error_flag, the
// roles leave their loops, tensor memory is freed and the kernel returns.
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_RESIDUAL = 2;

struct GemmParams {
    void* out;
    int M, N, K, ldo;
    int up_offset;  // MODE_SWIGLU: row of w where the up matrix starts
    int* error_flag;
    // input in factored normalised form (see llm_linear_decode): x holds v * norm_weight, in_ss [in_parts, M] partial
    // sums of v^2 per row; the product's rows are scaled by rsqrt(sum / K + in_eps).  Null: x is what it is.
    const float* in_ss;
    int in_parts;
    float in_eps;
    // MODE_RESIDUAL: the product is added to resid [M, N] (float32, in place); xw_out [M, N] = resid * norm_w in
    // bfloat16 and ss_out [column tiles, M] = partial sums of resid^2 hand the stream on for the next norm
    float* resid;
    const float* norm_w;
    __nv_bfloat16* xw_out;
    float* ss_out;
};

template <typename TO>
__device__ __forceinline__ void store32(TO* dst, const float (&v)[32], int valid);
template <>
__device__ __forceinline__ void store32<float>(float* dst, const float (&v)[32], int valid) {
    if (valid == 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = v[i];
    }
}
template <>
__device__ __forceinline__ void store32<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[32], int valid) {
    if (valid == 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            uint4 u;
            __nv_bfloat162 a = __floats2bfloat162_rn(v[i], v[i + 1]), b = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
            __nv_bfloat162 c = __floats2bfloat162_rn(v[i + 4], v[i + 5]), d = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
            u.x = *reinterpret_cast<unsigned*>(&a);
            u.y = *reinterpret_cast<unsigned*>(&b);
            u.z = *reinterpret_cast<unsigned*>(&c);
            u.w = *reinterpret_cast<unsigned*>(&d);
            *reinterpret_cast<uint4*>(dst + i) = u;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = __float2bfloat16_rn(v[i]);
    }
}

template <int BN, int MODE, int STAGES, typename TO>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap) {
    constexpr int NB = MODE == MODE_SWIGLU ? 2 : 1;           // w tiles per slot
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr int SLOT_BYTES = A_BYTES + NB * B_BYTES;
    // MODE_SWIGLU: the gate's and the up's tiles lie one after the other in the slot, which is one K-major tile of
    // 2 BN rows: one product of N = 2 BN fills columns [0, BN) with the gate's sums and [BN, 2 BN) with the up's
    constexpr int UMMA_N = NB * BN;
    static_assert(UMMA_N % 16 == 0 && UMMA_N >= 16 && UMMA_N <= 256, "tcgen05.mma with M = 128 takes N in steps of 16 up to 256");
    // two accumulators, so that the epilogue of a tile runs under the products of the next one
    constexpr int ACC_COLS = UMMA_N <= 32 ? 32 : UMMA_N <= 64 ? 64 : UMMA_N <= 128 ? 128 : 256;
    constexpr int TMEM_COLS = 2 * ACC_COLS;
    constexpr unsigned IDESC = umma::idesc_bf16(BM, UMMA_N, false);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* epi_s = reinterpret_cast<float*>(ring + (size_t)STAGES * SLOT_BYTES);  // MODE_RESIDUAL: [4 warps][32][33]
    __shared__ __align__(8) unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base;
    __shared__ int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.K + BK - 1) / BK;
    // tiles in row-major order of (column tile, row tile): CTAs that run at the same time share their w tiles
    const int row_tiles = (p.M + BM - 1) / BM, col_tiles = (p.N + BN - 1) / BN, tiles = row_tiles * col_tiles;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            tma::mbar_init(&full[s], 1);
            tma::mbar_init(&empty[s], 1);
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            tma::mbar_init(&acc_full[b], 1);
            tma::mbar_init(&acc_empty[b], 4);
        }
        gave_up = 0;
        tma::mbar_fence_init();
        tma::prefetch_map(&xmap);
        tma::prefetch_map(&wmap);
    }
    if (warp == 1) {  // one warp allocates the accumulators' columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma::smem_addr(&tmem_base)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    pdl_trigger();
    pdl_wait();  // x comes from the kernel before

    auto fail = [&]() {
        gave_up = 1;
        if (p.error_flag) atomicExch(p.error_flag, 1);
    };

    if (warp == 0 && lane == 0) {
        // ---- producer: the k-blocks of all of this CTA's tiles, one after the other through the ring ----
        int it = 0;
        for (int tile = blockIdx.x; tile < tiles && !gave_up; tile += gridDim.x) {
            const int m0 = (tile % row_tiles) * BM, n0 = (tile / row_tiles) * BN;
            for (int kb = 0; kb < kblocks && !gave_up; ++kb, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !tma::mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) {
                    fail();
                    break;
                }
                unsigned char* slot = ring + (size_t)s * SLOT_BYTES;
                tma::mbar_expect_tx(&full[s], SLOT_BYTES);
                tma::load_2d(slot, &xmap, kb * BK, m0, &full[s]);
                tma::load_2d(slot + A_BYTES, &wmap, kb * BK, n0, &full[s]);
                if (NB == 2) tma::load_2d(slot + A_BYTES + B_BYTES, &wmap, kb * BK, p.up_offset + n0, &full[s]);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- tensor-core issuer ----
        int it = 0, i = 0;
        for (int tile = blockIdx.x; tile < tiles && !gave_up; tile += gridDim.x, ++i) {
            const int buf = i & 1;
            const unsigned d_tmem = tmem_base + buf * ACC_COLS;
            if (i >= 2 && !tma::mbar_wait(&acc_empty[buf], ((i >> 1) - 1) & 1)) {  // the epilogue has read this accumulator
                fail();
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            for (int kb = 0; kb < kblocks && !gave_up; ++kb, ++it) {
                const int s = it % STAGES;
                if (!tma::mbar_wait(&full[s], (it / STAGES) & 1)) {
                    fail();
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* slot = ring + (size_t)s * SLOT_BYTES;
                const unsigned long long a = umma::desc_sw128(slot), b = umma::desc_sw128(slot + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // 16 k = 32 bytes further along the 128-byte rows: the start address moves by two 16-byte units
                    umma::mma_bf16(d_tmem, a + 2 * k, b + 2 * k, IDESC, (kb | k) != 0);
                }
                umma::commit(&empty[s]);  // arrives when the products above have read the slot
            }
            umma::commit(&acc_full[buf]);  // arrives when every product of the tile has landed in tensor memory
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w may touch the 32 lanes (warp % 4) * 32 .. of tensor memory ----
        const int quarter = warp & 3;
        int i = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++i) {
            const int buf = i & 1;
            const int m0 = (tile % row_tiles) * BM, n0 = (tile / row_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            const bool ok = __all_sync(0xffffffffu, !gave_up && tma::mbar_wait(&acc_full[buf], (i >> 1) & 1));
            if (!ok) {
                if (lane == 0) fail();
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned lane_base = tmem_base + buf * ACC_COLS + ((unsigned)(quarter * 32) << 16);
            float row_scale = 1.f;
            if (p.in_ss && row < p.M) {
                float sum = 0.f;
                for (int part = 0; part < p.in_parts; ++part) sum += p.in_ss[(size_t)part * p.M + row];  // a fixed order
                row_scale = rsqrtf(sum / (float)p.K + p.in_eps);
            }
            float squares[MODE == MODE_RESIDUAL ? 32 : 1];  // per row of the warp's 32, this lane's columns
#pragma unroll
            for (int rr = 0; rr < (MODE == MODE_RESIDUAL ? 32 : 1); ++rr) squares[rr] = 0.f;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                float v[32];
                umma::tmem_ld32(lane_base + c, v);
                const int col = n0 + c;
                if (MODE == MODE_SWIGLU) {
                    float u[32];
                    umma::tmem_ld32(lane_base + BN + c, u);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float g = v[j] * row_scale;
                        v[j] = __fdividef(g, 1.f + __expf(-g)) * (u[j] * row_scale);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] *= row_scale;
                }
                if constexpr (MODE == MODE_RESIDUAL) {
                    // The thread holds 32 columns of ONE row; the stream wants a warp on 32 columns of one row at a
                    // time (128 bytes side by side).  The warp's 32 x 32 piece turns round in shared memory.
                    float* turn = epi_s + (size_t)(warp - 2) * 32 * 33;
#pragma unroll
                    for (int j = 0; j < 32; ++j) turn[lane * 33 + j] = v[j];
                    __syncwarp();
                    const int my_col = col + lane;
                    const bool col_ok = my_col < p.N;
                    const float w_here = col_ok ? p.norm_w[my_col] : 0.f;
                    // every load of the stream goes out before the first store (the compiler cannot know that the
                    // stores do not touch what the later loads read)
                    float before[32];
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr) {
                        const int r_g = m0 + quarter * 32 + rr;
                        before[rr] = r_g < p.M && col_ok ? __ldcg(p.resid + (size_t)r_g * p.N + my_col) : 0.f;
                    }
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr) {
                        const int r_g = m0 + quarter * 32 + rr;
                        if (r_g < p.M && col_ok) {
                            const size_t at = (size_t)r_g * p.N + my_col;
                            const float r = before[rr] + turn[rr * 33 + lane];
                            p.resid[at] = r;
                            p.xw_out[at] = __float2bfloat16_rn(r * w_here);
                            squares[rr] += r * r;
                        }
                    }
                    __syncwarp();
                    continue;
                }
                if (row >= p.M || col >= p.N) continue;
                store32<TO>(reinterpret_cast<TO*>(p.out) + (size_t)row * p.ldo + col, v, min(32, p.N - col));
            }
            if constexpr (MODE == MODE_RESIDUAL) {
#pragma unroll
                for (int rr = 0; rr < 32; ++rr) {
                    const float total = warp_sum(squares[rr]);
                    const int r_g = m0 + quarter * 32 + rr;
                    if (lane == 0 && r_g < p.M) p.ss_out[(size_t)(tile / row_tiles) * p.M + r_g] = total;
                }
            }
            // this warp has read its lanes of the accumulator: the tile after next may overwrite them
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&acc_empty[buf]);
        }
    }
    // everyone is done with tensor memory: the allocating warp gives it back
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
    }
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

template <int BN, int MODE, int STAGES, typename TO>
int launch(const void* x, int ldx, const void* w, int w_rows, const GemmParams& p, cudaStream_t stream) {
    constexpr int NB = MODE == MODE_SWIGLU ? 2 : 1;
    constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + NB * BN * BK * 2) + 1024 + (MODE == MODE_RESIDUAL ? 4 * 32 * 33 * sizeof(float) : 0);
    auto kernel = gemm_tcgen05_kernel<BN, MODE, STAGES, TO>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const CUtensorMap* xmap = tma::cached_map_2d_bf16(x, p.M, p.K, ldx, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    const CUtensorMap* wmap = tma::cached_map_2d_bf16(w, w_rows, p.K, p.K, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!xmap || !wmap) return LLM_ERR_UNSUPPORTED;
    const long long tiles = (long long)((p.N + BN - 1) / BN) * ((p.M + BM - 1) / BM);
    if (tiles > 0x7fffffffLL) return LLM_ERR_UNSUPPORTED;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());  // one CTA per SM walks its share of the tiles
    return launch_pdl(kernel, dim3(grid), dim3(THREADS), smem, stream, p, *xmap, *wmap);
}

}  // namespace

// How many partial sums of squares per row mode 2 writes for N features (its tiles are 256 columns wide).
LLM_EXPORT int llm_gemm_tcgen05_parts(int N) { return (N + 255) / 256; }

// bfloat16 x [M, K] (row stride ldx, a multiple of 8) times w^T (w contiguous [N or up_offset + N, K]).
//   mode 0: out [M, N] (row stride ldo) in bfloat16 or float32.
//   mode 1: w = [gate | up], the up rows starting at row up_offset; out [M, N] bfloat16 = silu(gate) * up.
//   mode 2: resid [M, N] (float32) += product; xw_out [M, N] = resid * norm_w (bfloat16); ss_out
//           [llm_gemm_tcgen05_parts(N), M] = partial sums of resid^2.  out is not used; N a multiple of 8.
// in_ss (or null): [in_parts, M] partial sums of squares of the rows that x was made from; the product's rows are
// scaled by rsqrt(sum / K + in_eps).  Needs K a multiple of 8 and 16-byte aligned bases; otherwise LLM_ERR_UNSUPPORTED.
LLM_EXPORT int llm_gemm_tcgen05_fused(const void* x, int ldx, const void* w, void* out, int out_dtype, int M, int N, int K, int ldo,
                                      int mode, int up_offset, const float* in_ss, int in_parts, float in_eps, float* resid,
                                      const float* norm_w, void* xw_out, float* ss_out, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K < 8 || (K & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return LLM_ERR_UNSUPPORTED;
    GemmParams p = {};
    p.out = out;
    p.M = M;
    p.N = N;
    p.K = K;
    p.ldo = ldo;
    p.up_offset = up_offset;
    p.error_flag = error_flag;
    p.in_ss = in_ss;
    p.in_parts = in_ss ? in_parts : 0;
    p.in_eps = in_eps;
    if (mode == MODE_RESIDUAL) {
        if (!resid || !norm_w || !xw_out || !ss_out) return LLM_ERR_BAD_ARGUMENT;
        if ((N & 7) || ((uintptr_t)resid & 15) || ((uintptr_t)norm_w & 15) || ((uintptr_t)xw_out & 15)) return LLM_ERR_UNSUPPORTED;
        p.resid = resid;
        p.norm_w = norm_w;
        p.xw_out = (__nv_bfloat16*)xw_out;
        p.ss_out = ss_out;
        return launch<256, MODE_RESIDUAL, 4, __nv_bfloat16>(x, ldx, w, N, p, stream);
    }
    if (mode == MODE_SWIGLU) {
        if (out_dtype != LLM_BF16) return LLM_ERR_BAD_ARGUMENT;
        return launch<128, MODE_SWIGLU, 4, __nv_bfloat16>(x, ldx, w, up_offset + N, p, stream);
    }
    if (mode != MODE_PLAIN) return LLM_ERR_BAD_ARGUMENT;
    // the tile width that wastes the fewest SM-rounds: wide tiles re-read x less often, but the last round of
    // CTAs should not be nearly empty
    const int row_tiles = (M + BM - 1) / BM, sms = sm_count();
    int best = 128;
    double best_cost = 1e30;
    for (int bn : {256, 192, 160, 128}) {
        const long long tiles = (long long)((N + bn - 1) / bn) * row_tiles;
        const double rounds = (double)((tiles + sms - 1) / sms);
        const double cost = rounds * bn * (bn == 256 ? 1.0 : bn == 192 ? 1.03 : bn == 160 ? 1.06 : 1.12);
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    if (out_dtype == LLM_BF16) {
        if (best == 256) return launch<256, MODE_PLAIN, 4, __nv_bfloat16>(x, ldx, w, N, p, stream);
        if (best == 192) return launch<192, MODE_PLAIN, 5, __nv_bfloat16>(x, ldx, w, N, p, stream);
        if (best == 160) return launch<160, MODE_PLAIN, 5, __nv_bfloat16>(x, ldx, w, N, p, stream);
        return launch<128, MODE_PLAIN, 6, __nv_bfloat16>(x, ldx, w, N, p, stream);
    }
    if (out_dtype == LLM_F32) {
        if (best >= 192) return launch<256, MODE_PLAIN, 4, float>(x, ldx, w, N, p, stream);
        return launch<128, MODE_PLAIN, 6, float>(x, ldx, w, N, p, stream);
    }
    return LLM_ERR_BAD_ARGUMENT;
}

LLM_EXPORT int llm_gemm_tcgen05(const void* x, int ldx, const void* w, void* out, int out_dtype, int M, int N, int K, int ldo,
                                int mode, int up_offset, int* error_flag, cudaStream_t stream) {
    if (mode != MODE_PLAIN && mode != MODE_SWIGLU) return LLM_ERR_BAD_ARGUMENT;
    return llm_gemm_tcgen05_fused(x, ldx, w, out, out_dtype, M, N, K, ldo, mode, up_offset, nullptr, 0, 0.f, nullptr, nullptr, nullptr,
                                  nullptr, error_flag, stream);
}
