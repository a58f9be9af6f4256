// y[M, N] = x[M, K] * w[N, K]^T on the CUDA cores with 32-bit fused multiply-adds.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-precision
// mode), and it takes every size.  Each output element is accumulated by one thread, k-tile
// by k-tile in ascending k, so a row's result does not depend on how many other rows are in the
// batch or where the row lies in it.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out, int M, int N, int K,
                 int ldx, int ldw, int ldo) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int lrow = tid / 4, lk = (tid % 4) * 4;  // each thread stages 4 consecutive k of one row

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int m = m0 + lrow, n = n0 + lrow;
            xs[lk + e][lrow] = (m < M && k < K) ? to_float(x[(size_t)m * ldx + k]) : 0.f;
            ws[lk + e][lrow] = (n < N && k < K) ? to_float(w[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
        // a partial sum per k-tile, then one addition into the total: the rounding error grows with
        // sqrt(K / BK) instead of sqrt(K), and the order is still fixed
        float part[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) part[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) out[(size_t)m * ldo + n] = from_float<TO>(acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TO>
int launch(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
           cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_simt_kernel<TX, TW, TO><<<grid, THREADS, 0, stream>>>((const TX*)x, (const TW*)w, (TO*)out, M, N, K, ldx,
                                                               ldw, ldo);
    return launch_status();
}

}  // namespace

LLM_EXPORT int llm_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype, int M,
                             int N, int K, int ldx, int ldw, int ldo, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K < 0 || ldx < K || ldw < K || ldo < N) return LLM_ERR_BAD_ARGUMENT;
    if ((M + BM - 1) / BM > 65535) return LLM_ERR_UNSUPPORTED;
    using bf = __nv_bfloat16;
    if (x_dtype == LLM_F32 && w_dtype == LLM_F32 && out_dtype == LLM_F32)
        return launch<float, float, float>(x, w, out, M, N, K, ldx, ldw, ldo, stream);
    if (x_dtype == LLM_BF16 && w_dtype == LLM_BF16 && out_dtype == LLM_BF16)
        return launch<bf, bf, bf>(x, w, out, M, N, K, ldx, ldw, ldo, stream);
    if (x_dtype == LLM_BF16 && w_dtype == LLM_BF16 && out_dtype == LLM_F32)
        return launch<bf, bf, float>(x, w, out, M, N, K, ldx, ldw, ldo, stream);
    return LLM_ERR_BAD_ARGUMENT;
}
