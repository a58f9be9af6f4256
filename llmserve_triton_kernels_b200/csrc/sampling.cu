// Next-token choice on the device: argmax, and temperature sampling with optional top-k and
// top-p, one block per row of 32-bit logits.
//
// The reference's sampler (src/llmserve/sampling/sampler.py:16-39) divides by the temperature,
// keeps the k largest (ties kept), drops a token when the probability mass before it in
// descending order exceeds top_p, and draws from the softmax of what is left.  The same rules
// are applied here without sorting: the k-th largest value and the top-p cut are found by a
// radix search over the order-preserving integer image of the floats, and the draw is the
// inverse of the cumulative distribution in vocabulary order at a uniform number u that comes
// from a counter-based generator keyed by (seed, counter) — so a row's token depends on
// nothing but its logits, its parameters, its seed and how many tokens it has drawn before.
#include "common.cuh"

namespace {

constexpr int THREADS = 512;

__device__ __forceinline__ unsigned ordered_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long counter) {
    unsigned long long x = seed ^ (counter * 0x9E3779B97F4A7C15ULL + 0xD1B54A32D192ED03ULL);
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    x = x ^ (x >> 31);
    return (float)(x >> 40) * (1.0f / 16777216.0f);
}

struct MaxIdx {
    float v;
    int i;
};

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// Largest value and its lowest index over the block; every thread gets the result.
__device__ MaxIdx block_argmax(MaxIdx mine, MaxIdx* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other{__shfl_xor_sync(0xffffffffu, mine.v, o), __shfl_xor_sync(0xffffffffu, mine.i, o)};
        mine = better(mine, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    if (warp == 0) {
        const int nwarps = blockDim.x >> 5;
        MaxIdx t = lane < nwarps ? scratch[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxIdx other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ MaxIdx row_argmax(const float* row, int vocab, MaxIdx* scratch) {
    MaxIdx mine{-INFINITY, 0x7fffffff};
    if ((vocab & 3) == 0 && ((uintptr_t)row & 15) == 0) {
        // four loads of 16 bytes in flight per thread: the scan is bound by load latency, not by comparisons
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int n4 = vocab >> 2, step = blockDim.x;
        for (int i = threadIdx.x; i < n4; i += 4 * step) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = i + u * step < n4 ? row4[i + u * step] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int base = (i + u * step) * 4;
                mine = better(mine, MaxIdx{v[u].x, base});
                mine = better(mine, MaxIdx{v[u].y, base + 1});
                mine = better(mine, MaxIdx{v[u].z, base + 2});
                mine = better(mine, MaxIdx{v[u].w, base + 3});
            }
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) mine = better(mine, MaxIdx{row[i], i});
    }
    return block_argmax(mine, scratch);
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    __shared__ MaxIdx scratch[33];
    pdl_trigger();
    pdl_wait();
    const MaxIdx best = row_argmax(logits + (size_t)blockIdx.x * vocab, vocab, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = best.i;
}

// ---- temperature sampling -----------------------------------------------------------------------
//
// One block of 1024 threads per row.  The row, divided by its temperature, is kept in shared memory
// where it fits (a vocabulary of up to about 40,000); a larger one is read again from global memory
// (it lies in L2) in every pass.  Both cuts are radix searches over the keys, four bits a pass: a
// pass adds the weight of every element whose higher bits match the prefix found so far into the
// bin of its next four bits, and the prefix grows by the largest digit whose weight at and above it
// still passes the threshold.  Weights are 1 for top-k and exp(x - max) for top-p.  Every thread
// has its own sixteen bins in shared memory, so the additions need no atomics and their order is
// fixed.  After the first passes few elements match the prefix, so the later ones cost little.
constexpr int S_THREADS = 1024;
constexpr int S_WARPS = S_THREADS / 32;
constexpr int BINS = 16;

struct SampleShared {
    MaxIdx best[33];
    float sum[33];
    float halves[2 * BINS];
    float group[S_WARPS];
};

template <bool IN_SMEM>
__device__ __forceinline__ float scaled(const float* xs, const float* row, float temp, int i) {
    return IN_SMEM ? xs[i] : row[i] / temp;
}

// The largest key T for which G(T) > threshold, where G(T) is the summed weight of the elements
// that are kept (key >= floor_key) and have key >= T.  G(0) is taken to pass.
template <bool IN_SMEM, bool WEIGHTED>
__device__ unsigned radix_search(const float* xs, const float* row, float temp, int vocab, unsigned floor_key,
                                 float x_max, float threshold, float* bins, SampleShared& sh) {
    static_assert(2 * BINS == S_WARPS, "two warps add up one bin");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* mine = bins + threadIdx.x;  // this thread's share of bin j is mine[j * S_THREADS]: no two threads meet in a bank
    unsigned t = 0u;
    float base = 0.f;  // weight of the elements whose higher bits lie above the prefix
    for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
        for (int j = 0; j < BINS; ++j) mine[j * S_THREADS] = 0.f;
        for (int i = threadIdx.x; i < vocab; i += S_THREADS) {
            const float x = scaled<IN_SMEM>(xs, row, temp, i);
            const unsigned key = ordered_key(x);
            if (key < floor_key) continue;
            if (shift < 28 && (key >> (shift + 4)) != (t >> (shift + 4))) continue;
            mine[((key >> shift) & 15u) * S_THREADS] += WEIGHTED ? expf(x - x_max) : 1.f;
        }
        __syncthreads();
        {  // bin j: warps 2j and 2j+1 add half of the threads' shares each
            const float* b = bins + (warp >> 1) * S_THREADS + (warp & 1) * (S_THREADS / 2);
            float s = 0.f;
#pragma unroll
            for (int u = 0; u < S_THREADS / 64; ++u) s += b[u * 32 + lane];
            s = warp_sum(s);
            if (lane == 0) sh.halves[warp] = s;
        }
        __syncthreads();
        float above = base;  // weight above digit j, from the top digit down
        int digit = 0;
        for (int j = BINS - 1; j >= 1; --j) {
            const float with_j = above + (sh.halves[2 * j] + sh.halves[2 * j + 1]);
            if (with_j > threshold) {
                digit = j;
                break;
            }
            above = with_j;
        }
        base = above;
        t |= (unsigned)digit << shift;
    }
    return t;
}

template <bool IN_SMEM>
__global__ void __launch_bounds__(S_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
              int* __restrict__ out) {
    extern __shared__ __align__(16) float dyn[];
    __shared__ SampleShared sh;
    const int nseg = (vocab + 31) / 32;  // runs of 32 consecutive tokens
    float* bins = dyn;
    float* seg = bins + BINS * S_THREADS;
    float* xs = seg + nseg;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rowi = blockIdx.x;
    const float* row = logits + (size_t)rowi * vocab;
    const float temp = temperature[rowi];
    const bool greedy = !(temp > 0.f);

    // the largest logit, and the scaled row into shared memory; eight loads in flight per thread
    MaxIdx mine{-INFINITY, 0x7fffffff};
    for (int i0 = threadIdx.x; i0 < vocab; i0 += 8 * S_THREADS) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = i0 + u * S_THREADS < vocab ? row[i0 + u * S_THREADS] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * S_THREADS;
            if (i < vocab) {
                mine = better(mine, MaxIdx{v[u], i});
                if (IN_SMEM && !greedy) xs[i] = v[u] / temp;
            }
        }
    }
    const MaxIdx best = block_argmax(mine, sh.best);  // its barriers also publish xs
    if (greedy) {
        if (threadIdx.x == 0) out[rowi] = best.i;
        return;
    }
    const float x_max = best.v / temp;

    // lowest key that stays after top-k: the k-th largest value (ties with it stay)
    unsigned floor_key = 0u;
    const int k = top_k[rowi];
    if (k > 0 && k < vocab) floor_key = radix_search<IN_SMEM, false>(xs, row, temp, vocab, 0u, x_max, (float)k - 0.5f, bins, sh);

    // top-p: a token stays iff the mass of strictly larger values is <= top_p, that is, iff its key is at
    // least the largest key T whose mass at and above T still exceeds top_p
    const float p_cut = top_p[rowi];
    if (p_cut < 1.f) {
        float z = 0.f;
        for (int i = threadIdx.x; i < vocab; i += S_THREADS) {
            const float x = scaled<IN_SMEM>(xs, row, temp, i);
            if (ordered_key(x) >= floor_key) z += expf(x - x_max);
        }
        z = block_sum(z, sh.sum);
        floor_key = max(floor_key, radix_search<IN_SMEM, true>(xs, row, temp, vocab, floor_key, x_max, p_cut * z, bins, sh));
    }

    // Inverse of the cumulative distribution in vocabulary order, in three levels: the mass of every run of 32
    // tokens, of every group of runs (one group per warp), then a walk through one group and one run.
    for (int s = warp; s < nseg; s += S_WARPS) {
        const int i = s * 32 + lane;
        float e = 0.f;
        if (i < vocab) {
            const float x = scaled<IN_SMEM>(xs, row, temp, i);
            if (ordered_key(x) >= floor_key) e = expf(x - x_max);
        }
        e = warp_sum(e);
        if (lane == 0) seg[s] = e;
    }
    __syncthreads();
    const int per = (nseg + S_WARPS - 1) / S_WARPS;  // runs per group
    {
        float g = 0.f;
        for (int j = lane; j < per; j += 32) {
            const int s = warp * per + j;
            if (s < nseg) g += seg[s];
        }
        g = warp_sum(g);
        if (lane == 0) sh.group[warp] = g;
    }
    __syncthreads();
    if (warp != 0) return;
    float z = 0.f;
    for (int w = 0; w < S_WARPS; ++w) z += sh.group[w];
    const float target = uniform_from(seeds[rowi], counters[rowi]) * z;
    // the first group, run and token at which the running sum passes the target; where rounding lets it slip
    // through a level, the last one of that level that has any mass
    float run = 0.f;
    int g_found = -1, g_last = -1;
    float run_at_last = 0.f;
    for (int w = 0; w < S_WARPS; ++w) {
        const float g = sh.group[w];
        if (g > 0.f) {
            g_last = w;
            run_at_last = run;
            if (run + g > target) {
                g_found = w;
                break;
            }
        }
        run += g;
    }
    if (g_found < 0) g_found = g_last, run = run_at_last;
    int token = best.i;
    if (g_found >= 0) {
        int s_found = -1, s_last = -1;
        for (int j = 0; j < per; ++j) {
            const int s = g_found * per + j;
            if (s >= nseg) break;
            const float m = seg[s];
            if (m > 0.f) {
                s_last = s;
                run_at_last = run;
                if (run + m > target) {
                    s_found = s;
                    break;
                }
            }
            run += m;
        }
        if (s_found < 0) s_found = s_last, run = run_at_last;
        if (s_found >= 0) {
            const int i = s_found * 32 + lane;
            float e = 0.f;
            if (i < vocab) {
                const float x = scaled<IN_SMEM>(xs, row, temp, i);
                if (ordered_key(x) >= floor_key) e = expf(x - x_max);
            }
            int l_found = -1, l_last = -1;
            for (int l = 0; l < 32; ++l) {
                const float m = __shfl_sync(0xffffffffu, e, l);
                if (l_found >= 0) continue;
                if (m > 0.f) {
                    l_last = l;
                    if (run + m > target) l_found = l;
                }
                run += m;
            }
            if (l_found < 0) l_found = l_last;
            if (l_found >= 0) token = s_found * 32 + l_found;
        }
    }
    if (lane == 0) out[rowi] = token;
}

}  // namespace

LLM_EXPORT int llm_argmax(const float* logits, int rows, int vocab, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return LLM_ERR_BAD_ARGUMENT;
    return launch_pdl(argmax_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, vocab, out);
}

LLM_EXPORT int llm_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                          const float* top_p, const unsigned long long* seeds, const unsigned long long* counters,
                          int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return LLM_ERR_BAD_ARGUMENT;
    static const int smem_limit = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        return v - (int)sizeof(SampleShared) - 1024;
    }();
    const size_t seg_bytes = (size_t)(BINS * S_THREADS + (vocab + 31) / 32) * sizeof(float);
    const size_t row_bytes = (size_t)vocab * sizeof(float);
    if ((long long)(seg_bytes + row_bytes) <= (long long)smem_limit) {
        static const cudaError_t opted =
            cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_limit);
        if (opted != cudaSuccess) return (int)opted;
        sample_kernel<true><<<rows, S_THREADS, seg_bytes + row_bytes, stream>>>(logits, vocab, temperature, top_k, top_p, seeds, counters, out);
    } else {
        if ((long long)seg_bytes > (long long)smem_limit) return LLM_ERR_UNSUPPORTED;
        static const cudaError_t opted =
            cudaFuncSetAttribute(sample_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_limit);
        if (opted != cudaSuccess) return (int)opted;
        sample_kernel<false><<<rows, S_THREADS, seg_bytes, stream>>>(logits, vocab, temperature, top_k, top_p, seeds, counters, out);
    }
    return launch_status();
}
