// Next-token choice on the device: argmax, and temperature sampling with optional top-k and
// top-p, one block per row of 32-bit logits.
//
// The reference's sampler (src/llmserve/sampling/sampler.py:16-39) divides by the temperature,
// keeps the k largest (ties kept), drops a token when the probability mass before it in
// descending order exceeds top_p, and draws from the softmax of what is left.  The same rules
// are applied here without sorting: the k-th largest value and the top-p cut are found by a
// bitwise search over the order-preserving integer image of the floats, and the draw is the
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

__device__ __forceinline__ int block_count(int mine, float* scratch) {
    return (int)(block_sum((float)mine, scratch) + 0.5f);  // counts stay far below 2^24
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
              int* __restrict__ out) {
    __shared__ MaxIdx scratch_mi[33];
    __shared__ float scratch[33];
    __shared__ float partial[THREADS];
    const int rowi = blockIdx.x;
    const float* row = logits + (size_t)rowi * vocab;
    const float temp = temperature[rowi];
    const MaxIdx best = row_argmax(row, vocab, scratch_mi);
    if (!(temp > 0.f)) {
        if (threadIdx.x == 0) out[rowi] = best.i;
        return;
    }
    const float x_max = best.v / temp;

    // lowest key that stays after top-k: the k-th largest value (ties with it stay)
    unsigned floor_key = 0u;
    const int k = top_k[rowi];
    if (k > 0 && k < vocab) {
        unsigned t = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            int c = 0;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += ordered_key(row[i] / temp) >= cand;
            if (block_count(c, scratch) >= k) t = cand;
        }
        floor_key = t;
    }

    // normaliser over what top-k left
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i] / temp;
        if (ordered_key(x) >= floor_key) z += expf(x - x_max);
    }
    z = block_sum(z, scratch);

    // top-p: a token stays iff the mass of strictly larger values is <= top_p
    const float p_cut = top_p[rowi];
    if (p_cut < 1.f) {
        // Largest key t whose mass-above still exceeds top_p; tokens with larger keys stay.  The
        // mass above key 0 is all of it (no finite float maps to 0), which exceeds top_p < 1, so
        // the search starts from a key for which the condition holds.
        unsigned t = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            float above = 0.f;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const float x = row[i] / temp;
                const unsigned key = ordered_key(x);
                if (key >= floor_key && key > cand) above += expf(x - x_max);
            }
            above = block_sum(above, scratch);
            if (above > p_cut * z) t = cand;
        }
        floor_key = max(floor_key, t + 1u);
        z = 0.f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float x = row[i] / temp;
            if (ordered_key(x) >= floor_key) z += expf(x - x_max);
        }
        z = block_sum(z, scratch);
    }

    // inverse of the cumulative distribution in vocabulary order
    const float target = uniform_from(seeds[rowi], counters[rowi]) * z;
    const int seg = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(vocab, (int)threadIdx.x * seg), end = min(vocab, begin + seg);
    float local = 0.f;
    for (int i = begin; i < end; ++i) {
        const float x = row[i] / temp;
        if (ordered_key(x) >= floor_key) local += expf(x - x_max);
    }
    partial[threadIdx.x] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = 0.f;
        int owner = -1;
        for (int th = 0; th < (int)blockDim.x; ++th) {
            if (partial[th] > 0.f && run + partial[th] > target) {
                owner = th;
                break;
            }
            run += partial[th];
        }
        int token = -1;
        if (owner >= 0) {
            const int b = min(vocab, owner * seg), e = min(vocab, b + seg);
            for (int i = b; i < e; ++i) {
                const float x = row[i] / temp;
                if (ordered_key(x) < floor_key) continue;
                run += expf(x - x_max);
                token = i;  // the last kept token of the segment if rounding leaves the target unreached
                if (run > target) break;
            }
        }
        if (token < 0) {  // the target fell past the end by rounding: the last kept token
            for (int i = vocab - 1; i >= 0; --i)
                if (ordered_key(row[i] / temp) >= floor_key) {
                    token = i;
                    break;
                }
        }
        out[rowi] = token < 0 ? best.i : token;
    }
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
    sample_kernel<<<rows, THREADS, 0, stream>>>(logits, vocab, temperature, top_k, top_p, seeds, counters, out);
    return launch_status();
}
