// Row-wise kernels: token embedding, RMS norm fused with the residual sum, rotary encoding fused
// with the write of keys and values into their pages, the gated activation, and a projection's bias.
//
// All of them are bound by memory traffic; each row is read once and written once.  Statistics,
// angles and the residual sum are 32-bit whatever the element type.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// embedding: out[t, :] = float(table[ids[t], :])
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                             int hidden, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;  // launch-side checks reject such ids; never read out of range
    const T* src = table + (size_t)id * hidden;
    float* dst = out + (size_t)t * hidden;
    if ((hidden & 3) == 0) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float v[4];
            load4(src + i, v);
            store4(dst + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]);
    }
}

LLM_EXPORT int llm_embed(const int* ids, const void* table, int table_dtype, float* out, int n, int hidden,
                         int vocab, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == LLM_F32)
        return launch_pdl(embed_kernel<float>, dim3(n), dim3(threads), 0, stream, ids, (const float*)table, out, hidden, vocab);
    if (table_dtype == LLM_BF16)
        return launch_pdl(embed_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream, ids, (const __nv_bfloat16*)table, out, hidden, vocab);
    return LLM_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// RMS norm with the residual sum: v = resid[row] (+ delta[row]); resid[row] = v (when all rows are
// produced); out[i] = v * rsqrt(mean(v^2) + eps) * weight.  `rows` selects input rows (then the
// residual is left untouched).
// ---------------------------------------------------------------------------------------------
template <typename TD, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const float* __restrict__ weight,
                               float eps, const int* __restrict__ rows, TO* __restrict__ out, int hidden) {
    extern __shared__ float row[];  // hidden floats, then 33 for the reduction
    float* scratch = row + hidden;
    pdl_trigger();
    pdl_wait();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* x = resid + (size_t)r * hidden;
    const TD* d = delta ? delta + (size_t)r * hidden : nullptr;
    float ss = 0.f;
    const bool vec = (hidden & 3) == 0;
    if (vec) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float v[4];
            load4(x + i, v);
            if (d) {
                float dv[4];
                load4(d + i, dv);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] += dv[e];
            }
            store4(row + i, v);
#pragma unroll
            for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = x[i];
            if (d) v += to_float(d[i]);
            row[i] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = rsqrtf(ss / (float)hidden + eps);
    TO* y = out + (size_t)o * hidden;
    const bool write_back = d && !rows;
    if (vec) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float v[4], wv[4];
            load4(row + i, v);
            load4(weight + i, wv);
            if (write_back) store4(x + i, v);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = v[e] * scale * wv[e];
            store4(y + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = row[i];
            if (write_back) x[i] = v;
            y[i] = from_float<TO>(v * scale * weight[i]);
        }
    }
}

// The same for rows whose length is a multiple of 4 and at most 8 float4 a thread: the row stays in registers, and all
// of a thread's loads are asked for before the first is used (the kernel is a chain of trips to L2 otherwise: load, sum,
// weight, store).  Few threads a row, so that many rows are in flight on an SM.
template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(256) rmsnorm_registers_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                                                const float* __restrict__ weight, float eps,
                                                                const int* __restrict__ rows, TO* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    pdl_trigger();
    const int o = blockIdx.x, t4 = threadIdx.x * 4, step = blockDim.x * 4;
    float w[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j)  // the weights do not depend on the kernel in front
        if (t4 + j * step < hidden) load4(weight + t4 + j * step, w[j]);
    pdl_wait();
    const int r = rows ? rows[o] : o;
    float* x = resid + (size_t)r * hidden;
    const TD* d = delta ? delta + (size_t)r * hidden : nullptr;
    float v[NV][4], dv[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (t4 + j * step < hidden) {
            load4(x + t4 + j * step, v[j]);
            if (d) load4(d + t4 + j * step, dv[j]);
        }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (t4 + j * step < hidden) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (d) v[j][e] += dv[j][e];
                ss += v[j][e] * v[j][e];
            }
        }
    ss = block_sum(ss, scratch);
    const float scale = rsqrtf(ss / (float)hidden + eps);
    TO* y = out + (size_t)o * hidden;
    const bool write_back = d && !rows;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (t4 + j * step < hidden) {
            if (write_back) store4(x + t4 + j * step, v[j]);
            float n[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) n[e] = v[j][e] * scale * w[j][e];
            store4(y + t4 + j * step, n);
        }
}

template <typename TD, typename TO>
static int rmsnorm_launch(float* resid, const void* delta, const float* weight, float eps, const int* rows, void* out,
                          int n_out, int hidden, cudaStream_t stream) {
    if ((hidden & 3) == 0 && hidden <= 8192) {  // the row in registers
        const int threads = hidden <= 512 ? 32 : (hidden <= 4096 ? 128 : 256), nv = (hidden / 4 + threads - 1) / threads;
        auto go = [&](auto kernel) {
            return launch_pdl(kernel, dim3(n_out), dim3(threads), 0, stream, resid, (const TD*)delta, weight, eps, rows, (TO*)out, hidden);
        };
        if (nv <= 2) return go(rmsnorm_registers_kernel<TD, TO, 2>);
        if (nv <= 4) return go(rmsnorm_registers_kernel<TD, TO, 4>);
        return go(rmsnorm_registers_kernel<TD, TO, 8>);
    }
    const size_t smem = (size_t)(hidden + 33) * sizeof(float);
    if (smem > 200 * 1024) return LLM_ERR_UNSUPPORTED;
    auto kernel = rmsnorm_kernel<TD, TO>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return launch_pdl(kernel, dim3(n_out), dim3(threads), smem, stream, resid, (const TD*)delta, weight, eps, rows, (TO*)out, hidden);
}

LLM_EXPORT int llm_rmsnorm(float* resid, const void* delta, int delta_dtype, const float* weight, float eps,
                           const int* rows, void* out, int out_dtype, int n_out, int hidden, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (out_dtype == LLM_F32 && (delta == nullptr || delta_dtype == LLM_F32))
        return rmsnorm_launch<float, float>(resid, delta, weight, eps, rows, out, n_out, hidden, stream);
    if (out_dtype == LLM_BF16 && (delta == nullptr || delta_dtype == LLM_BF16))
        return rmsnorm_launch<__nv_bfloat16, __nv_bfloat16>(resid, delta, weight, eps, rows, out, n_out, hidden, stream);
    if (out_dtype == LLM_BF16 && delta_dtype == LLM_F32)
        return rmsnorm_launch<float, __nv_bfloat16>(resid, delta, weight, eps, rows, out, n_out, hidden, stream);
    if (out_dtype == LLM_F32 && delta_dtype == LLM_BF16)
        return rmsnorm_launch<__nv_bfloat16, float>(resid, delta, weight, eps, rows, out, n_out, hidden, stream);
    return LLM_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// rotary encoding of q (in place) and k, and the write of k and v into their pages.
//
// qkv row: [H query heads | KV key heads | KV value heads] x D (the last two only when write_kv).
// table row p: [cos(p * f_0..f_{D/2-1}) | sin(...)], 32-bit; null: no rotation.
// pool plane: [pages, 2, KV, page_size, D]; slot = page * page_size + offset.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                     const float* __restrict__ table, int table_rows, const int* __restrict__ slot_map,
                                     T* __restrict__ pool, int H, int KV, int D, int page_size, int write_kv) {
    pdl_trigger();
    // the token's position and slot are the step's own arrays, written long before: they are read while the kernel in
    // front still runs, so that only one trip to memory (the row itself) is left behind the wait
    const int t = blockIdx.x;
    T* row = qkv + (size_t)t * row_stride;
    const int half = D >> 1;
    int pos = positions[t];
    if (pos < 0) pos = 0;
    if (pos >= table_rows) pos = table_rows - 1;  // guarded on the host; never read out of range
    const float* cs = table ? table + (size_t)pos * D : nullptr;

    size_t k_base = 0, v_base = 0;
    if (write_kv) {
        const int slot = slot_map[t];
        const int page = slot / page_size, off = slot - page * page_size;
        k_base = ((size_t)(page * 2 + 0) * KV) * page_size * D + (size_t)off * D;
        v_base = ((size_t)(page * 2 + 1) * KV) * page_size * D + (size_t)off * D;
    }
    const size_t head_stride = (size_t)page_size * D;
    pdl_wait();

    if ((D & 7) == 0 && (row_stride & 3) == 0) {
        // four pairs (j, j + D/2) at a time
        const int quads = half >> 2;
        for (int i = threadIdx.x; i < (H + (write_kv ? KV : 0)) * quads; i += blockDim.x) {
            const int h = i / quads, j = (i - h * quads) * 4;
            T* x = row + h * D;
            float a[4], b[4], c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f}, lo[4], hi[4];
            load4(x + j, a);
            load4(x + j + half, b);
            if (cs) {
                load4(cs + j, c);
                load4(cs + half + j, sn);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                lo[e] = a[e] * c[e] - b[e] * sn[e];
                hi[e] = b[e] * c[e] + a[e] * sn[e];
            }
            T* dst = h < H ? x : pool + k_base + (h - H) * head_stride;
            store4(dst + j, lo);
            store4(dst + j + half, hi);
        }
        if (write_kv) {
            for (int i = threadIdx.x; i < KV * (D >> 2); i += blockDim.x) {
                const int h = i / (D >> 2), j = (i - h * (D >> 2)) * 4;
                float v[4];
                load4(row + (H + KV + h) * D + j, v);
                store4(pool + v_base + h * head_stride + j, v);
            }
        }
        return;
    }
    // query heads, rotated in place
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        T* x = row + h * D;
        const float a = to_float(x[j]), b = to_float(x[j + half]);
        const float c = cs ? cs[j] : 1.f, s = cs ? cs[half + j] : 0.f;
        x[j] = from_float<T>(a * c - b * s);
        x[j + half] = from_float<T>(b * c + a * s);
    }
    if (!write_kv) return;
    // key heads, rotated into their page
    for (int i = threadIdx.x; i < KV * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        const T* x = row + (H + h) * D;
        const float a = to_float(x[j]), b = to_float(x[j + half]);
        const float c = cs ? cs[j] : 1.f, s = cs ? cs[half + j] : 0.f;
        T* dst = pool + k_base + h * head_stride;
        dst[j] = from_float<T>(a * c - b * s);
        dst[j + half] = from_float<T>(b * c + a * s);
    }
    // value heads, copied
    for (int i = threadIdx.x; i < KV * D; i += blockDim.x) {
        const int h = i / D, j = i - h * D;
        pool[v_base + h * head_stride + j] = row[(H + KV + h) * D + j];
    }
}

LLM_EXPORT int llm_rope_kv_write(void* qkv, int dtype, int row_stride, const int* positions, const float* table,
                                 int table_rows, const int* slot_map, void* pool, int n, int H, int KV, int D,
                                 int page_size, int write_kv, cudaStream_t stream) {
    if (n <= 0) return 0;
    if ((D & 1) || D <= 0 || H <= 0 || KV < 0 || page_size <= 0) return LLM_ERR_BAD_ARGUMENT;
    const int threads = 128;  // (measured on 2,048 tokens x 36 heads of 64: 512 threads a token 11.4 us, 256 8.3, 128 6.6, 64 6.7, 32 8.5)
    if (dtype == LLM_F32)
        return launch_pdl(rope_kv_write_kernel<float>, dim3(n), dim3(threads), 0, stream, (float*)qkv, row_stride, positions,
                          table, table_rows, slot_map, (float*)pool, H, KV, D, page_size, write_kv);
    if (dtype == LLM_BF16)
        return launch_pdl(rope_kv_write_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream, (__nv_bfloat16*)qkv, row_stride,
                          positions, table, table_rows, slot_map, (__nv_bfloat16*)pool, H, KV, D, page_size, write_kv);
    return LLM_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// gated activation: out[t, j] = silu(gate_up[t, j]) * gate_up[t, I + j], in 32-bit
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if ((inter & 3) == 0) {
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += stride * 4) {
            const size_t t = i / inter;
            const int j = (int)(i - t * inter);
            float g[4], u[4];
            load4(gate_up + t * 2 * inter + j, g);
            load4(gate_up + t * 2 * inter + inter + j, u);
#pragma unroll
            for (int e = 0; e < 4; ++e) g[e] = g[e] / (1.f + expf(-g[e])) * u[e];
            store4(out + i, g);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t t = i / inter;
        const int j = (int)(i - t * inter);
        const float g = to_float(gate_up[t * 2 * inter + j]);
        const float u = to_float(gate_up[t * 2 * inter + inter + j]);
        out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

LLM_EXPORT int llm_swiglu(const void* gate_up, void* out, int dtype, int n, int inter, cudaStream_t stream) {
    if (n <= 0) return 0;
    const size_t total = (size_t)n * inter;
    const int threads = 256;
    const size_t want = (total / 4 + threads - 1) / threads + 1;
    const size_t most = 148 * 16;  // sixteen blocks an SM of a B200; the kernel's loop strides over what is left
    const int blocks = (int)(want < most ? want : most);
    if (dtype == LLM_F32)
        return launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inter, total);
    if (dtype == LLM_BF16)
        return launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up,
                          (__nv_bfloat16*)out, inter, total);
    return LLM_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// bias of a projection: x[t, j] += bias[j], summed in 32-bit and rounded once.  The products of layers
// without a bias never come here; a layer with one runs its product, then this.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, int ld, const T* __restrict__ bias, int cols, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t t = i / cols;
        const int j = (int)(i - t * cols);
        T* p = x + t * ld + j;
        *p = from_float<T>(to_float(*p) + to_float(bias[j]));
    }
}

LLM_EXPORT int llm_add_bias(void* x, int dtype, int rows, int cols, int ld, const void* bias, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (ld < cols) return LLM_ERR_BAD_ARGUMENT;
    const size_t total = (size_t)rows * cols;
    const int threads = 256;
    const size_t want = (total + threads - 1) / threads, most = 148 * 16;
    const int blocks = (int)(want < most ? want : most);
    if (dtype == LLM_F32)
        return launch_pdl(add_bias_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)x, ld, (const float*)bias, cols, total);
    if (dtype == LLM_BF16)
        return launch_pdl(add_bias_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)x, ld,
                          (const __nv_bfloat16*)bias, cols, total);
    return LLM_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// A step's integer arrays from pinned host memory to the device, read by the kernel itself: for a
// few kilobytes one round trip over the bus is shorter than a copy by the copy engine, which the
// stream has to hand over to and take back from.  `words` 32-bit words; the first `head_words`
// come from `head` on the device instead where it is given (token ids that the step before chose
// and the host has not seen yet).
// ---------------------------------------------------------------------------------------------
__global__ void fetch_words_kernel(const int* __restrict__ host, int* __restrict__ dev, const int* __restrict__ head,
                                   int head_words, int words) {
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const bool from_head = head != nullptr && i < head_words;
    // the host's memory does not change while the kernel runs, but no cached copy of it may outlive the kernel
    const int v = i < words && !from_head ? __ldcv(host + i) : 0;
    pdl_wait();  // the kernels before may still read the arrays of their step, and one of them writes `head`
    if (i < words) dev[i] = from_head ? head[i] : v;
}

LLM_EXPORT int llm_fetch_words(const int* host, int* dev, const int* head, int head_words, int words, cudaStream_t stream) {
    if (words <= 0) return 0;
    if (head_words < 0 || head_words > words) return LLM_ERR_BAD_ARGUMENT;
    const int threads = 256;
    return launch_pdl(fetch_words_kernel, dim3((words + threads - 1) / threads), dim3(threads), 0, stream, host, dev, head, head_words, words);
}
