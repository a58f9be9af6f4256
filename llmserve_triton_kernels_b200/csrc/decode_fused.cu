// A whole decode step of a stack of pre-norm layers (RMS norm, rotary grouped-query attention over
// the paged cache, RMS norm, gated feed-forward) in ONE kernel, for up to 8 tokens.
//
// A decode step of a small batch is a chain of short, memory-bound operations; run as one kernel
// each, every link pays a launch, a ramp-up of its loads and a tail.  Here one CTA per SM stays
// resident for the whole step (a cooperative launch, so that all CTAs are resident together) and
// walks the phases of every layer, meeting the other CTAs at a grid-wide barrier between phases:
//
//   embedding + first norm | per layer: [stacked projection + rotary + cache write] | [attention] |
//   [output projection + residual + norm] | [gate/up + SwiGLU] | [down + residual + norm] | output matrix
//
// The phases are the device functions of the separate kernels (linear_stream.cuh, attention_tile.cuh),
// so both ways compute the same thing.  Every wait (mbarrier, grid barrier) is bounded; if one gives
// up, the CTA sets *error_flag and leaves (the others then give up at their next barrier).
#include "attention_tile.cuh"
#include "grid_sync.cuh"
#include "linear_stream.cuh"

namespace {

using namespace lin;

struct alignas(64) FusedLayer {
    CUtensorMap w_in, w_out, w_gate_up, w_down;  // boxes of 8, 16, 8 and 16 rows x 128 k
    const float* ff_norm_w;                      // the norm between attention and feed-forward
    const float* next_norm_w;                    // the norm that meets the stream after this layer
    float ff_eps, next_eps;
    __nv_bfloat16* pool;                         // this layer's plane [pages, 2, KV, page_size, D]
    const int* page_table;
    const int* slot_map;
    int table_width, window;
    float scale_log2;
    int group_in, group_out, group_gate_up, group_down;
};

struct FusedParams {
    int M, hidden, H, KV, D, inter, vocab, page_size, n_layers;
    const int* token_ids;
    const __nv_bfloat16* embedding;
    const float* first_norm_w;
    float first_eps;
    const int* positions;
    const float* rotary;
    int rotary_rows;
    const int* cu_tokens;
    const int* ctx_lens;
    float* resid;          // [M, hidden]
    __nv_bfloat16* xw;     // [M, hidden]
    float* ss;             // [ceil(hidden / 16), M]
    __nv_bfloat16* q;      // [M, H D]
    __nv_bfloat16* attn;   // [M, H D]
    __nv_bfloat16* act;    // [M, inter]
    int attn_splits;
    float* part_o;
    float* part_ml;
    int* counters;
    const FusedLayer* layers;
    int group_head;
    float* logits;         // [M, vocab]
    unsigned* barrier;
    int* error_flag;
    unsigned long long* timeline;  // [CTAs, timeline_len, 2] (global timer, SM clock) at each barrier's two sides, or null
    int timeline_len;
};

// The teams' partial sums have room for two tiles of a team (2 x WARPS x 4 x 32 floats): the host's choice of warps
// per tile keeps to that.
struct Smem {
    __nv_bfloat16* ring;
    float* red;
    __nv_bfloat16* x_s;
    float* row_scale;
    unsigned long long (*full)[SLOTS];
};

// A product in three steps.  phase_plan: its split of the work and what the end of its first tile needs besides the
// product (nothing that depends on the product's input).  Its boxes of weights are asked for as the product before
// it frees the ring's slots (weights depend on nothing), and by phase_arm once that product is done.  phase_run: the
// rest, once the input is there (after the grid barrier).
template <int MODE>
__device__ __forceinline__ void phase_plan(StreamState& st, const LinearParams& lp, unsigned base) {
    stream_plan<MODE, 1>(st, lp, base);
}

__device__ __forceinline__ void phase_arm(StreamState& st, const CUtensorMap* map, const Smem& sm) {
    const int warp = threadIdx.x >> 5;
    stream_arm(st, map, sm.ring + (size_t)warp * SLOTS * SLOT_ELEMS, sm.full[warp], 0);
}

template <int MODE, typename TO, typename Stamp>
__device__ __forceinline__ bool phase_run(StreamState& st, const LinearParams& lp, const CUtensorMap* map, const Smem& sm, unsigned& base,
                                          Stamp& stamp, StreamState* next, const CUtensorMap* next_map) {
    const int warp = threadIdx.x >> 5;
    stream_stage_x<1>(lp, sm.x_s, sm.row_scale);
    __syncthreads();
    stamp();
    const bool ok = stream_run<1, MODE, TO>(st, lp, map, sm.ring + (size_t)warp * SLOTS * SLOT_ELEMS, sm.full[warp], sm.red, sm.x_s,
                                            sm.row_scale, next, next_map);
    base += (unsigned)st.units;
    if (next) phase_arm(*next, next_map, sm);  // the ring is this product's no more
    return ok;
}

template <int D>
__global__ void __launch_bounds__(THREADS) decode_fused_kernel(const FusedParams p, const __grid_constant__ CUtensorMap head_map) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float row_scale[8];
    __shared__ __align__(8) unsigned long long full[WARPS][SLOTS];
    __shared__ float reduce_scratch[33];
    Smem sm;
    sm.ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    sm.red = reinterpret_cast<float*>(smem_raw + (size_t)WARPS * SLOTS * SLOT_ELEMS * 2);
    sm.x_s = reinterpret_cast<__nv_bfloat16*>(sm.red + 2 * WARPS * 4 * 32);
    sm.row_scale = row_scale;
    sm.full = full;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (lane == 0) {
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl) tma::mbar_init(&full[warp][sl], 1);
        tma::mbar_fence_init();
    }
    __syncthreads();
    unsigned base = 0, arrivals = 0;
    const int M = p.M, hidden = p.hidden;
    bool ok = true;
    int stamps = 0;
    auto stamp = [&]() {
        if (p.timeline && tid == 0 && stamps < p.timeline_len) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
            p.timeline[((size_t)blockIdx.x * p.timeline_len + stamps) * 2] = t;
            p.timeline[((size_t)blockIdx.x * p.timeline_len + stamps++) * 2 + 1] = (unsigned long long)clock64();
        }
    };
#define FUSED_BARRIER()                                                \
    do {                                                               \
        stamp();                                                       \
        if (!ok || !grid_sync::barrier(p.barrier, arrivals)) {         \
            if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 1); \
            return;                                                    \
        }                                                              \
        stamp();                                                       \
    } while (0)

    // ---- embedding, and the stream in factored normalised form for the first norm (one part per row) ----
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        int id = p.token_ids[m];
        if (id < 0 || id >= p.vocab) id = 0;
        const __nv_bfloat16* src = p.embedding + (size_t)id * hidden;
        float sq = 0.f;
        for (int i = tid; i < hidden; i += THREADS) {
            const float v = __bfloat162float(src[i]);
            p.resid[(size_t)m * hidden + i] = v;
            p.xw[(size_t)m * hidden + i] = __float2bfloat16_rn(v * p.first_norm_w[i]);
            sq += v * v;
        }
        sq = block_sum(sq, reduce_scratch);
        if (tid == 0) p.ss[m] = sq;
    }
    const int hidden_parts = (hidden + 15) / 16;
    // With head size 64 the attention's ring of keys and values fits beside the weights' ring, so the output
    // projection's first weights can be on their way while attention runs; with 128 it takes the weights' place.
    constexpr bool ATTN_BESIDE = D == 64;
    constexpr int ATTN_STAGES = ATTN_BESIDE ? 3 : attn::stages_of(D, 4);
    unsigned char* attn_smem = ATTN_BESIDE ? reinterpret_cast<unsigned char*>(sm.red) : smem_raw;

    LinearParams qkv = {}, out = {}, gate_up = {}, down = {}, head = {};
    StreamState st_a, st_b;  // the product that runs and the one that follows it, by turns
    auto set_qkv = [&](int l, int in_parts, float in_eps) {
        const FusedLayer& L = p.layers[l];
        qkv.M = M; qkv.error_flag = p.error_flag;
        qkv.x = p.xw; qkv.ldx = hidden; qkv.K = hidden; qkv.N = (p.H + 2 * p.KV) * p.D;
        qkv.in_ss = p.ss; qkv.in_parts = in_parts; qkv.in_eps = in_eps;
        qkv.out = p.q; qkv.ldo = p.H * p.D; qkv.group = L.group_in;
        qkv.positions = p.positions; qkv.rotary = p.rotary; qkv.rotary_rows = p.rotary_rows;
        qkv.slot_map = L.slot_map; qkv.pool = L.pool; qkv.H = p.H; qkv.KV = p.KV; qkv.D = p.D; qkv.page_size = p.page_size;
    };
    set_qkv(0, 1, p.first_eps);
    phase_plan<MODE_QKV>(st_a, qkv, base);
    phase_arm(st_a, &p.layers[0].w_in, sm);
    FUSED_BARRIER();

    for (int l = 0; l < p.n_layers; ++l) {
        const FusedLayer& L = p.layers[l];
        const bool last = l + 1 == p.n_layers;
        // ---- stacked projection, rotary encoding, cache write (st_a); the output projection follows (st_b) ----
        out.M = M; out.error_flag = p.error_flag;
        out.x = p.attn; out.ldx = p.H * p.D; out.K = p.H * p.D; out.N = hidden; out.group = L.group_out;
        out.resid = p.resid; out.norm_w = L.ff_norm_w; out.xw_out = p.xw; out.ss_out = p.ss; out.resid_early = 1;
        phase_plan<MODE_RESIDUAL>(st_b, out, base + (unsigned)st_a.units);
        ok = phase_run<MODE_QKV, __nv_bfloat16>(st_a, qkv, &L.w_in, sm, base, stamp, ATTN_BESIDE ? &st_b : nullptr, &L.w_out);
        FUSED_BARRIER();

        // ---- attention: items are (request, key/value head, split of the keys) ----
        {
            attn::AttnParams ap;
            ap.q = p.q;
            ap.q_stride = p.H * p.D;
            ap.out = p.attn;
            ap.out_stride = p.H * p.D;
            ap.pool = L.pool;
            ap.page_table = L.page_table;
            ap.table_width = L.table_width;
            ap.cu_tokens = p.cu_tokens;
            ap.ctx_lens = p.ctx_lens;
            ap.H = p.H;
            ap.KV = p.KV;
            ap.G = p.H / p.KV;
            ap.page_size = p.page_size;
            ap.window = L.window;
            ap.tiles_per_request = 1;
            ap.scale_log2 = L.scale_log2;
            ap.splits = p.attn_splits;
            ap.part_o = p.part_o;
            ap.part_ml = p.part_ml;
            ap.counters = p.counters;
            ap.skip_tokens_from = 0;
            const int items = M * p.KV * p.attn_splits;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int split = item % p.attn_splits, rest = item / p.attn_splits;
                // the attention tile is written for four warps: the first four compute it
                if (warp < 4) attn::attention_tile<D, 1, 4, 32, ATTN_STAGES>(ap, split, rest % p.KV, rest / p.KV, 0, attn_smem, false);
                __syncthreads();  // shared memory is free again
            }
        }
        if (!ATTN_BESIDE) phase_arm(st_b, &L.w_out, sm);
        FUSED_BARRIER();

        // ---- output projection into the residual stream (st_b); gate and up follow (st_a) ----
        gate_up.M = M; gate_up.error_flag = p.error_flag;
        gate_up.x = p.xw; gate_up.ldx = hidden; gate_up.K = hidden; gate_up.N = p.inter;
        gate_up.in_ss = p.ss; gate_up.in_parts = hidden_parts; gate_up.in_eps = L.ff_eps;
        gate_up.out = p.act; gate_up.ldo = p.inter; gate_up.up_offset = p.inter; gate_up.group = L.group_gate_up;
        phase_plan<MODE_SWIGLU>(st_a, gate_up, base + (unsigned)st_b.units);
        ok = phase_run<MODE_RESIDUAL, __nv_bfloat16>(st_b, out, &L.w_out, sm, base, stamp, &st_a, &L.w_gate_up);
        FUSED_BARRIER();

        // ---- gate and up with the activation (st_a); down follows (st_b) ----
        down.M = M; down.error_flag = p.error_flag;
        down.x = p.act; down.ldx = p.inter; down.K = p.inter; down.N = hidden; down.group = L.group_down;
        down.resid = p.resid; down.norm_w = L.next_norm_w; down.xw_out = p.xw; down.ss_out = p.ss; down.resid_early = 1;
        phase_plan<MODE_RESIDUAL>(st_b, down, base + (unsigned)st_a.units);
        ok = phase_run<MODE_SWIGLU, __nv_bfloat16>(st_a, gate_up, &L.w_gate_up, sm, base, stamp, &st_b, &L.w_down);
        FUSED_BARRIER();

        // ---- down into the residual stream (st_b); the next layer's stacked projection or the output matrix follows ----
        const CUtensorMap* after;
        if (!last) {
            set_qkv(l + 1, hidden_parts, L.next_eps);
            phase_plan<MODE_QKV>(st_a, qkv, base + (unsigned)st_b.units);
            after = &p.layers[l + 1].w_in;
        } else {
            head.M = M; head.error_flag = p.error_flag;
            head.x = p.xw; head.ldx = hidden; head.K = hidden; head.N = p.vocab;
            head.in_ss = p.ss; head.in_parts = hidden_parts; head.in_eps = L.next_eps;
            head.out = p.logits; head.ldo = p.vocab; head.group = p.group_head;
            phase_plan<MODE_PLAIN>(st_a, head, base + (unsigned)st_b.units);
            after = &head_map;
        }
        ok = phase_run<MODE_RESIDUAL, __nv_bfloat16>(st_b, down, &L.w_down, sm, base, stamp, &st_a, after);
        FUSED_BARRIER();
    }

    // ---- output matrix ----
    ok = phase_run<MODE_PLAIN, float>(st_a, head, &head_map, sm, base, stamp, nullptr, nullptr);
    stamp();
    if (!ok && tid == 0 && p.error_flag) atomicExch(p.error_flag, 1);
#undef FUSED_BARRIER
}

unsigned long long* g_timeline = nullptr;  // see llm_decode_fused_timeline
int g_timeline_len = 0;

int sm_count() {
    static int count = 0;
    if (count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0) count = 148;
    }
    return count;
}

int kblocks_of(int K) { return (K + BOXK - 1) / BOXK; }

size_t smem_bytes(int k_max, int D) {
    const size_t linear = (size_t)WARPS * SLOTS * SLOT_ELEMS * 2 + (size_t)2 * WARPS * 4 * 32 * sizeof(float) + (size_t)8 * (k_max + X_PAD) * 2;
    const size_t ring = (size_t)WARPS * SLOTS * SLOT_ELEMS * 2;
    // head size 64: attention's three tiles of keys and values lie behind the weights' ring; 128: in its place
    const size_t attention = D == 64 ? ring + (size_t)3 * 2 * 128 * D * 2 : (size_t)attn::stages_of(D, 4) * 2 * 128 * D * 2;
    return linear > attention ? linear : attention;
}

}  // namespace

LLM_EXPORT int llm_fused_layer_bytes() { return (int)sizeof(FusedLayer); }

// Fills one layer's record (host memory, 64-byte aligned, llm_fused_layer_bytes() long) for a model of the given sizes.
LLM_EXPORT int llm_fused_layer_fill(void* dst, const void* w_in, const void* w_out, const void* w_gate_up, const void* w_down,
                                    int hidden, int H, int KV, int D, int inter, const float* ff_norm_w, float ff_eps,
                                    const float* next_norm_w, float next_eps, void* pool, const int* page_table, int table_width,
                                    const int* slot_map, int window, float scale) {
    if (((uintptr_t)dst & 63) || (hidden & 7) || (inter & 7) || (D & 15)) return LLM_ERR_UNSUPPORTED;
    FusedLayer L = {};
    const int qkv_rows = (H + 2 * KV) * D, grid = sm_count();
    if (!tma::make_map_2d_bf16(&L.w_in, w_in, qkv_rows, hidden, hidden, 8, BOXK, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !tma::make_map_2d_bf16(&L.w_out, w_out, hidden, H * D, H * D, 16, BOXK, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !tma::make_map_2d_bf16(&L.w_gate_up, w_gate_up, 2 * inter, hidden, hidden, 8, BOXK, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !tma::make_map_2d_bf16(&L.w_down, w_down, hidden, inter, inter, 16, BOXK, CU_TENSOR_MAP_SWIZZLE_NONE))
        return LLM_ERR_UNSUPPORTED;
    L.ff_norm_w = ff_norm_w;
    L.ff_eps = ff_eps;
    L.next_norm_w = next_norm_w;
    L.next_eps = next_eps;
    L.pool = (__nv_bfloat16*)pool;
    L.page_table = page_table;
    L.table_width = table_width;
    L.slot_map = slot_map;
    L.window = window;
    L.scale_log2 = scale * 1.4426950408889634f;
    L.group_in = choose_group(qkv_rows / 16, kblocks_of(hidden), grid, 2);
    L.group_out = choose_group((hidden + 15) / 16, kblocks_of(H * D), grid, 2);
    L.group_gate_up = choose_group((inter + 7) / 8, kblocks_of(hidden), grid, 2);
    L.group_down = choose_group((hidden + 15) / 16, kblocks_of(inter), grid, 2);
    memcpy(dst, &L, sizeof L);
    return 0;
}

// For profiling: later launches of llm_decode_fused record, per CTA, the device's global timer when the CTA arrives
// at and when it leaves each grid-wide barrier (and once at its end), with the SM's cycle counter beside it, into
// buffer [CTAs, len, 2] (device memory, the
// caller zeroes it); null switches it off.  A graph keeps the setting it was captured with.
LLM_EXPORT int llm_decode_fused_timeline(unsigned long long* buffer, int len) {
    g_timeline = len > 0 ? buffer : nullptr;
    g_timeline_len = buffer ? len : 0;
    return 0;
}

// One decode step of M <= 8 tokens (one per request) through n_layers layers and the output matrix.
// layers: device copy of the records filled above.  resid, xw, ss, q, attn, act, part_o, part_ml, counters
// (zeroed), barrier: device scratch of the sizes named in FusedParams.  Returns LLM_ERR_UNSUPPORTED for sizes
// the kernel does not take (the caller then runs the step kernel by kernel).
LLM_EXPORT int llm_decode_fused(int M, int hidden, int H, int KV, int D, int inter, int vocab, int page_size, int n_layers,
                                const int* token_ids, const void* embedding, const float* first_norm_w, float first_eps,
                                const int* positions, const float* rotary, int rotary_rows, const int* cu_tokens,
                                const int* ctx_lens, float* resid, void* xw, float* ss, void* q, void* attn_out, void* act,
                                int attn_splits, float* part_o, float* part_ml, int* counters, const void* layers,
                                const void* head, float* logits, unsigned* barrier, int* error_flag, cudaStream_t stream) {
    if (M < 1 || M > 8 || n_layers < 1 || (D != 64 && D != 128) || (hidden & 7) || (inter & 7) || H % KV || attn_splits < 1 ||
        attn_splits > 32 || H / KV > 16)
        return LLM_ERR_UNSUPPORTED;
    int dev = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop) return LLM_ERR_UNSUPPORTED;
    const int k_max = hidden > inter ? (hidden > H * D ? hidden : H * D) : (inter > H * D ? inter : H * D);
    const size_t smem = smem_bytes(k_max, D);
    if (smem > 227 * 1024) return LLM_ERR_UNSUPPORTED;
    CUtensorMap head_map;
    if (!tma::make_map_2d_bf16(&head_map, head, vocab, hidden, hidden, 16, BOXK, CU_TENSOR_MAP_SWIZZLE_NONE)) return LLM_ERR_UNSUPPORTED;
    FusedParams p = {};
    p.M = M; p.hidden = hidden; p.H = H; p.KV = KV; p.D = D; p.inter = inter; p.vocab = vocab; p.page_size = page_size;
    p.n_layers = n_layers;
    p.token_ids = token_ids;
    p.embedding = (const __nv_bfloat16*)embedding;
    p.first_norm_w = first_norm_w;
    p.first_eps = first_eps;
    p.positions = positions;
    p.rotary = rotary;
    p.rotary_rows = rotary_rows;
    p.cu_tokens = cu_tokens;
    p.ctx_lens = ctx_lens;
    p.resid = resid;
    p.xw = (__nv_bfloat16*)xw;
    p.ss = ss;
    p.q = (__nv_bfloat16*)q;
    p.attn = (__nv_bfloat16*)attn_out;
    p.act = (__nv_bfloat16*)act;
    p.attn_splits = attn_splits;
    p.part_o = part_o;
    p.part_ml = part_ml;
    p.counters = counters;
    p.layers = (const FusedLayer*)layers;
    p.group_head = choose_group((vocab + 15) / 16, kblocks_of(hidden), sm_count(), 2);
    p.logits = logits;
    p.barrier = barrier;
    p.error_flag = error_flag;
    p.timeline = g_timeline;
    p.timeline_len = g_timeline_len;
    cudaError_t e = cudaMemsetAsync(barrier, 0, sizeof(unsigned), stream);
    if (e != cudaSuccess) return (int)e;
    void* kernel = D == 64 ? (void*)decode_fused_kernel<64> : (void*)decode_fused_kernel<128>;
    static size_t configured[2] = {0, 0};
    size_t& conf = configured[D == 64 ? 0 : 1];
    if (smem > conf) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        conf = smem;
    }
    void* args[] = {(void*)&p, (void*)&head_map};
    return (int)cudaLaunchCooperativeKernel(kernel, dim3(sm_count()), dim3(THREADS), args, smem, stream);
}
