// The TMA unit from plain CUDA: tensor maps made on the host through the driver's entry point
// (no link against libcuda), tiled bulk copies into shared memory, and the mbarriers that count
// their bytes.  Every wait is bounded: a wait that gives up returns false, and the caller sets
// an error flag and runs to its end instead of hanging the GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

namespace tma {

// ---- host -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A map over a row-major 16-bit matrix [rows, cols] (row stride ld elements, a multiple of 8) with boxes of
// [box_rows, box_cols]; what lies outside the matrix reads as zero.  Returns false if the driver refuses.
inline bool make_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                             uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};  // bytes between rows
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A map over a row-major 16-bit matrix [rows, cols], cols a multiple of 64, seen as [cols / 64][rows][64]: a box is
// `box_rows` rows of two consecutive 64-element pieces, laid down in shared memory as [2][box_rows][64] with the
// 128-byte swizzle (the 16-byte chunk c of row r lies at chunk c ^ (r & 7)).  Coordinates: (0, row, piece).
inline bool make_map_row_pieces_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                                     uint64_t ld = 0) {  // ld: elements from row to row (0: cols)
    EncodeTiledFn fn = encode_fn();
    if (!fn || cols % 64) return false;
    const cuuint64_t dims[3] = {64, rows, cols / 64};
    const cuuint64_t strides[2] = {(ld ? ld : cols) * 2, 128};  // bytes between rows, between pieces
    const cuuint32_t box[3] = {64, box_rows, 2};
    const cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Maps are cached by (address, shape, box): weights and cache pools live for the life of the model, and
// activations of a shape come back to the same addresses from a caching allocator.  Null if the driver refuses.
inline const CUtensorMap* cached_map_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                                             uint32_t box_cols, CUtensorMapSwizzle swizzle) {
    struct Key {
        const void* p;
        uint64_t rows, cols, ld;
        uint32_t box_rows, box_cols;
        int swizzle;
        bool operator==(const Key& o) const {
            return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && box_cols == o.box_cols &&
                   swizzle == o.swizzle;
        }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return std::hash<const void*>()(k.p) ^ (size_t)(k.rows * 0x9E3779B97F4A7C15ull) ^ (size_t)(k.cols << 8) ^ (size_t)(k.ld << 40) ^
                   (size_t)(k.box_rows << 3) ^ (size_t)k.box_cols ^ ((size_t)k.swizzle << 60);
        }
    };
    static std::unordered_map<Key, CUtensorMap, Hash> maps;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    const Key key{base, rows, cols, ld, box_rows, box_cols, (int)swizzle};
    auto it = maps.find(key);
    if (it != maps.end()) return &it->second;
    if (maps.size() > 4096) maps.clear();
    CUtensorMap map;
    if (!make_map_2d_bf16(&map, base, rows, cols, ld, box_rows, box_cols, swizzle)) return nullptr;
    return &maps.emplace(key, map).first->second;
}

// ---- device -----------------------------------------------------------------------------------
constexpr int WAIT_LIMIT = 1 << 22;  // tries before a wait gives up

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Waits for the phase of the given parity; false if it gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    for (int i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// One box of the map into shared memory (128-byte aligned); x counts elements along a row and must be a
// multiple of 8 for 16-bit elements, y counts rows.  The box's full size in bytes is counted on `bar`.
__device__ __forceinline__ void load_2d(void* smem, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(smem_addr(smem)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void load_3d(void* smem, const CUtensorMap* map, int x, int y, int z, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
                 ::"r"(smem_addr(smem)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

}  // namespace tma
