// Tensor-map (TMA) copies and the mbarriers they complete on, shared by the kernels that stage tiles with
// cp.async.bulk.tensor: device-side wrappers, and the host-side encoder with a cache of tensor maps.
//
// Every wait on an mbarrier is bounded: mbar_wait() returns false after MAX_POLLS polls and the caller then
// records the failure and leaves, so a lost copy can never hang the device.
//
// A tiled copy must start on a 16-byte boundary in its innermost coordinate (a multiple of 8 bfloat16); the
// callers only ever pass 0 or multiples of 64 there.  Outer coordinates are free, and rows beyond the tensor
// are zero-filled while still counting toward the barrier's byte count.
#pragma once
#include <cuda.h>

#include <unordered_map>

#include "common.cuh"

namespace {
constexpr unsigned MAX_POLLS = 1u << 20;   // a tile lands within microseconds; this is seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One look at the barrier: true when the phase with the given parity has completed.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Polls until the barrier's phase with the given parity has completed; false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (unsigned i = 0; i < MAX_POLLS; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// Box of the map at (c0 = innermost coordinate, c1 = row) into shared memory; its bytes complete on `bar`.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}

// The same for tensors seen with three to five dimensions (c0 innermost); the box lands as [c4][c3][c2][c1][c0].
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled g_encode = nullptr;

// Looks the driver's encoder up once (the library is not linked against the driver).
int tma_load_encoder() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query);
    if (e != cudaSuccess || query != cudaDriverEntryPointSuccess || !fn) return -15;
    g_encode = (EncodeTiled)fn;
    return 0;
}

// A row-major bfloat16 matrix [rows, cols] read in boxes of box_rows x box_cols (box_cols * 2 bytes <= 128) with
// the 128-byte swizzle: 16-byte chunk c of box row r lands at chunk c ^ (r % 8) of its 128-byte shared-memory row.
int make_map(CUtensorMap* map, const void* base, long long rows, int cols, int box_rows, int box_cols) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(__nv_bfloat16)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -20 - (int)r;
}

// A bfloat16 tensor of `rank` dimensions (2 to 5): dims and box in elements, innermost first; strides in bytes for
// dimensions 1 .. rank - 1 (multiples of 16; they need not grow with the dimension: a row-major matrix whose rows are
// cut into 64-column groups is [64][rows][groups] with strides {row, 128 bytes}).  128-byte swizzle, so box[0] * 2
// bytes <= 128.
int make_map_nd(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box) {
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -20 - (int)r;
}

struct MapKey {
    const void* base; long long rows; int cols, box_rows, box_cols;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 7919u) ^
               ((size_t)k.box_rows << 8) ^ (size_t)k.box_cols;
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;     // a map describes geometry only, so it stays right while the address does
size_t g_map_cache_limit = 4096;                                // entries kept before the cache is emptied

// The tensor map for (base, shape, box), encoded once and then found again.  The map is COPIED into the caller's
// storage: a launcher asks for several maps in a row, and a later call may empty the cache, so nothing may keep a
// pointer into it.
int cached_map(CUtensorMap* out, const void* base, long long rows, int cols, int box_rows, int box_cols = 64) {
    const MapKey key{base, rows, cols, box_rows, box_cols};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        if (g_maps.size() >= g_map_cache_limit) g_maps.clear();
        CUtensorMap map;
        const int status = make_map(&map, base, rows, cols, box_rows, box_cols);
        if (status) return status;
        it = g_maps.emplace(key, map).first;
    }
    *out = it->second;
    return 0;
}
}  // namespace
