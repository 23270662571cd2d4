// Shared helpers of the engine's CUDA sources (sm_100a).
//
// Storage types: float (the true 32-bit path) and __nv_bfloat16 (serving path).
// Arithmetic inside every kernel is float; storage is widened on load and rounded
// once, to nearest even, on store.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CISR_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side (ops/library.py)
enum : int { CISR_F32 = 0, CISR_BF16 = 1 };

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a whole block in a fixed order (warp shuffles, then warp 0 over the
// per-warp sums), so a row's result does not depend on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

static inline int launch_status() { return (int)cudaGetLastError(); }
