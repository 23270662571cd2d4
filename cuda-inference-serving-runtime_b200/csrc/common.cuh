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

// Programmatic dependent launch.  A kernel launched with the attribute may start while the kernel before it
// in the stream is still running; it must call pdl_wait() before it touches anything an earlier kernel wrote,
// and may do work that depends on nothing earlier (fetching weights) before that.  pdl_trigger() lets the
// kernel after this one start.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Whether launches carry the attribute: switched by the host (cisr_set_pdl in each library).
template <typename... KernelArgs, typename... Args>
static inline int launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                bool pdl, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
    return e == cudaSuccess ? (int)cudaGetLastError() : (int)e;
}
