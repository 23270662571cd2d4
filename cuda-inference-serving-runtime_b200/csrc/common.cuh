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

// dtype codes shared with the Python side (ops/kernels.py: F32, BF16)
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

// ---------------------------------------------------------------- kernel timeline (development builds)
// Compiled with -DCISR_TRACE=1 every kernel of a library records, per CTA, when its thread 0 entered, when its wait on
// the kernel before returned, up to four marks in between, when it left, and on which SM; the host reads the records back (cisr_trace_read) and
// lines the libraries' records up by the global timer.  Without the flag the macros are empty.
enum : int {
    TRACE_EMBEDDING = 1, TRACE_ADD_RMSNORM, TRACE_SWIGLU, TRACE_ROTARY_TABLE, TRACE_ROPE_STORE, TRACE_PAGE_COPY, TRACE_TABLE_UPDATE,
    TRACE_ATTN_PREFILL, TRACE_ATTN_DECODE_GATHER, TRACE_ATTN_DECODE_TMA, TRACE_ATTN_MERGE, TRACE_SAMPLE, TRACE_DECODE_ADVANCE,
    TRACE_SKINNY_PLAIN, TRACE_SKINNY_SWIGLU, TRACE_SKINNY_ROPE, TRACE_GEMM_TCGEN05, TRACE_ATTN_SIMT, TRACE_STREAM_GEMM,
    TRACE_MERGE_PROJ
};
#ifdef CISR_TRACE
struct TraceRecord { unsigned long long entered, waited, left, marks[4]; int kernel, block, sm, pad; };
constexpr unsigned TRACE_CAPACITY = 1u << 17;
__device__ TraceRecord g_trace_records[TRACE_CAPACITY];
__device__ unsigned g_trace_count;
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
struct TraceScope {
    unsigned long long entered, waited, marks[4];
    int kernel;
    __device__ __forceinline__ explicit TraceScope(int k) : entered(trace_now()), waited(0), marks{0, 0, 0, 0}, kernel(k) {}
    __device__ __forceinline__ void mark_waited() { waited = trace_now(); }
    __device__ __forceinline__ void mark(int i) { marks[i] = trace_now(); }
    __device__ __forceinline__ ~TraceScope() {
        if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
            const unsigned long long left = trace_now();     // before the counter's round trip to memory
            const unsigned i = atomicAdd(&g_trace_count, 1u);
            if (i < TRACE_CAPACITY) {
                unsigned sm;
                asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
                TraceRecord r;
                r.entered = entered; r.waited = waited; r.left = left; r.kernel = kernel;
                r.marks[0] = marks[0]; r.marks[1] = marks[1]; r.marks[2] = marks[2]; r.marks[3] = marks[3];
                r.block = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)); r.sm = (int)sm; r.pad = 0;
                g_trace_records[i] = r;
            }
        }
    }
};
#define CISR_TRACE_SCOPE(kernel_id) TraceScope cisr_trace_scope(kernel_id)
#define CISR_TRACE_WAITED() cisr_trace_scope.mark_waited()
#define CISR_TRACE_MARK(i) cisr_trace_scope.mark(i)
// Copies up to max_records records to `host` (72 bytes each), returns how many there were, and empties the buffer.
CISR_EXPORT int cisr_trace_read(void* host, int max_records) {
    unsigned count = 0;
    if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpyFromSymbol(&count, g_trace_count, sizeof(count)) != cudaSuccess) return -1;
    if (count > TRACE_CAPACITY) count = TRACE_CAPACITY;
    const unsigned n = count < (unsigned)max_records ? count : (unsigned)max_records;
    if (n && cudaMemcpyFromSymbol(host, g_trace_records, sizeof(TraceRecord) * (size_t)n) != cudaSuccess) return -1;
    const unsigned zero = 0;
    if (cudaMemcpyToSymbol(g_trace_count, &zero, sizeof(zero)) != cudaSuccess) return -1;
    return (int)n;
}
#else
#define CISR_TRACE_SCOPE(kernel_id)
#define CISR_TRACE_WAITED()
#define CISR_TRACE_MARK(i)
#endif

// Whether launches carry the attribute: switched by the host (cisr_set_pdl in each library).
// cluster_z > 1 launches thread-block clusters of that many CTAs along z (gridDim.z must be a multiple of it).
template <typename... KernelArgs, typename... Args>
static inline int launch_kernel_cluster(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        bool pdl, int cluster_z, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    config.attrs = attr;
    config.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
    return e == cudaSuccess ? (int)cudaGetLastError() : (int)e;
}
template <typename... KernelArgs, typename... Args>
static inline int launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                bool pdl, Args... args) {
    return launch_kernel_cluster(kernel, grid, block, smem, stream, pdl, 1, args...);
}
