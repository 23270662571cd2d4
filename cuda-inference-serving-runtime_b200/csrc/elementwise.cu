// Bandwidth-bound kernels of the model step: embedding gather, residual add fused
// with RMSNorm, SwiGLU, rotary tables, and rotary rotation fused with the write of
// keys and values into cache pages.
//
// Parity (formulas): kernels/execution.cu:2-5 (embedding), kernels/ops.cu:3-19 and
// kernels/execution.cu:12-24 (norm, residual+norm), kernels/execution.cu:7-10
// (SwiGLU), kernels/ops.cu:21-33 and kernels/execution.cu:28-40 (rotation, scatter)
// of nehanmohammed19/cuda-inference-serving-runtime.  The residual stream and every
// reduction stay in float here whatever the storage type.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_elementwise_set_pdl(int on) { g_pdl = on != 0; }

// ---------------------------------------------------------------- embedding
template <typename TT>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab) {
    CISR_TRACE_SCOPE(TRACE_EMBEDDING);
    // Under programmatic dependent launch the kernels after this one may start (and fetch their weights) while it runs.
    // It waits for the kernel before it although it reads nothing of it: a later kernel's wait on this one then also
    // covers everything before (the block table update at the head of a step).
    pdl_trigger();
    pdl_wait();
    CISR_TRACE_WAITED();
    const int row = blockIdx.x;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // host validates; clamp keeps a bad id from reading outside
    const TT* src = table + (size_t)id * hidden;
    float* dst = out + (size_t)row * hidden;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) dst[d] = to_float(src[d]);
}

CISR_EXPORT int cisr_embedding(const void* table, int table_dtype, const int* ids, float* out, int tokens,
                               int hidden, int vocab, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == CISR_BF16)
        return launch_kernel(embedding_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, s, g_pdl, (const __nv_bfloat16*)table, ids, out, hidden, vocab);
    return launch_kernel(embedding_kernel<float>, dim3(tokens), dim3(128), 0, s, g_pdl, (const float*)table, ids, out, hidden, vocab);
}

// ---------------------------------------------------------------- residual add + RMSNorm
// For output row r: src = rows ? rows[r] : r;  v = x[src] + delta[src];  (x[src] = v if write_back)
// out[r] = v * rsqrt(mean(v^2) + eps) * w.
template <typename WT, typename OT>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                   const WT* __restrict__ weight, OT* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps, int write_back) {
    CISR_TRACE_SCOPE(TRACE_ADD_RMSNORM);
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float* xr = x + src;
    const float* dr = delta ? delta + src : nullptr;
    extern __shared__ float row_cache[];  // hidden floats
    float sq = 0.f;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        float v = xr[d];
        if (dr) v += dr[d];
        if (write_back && dr) xr[d] = v;
        row_cache[d] = v;
        sq += v * v;
    }
    const float total = block_sum(sq, scratch);
    const float scale = rsqrtf(total / (float)hidden + eps);
    OT* o = out + (size_t)r * hidden;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x)
        o[d] = from_float<OT>(row_cache[d] * scale * to_float(weight[d]));
}

// Four weights and four outputs at a time (the row and the weights start on 16-byte boundaries, hidden % 4 == 0).
__device__ __forceinline__ float4 load_weights4(const float* w, int d4) { return reinterpret_cast<const float4*>(w)[d4]; }
__device__ __forceinline__ float4 load_weights4(const __nv_bfloat16* w, int d4) {
    const uint2 raw = reinterpret_cast<const uint2*>(w)[d4];
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void store4(float* o, int d4, float4 v) { reinterpret_cast<float4*>(o)[d4] = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* o, int d4, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo); raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(o)[d4] = raw;
}

// The same with 16-byte accesses, for widths that are multiples of 4.
template <typename WT, typename OT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                       const WT* __restrict__ weight, OT* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, float eps, int write_back) {
    CISR_TRACE_SCOPE(TRACE_ADD_RMSNORM);
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float row_cache[];
    pdl_trigger();
    pdl_wait();          // x and delta come from the kernels before
    CISR_TRACE_WAITED();
    const int r = blockIdx.x, h4 = hidden >> 2;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float4* xr = reinterpret_cast<float4*>(x + src);
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + src) : nullptr;
    float4* cache4 = reinterpret_cast<float4*>(row_cache);
    float sq = 0.f;
    for (int d = threadIdx.x; d < h4; d += blockDim.x) {
        float4 v = xr[d];
        if (dr) {
            const float4 dv = dr[d];
            v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
            if (write_back) xr[d] = v;
        }
        cache4[d] = v;
        sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float total = block_sum(sq, scratch);
    const float scale = rsqrtf(total / (float)hidden + eps);
    OT* o = out + (size_t)r * hidden;
    const bool wide = !(((uintptr_t)weight | (uintptr_t)o) & 15) && (hidden * sizeof(OT)) % 16 == 0;   // the same for the whole block
    for (int d = threadIdx.x; d < h4; d += blockDim.x) {
        const float4 v = cache4[d];
        if (wide) {
            const float4 w = load_weights4(weight, d);
            store4(o, d, make_float4(v.x * scale * w.x, v.y * scale * w.y, v.z * scale * w.z, v.w * scale * w.w));
            continue;
        }
        const float w0 = to_float(weight[4 * d]), w1 = to_float(weight[4 * d + 1]);
        const float w2 = to_float(weight[4 * d + 2]), w3 = to_float(weight[4 * d + 3]);
        o[4 * d] = from_float<OT>(v.x * scale * w0);
        o[4 * d + 1] = from_float<OT>(v.y * scale * w1);
        o[4 * d + 2] = from_float<OT>(v.z * scale * w2);
        o[4 * d + 3] = from_float<OT>(v.w * scale * w3);
    }
}

// A warp per row, the row in registers (V float4 per lane: widths up to 128 V), four rows per CTA: no shared memory
// and no barrier, every load of a lane in flight before the first is used, 8- or 16-byte stores.  Steps of many tokens
// spend a tenth of their time in this kernel, and a CTA per 576-wide row with scalar stores took 7 us for what the
// memory system moves in 2.
constexpr int NORM_WARPS = 4;
template <typename WT, typename OT, int V>
__global__ void __launch_bounds__(32 * NORM_WARPS)
add_rmsnorm_warp_kernel(float* __restrict__ x, const float* __restrict__ delta, const WT* __restrict__ weight,
                        OT* __restrict__ out, const int* __restrict__ rows, int n_rows, int hidden, float eps, int write_back) {
    CISR_TRACE_SCOPE(TRACE_ADD_RMSNORM);
    pdl_trigger();
    pdl_wait();          // x and delta come from the kernels before
    CISR_TRACE_WAITED();
    const int lane = threadIdx.x & 31, r = blockIdx.x * NORM_WARPS + (threadIdx.x >> 5), h4 = hidden >> 2;
    if (r >= n_rows) return;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float4* xr = reinterpret_cast<float4*>(x + src);
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + src) : nullptr;
    float4 v[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int d = lane + 32 * i;
        v[i] = d < h4 ? xr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sq = 0.f;
    if (dr) {
        float4 dv[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int d = lane + 32 * i;
            dv[i] = d < h4 ? dr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
            v[i].x += dv[i].x; v[i].y += dv[i].y; v[i].z += dv[i].z; v[i].w += dv[i].w;
            if (write_back && lane + 32 * i < h4) xr[lane + 32 * i] = v[i];
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) sq += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    const float scale = rsqrtf(warp_sum(sq) / (float)hidden + eps);
    OT* o = out + (size_t)r * hidden;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int d = lane + 32 * i;
        if (d >= h4) continue;
        const float4 w = load_weights4(weight, d);
        store4(o, d, make_float4(v[i].x * scale * w.x, v[i].y * scale * w.y, v[i].z * scale * w.z, v[i].w * scale * w.w));
    }
}

template <typename WT, typename OT, int V>
static int add_rmsnorm_warp_launch(float* x, const float* delta, const void* w, void* out, const int* rows, int n_rows,
                                   int hidden, float eps, int write_back, cudaStream_t s) {
    return launch_kernel(add_rmsnorm_warp_kernel<WT, OT, V>, dim3((n_rows + NORM_WARPS - 1) / NORM_WARPS), dim3(32 * NORM_WARPS), 0, s,
                         g_pdl, x, delta, (const WT*)w, (OT*)out, rows, n_rows, hidden, eps, write_back);
}

template <typename WT, typename OT>
static int add_rmsnorm_launch(float* x, const float* delta, const void* w, void* out, const int* rows, int n_rows,
                              int hidden, float eps, int write_back, cudaStream_t s) {
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return -2;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<WT, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const bool vec = (hidden & 3) == 0 && !(((uintptr_t)x | (uintptr_t)delta) & 15);
    // rows of up to 2048 floats whose weights and outputs are aligned too: a warp per row
    if (vec && hidden <= 2048 && !(((uintptr_t)w | (uintptr_t)out) & 15) && (hidden * sizeof(OT)) % 16 == 0) {
        const int per_lane = (hidden / 4 + 31) / 32;
        if (per_lane <= 2) return add_rmsnorm_warp_launch<WT, OT, 2>(x, delta, w, out, rows, n_rows, hidden, eps, write_back, s);
        if (per_lane <= 5) return add_rmsnorm_warp_launch<WT, OT, 5>(x, delta, w, out, rows, n_rows, hidden, eps, write_back, s);
        if (per_lane <= 8) return add_rmsnorm_warp_launch<WT, OT, 8>(x, delta, w, out, rows, n_rows, hidden, eps, write_back, s);
        return add_rmsnorm_warp_launch<WT, OT, 16>(x, delta, w, out, rows, n_rows, hidden, eps, write_back, s);
    }
    if (smem > 48 * 1024 && vec) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_vec_kernel<WT, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (vec) {
        const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
        return launch_kernel(add_rmsnorm_vec_kernel<WT, OT>, dim3(n_rows), dim3(threads), smem, s, g_pdl, x, delta, (const WT*)w,
                             (OT*)out, rows, hidden, eps, write_back);
    } else {
        const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
        add_rmsnorm_kernel<WT, OT><<<n_rows, threads, smem, s>>>(x, delta, (const WT*)w, (OT*)out, rows, hidden, eps, write_back);
    }
    return launch_status();
}

CISR_EXPORT int cisr_add_rmsnorm(float* x, const float* delta, const void* weight, int w_dtype, void* out,
                                 int out_dtype, const int* rows, int n_rows, int hidden, float eps, int write_back,
                                 void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (w_dtype == CISR_BF16 && out_dtype == CISR_BF16)
        return add_rmsnorm_launch<__nv_bfloat16, __nv_bfloat16>(x, delta, weight, out, rows, n_rows, hidden, eps, write_back, s);
    if (w_dtype == CISR_F32 && out_dtype == CISR_BF16)
        return add_rmsnorm_launch<float, __nv_bfloat16>(x, delta, weight, out, rows, n_rows, hidden, eps, write_back, s);
    if (w_dtype == CISR_BF16 && out_dtype == CISR_F32)
        return add_rmsnorm_launch<__nv_bfloat16, float>(x, delta, weight, out, rows, n_rows, hidden, eps, write_back, s);
    return add_rmsnorm_launch<float, float>(x, delta, weight, out, rows, n_rows, hidden, eps, write_back, s);
}

// ---------------------------------------------------------------- SwiGLU
// gate_up [T, 2I] float: gate in columns [0, I), up in [I, 2I).  out = gate/(1+exp(-gate)) * up.
template <typename OT>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, OT* __restrict__ out, int inter, size_t total) {
    CISR_TRACE_SCOPE(TRACE_SWIGLU);
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / inter;
    const int c = (int)(i - t * inter);
    const float g = gate_up[t * 2 * inter + c];
    const float u = gate_up[t * 2 * inter + inter + c];
    out[i] = from_float<OT>(g / (1.f + expf(-g)) * u);
}

CISR_EXPORT int cisr_swiglu(const float* gate_up, void* out, int out_dtype, int tokens, int inter, void* stream) {
    const size_t total = (size_t)tokens * inter;
    if (!total) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == CISR_BF16) swiglu_kernel<<<blocks, 256, 0, s>>>(gate_up, (__nv_bfloat16*)out, inter, total);
    else swiglu_kernel<<<blocks, 256, 0, s>>>(gate_up, (float*)out, inter, total);
    return launch_status();
}

// ---------------------------------------------------------------- rotary tables
// cos/sin [T, half] in float from double angles pos * inv_freq[i]; run once per step
// and shared by every layer that rotates with the same theta and width.
__global__ void rotary_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                    float* __restrict__ cos_out, float* __restrict__ sin_out, int half, int total) {
    CISR_TRACE_SCOPE(TRACE_ROTARY_TABLE);
    // No early start for the kernels after this one: the fused q/k/v kernels read these tables before their own wait
    // on their predecessor, so whatever runs between this kernel and them must not start before the tables are written.
    pdl_wait();          // nothing of the kernel before is read, but the chain of waits must not break (see embedding_kernel)
    CISR_TRACE_WAITED();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int t = i / half, f = i - t * half;
    double s, c;
    sincos((double)positions[t] * inv_freq[f], &s, &c);
    cos_out[i] = (float)c;
    sin_out[i] = (float)s;
}

CISR_EXPORT int cisr_rotary_tables(const int* positions, const double* inv_freq, float* cos_out, float* sin_out,
                                   int tokens, int half, void* stream) {
    const int total = tokens * half;
    if (total <= 0) return 0;
    return launch_kernel(rotary_table_kernel, dim3((total + 127) / 128), dim3(128), 0, (cudaStream_t)stream, g_pdl, positions, inv_freq,
                         cos_out, sin_out, half, total);
}

// ---------------------------------------------------------------- rotation + cache write
// proj [T, row_stride] float holds q at column 0, k at k_col, v at v_col (k_col < 0: no keys/values
// in this projection, nothing is written to the cache).  The first 2*rot_half coordinates of each head
// are rotated (pairs (i, i+rot_half), or (2i, 2i+1) when interleaved); the rest pass through.
// q goes to q_out [T, Hq, D]; k (rotated) and v go to page block_table[req_slot[req]][pos / P], offset pos % P,
// in caches laid out [pages, Hkv, P, D].
template <typename QT, typename CT>
__global__ void rope_store_kernel(const float* __restrict__ proj, int row_stride, int k_col, int v_col,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_half,
                                  int interleaved, QT* __restrict__ q_out, CT* __restrict__ k_cache,
                                  CT* __restrict__ v_cache, const int* __restrict__ token_req,
                                  const int* __restrict__ positions, const int* __restrict__ req_slot,
                                  const int* __restrict__ block_table, int table_width, int page_size, int hq,
                                  int hkv, int dim) {
    CISR_TRACE_SCOPE(TRACE_ROPE_STORE);
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * row_stride;
    const float* cs = cos_t ? cos_t + (size_t)t * rot_half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)t * rot_half : nullptr;
    const int rot = 2 * rot_half;
    // queries
    for (int i = threadIdx.x; i < hq * dim; i += blockDim.x) {
        const int h = i / dim, d = i - h * dim;
        const float* src = row + h * dim;
        float v = src[d];
        if (d < rot) {
            int f, other; bool first;
            if (interleaved) { f = d >> 1; first = !(d & 1); other = first ? d + 1 : d - 1; }
            else { first = d < rot_half; f = first ? d : d - rot_half; other = first ? d + rot_half : d - rot_half; }
            const float c = cs[f], s = sn[f], o = src[other];
            v = first ? v * c - o * s : v * c + o * s;
        }
        q_out[((size_t)t * hq + h) * dim + d] = from_float<QT>(v);
    }
    if (k_col < 0) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)req_slot[token_req[t]] * table_width + pos / page_size];
    const int off = pos % page_size;
    if (page < 0) return;  // the host reserves a page before every write; never follow a missing entry
    for (int i = threadIdx.x; i < hkv * dim; i += blockDim.x) {
        const int h = i / dim, d = i - h * dim;
        const float* src = row + k_col + h * dim;
        float v = src[d];
        if (d < rot) {
            int f, other; bool first;
            if (interleaved) { f = d >> 1; first = !(d & 1); other = first ? d + 1 : d - 1; }
            else { first = d < rot_half; f = first ? d : d - rot_half; other = first ? d + rot_half : d - rot_half; }
            const float c = cs[f], s = sn[f], o = src[other];
            v = first ? v * c - o * s : v * c + o * s;
        }
        const size_t dst = (((size_t)page * hkv + h) * page_size + off) * dim + d;
        k_cache[dst] = from_float<CT>(v);
        v_cache[dst] = from_float<CT>(row[v_col + h * dim + d]);
    }
}

CISR_EXPORT int cisr_rope_store(const float* proj, int row_stride, int k_col, int v_col, const float* cos_t,
                                const float* sin_t, int rot_half, int interleaved, void* q_out, int q_dtype,
                                void* k_cache, void* v_cache, int cache_dtype, const int* token_req,
                                const int* positions, const int* req_slot, const int* block_table, int table_width,
                                int page_size, int hq, int hkv, int dim, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    if (2 * rot_half > dim || rot_half < 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
#define CISR_ROPE(QT, CT)                                                                                          \
    rope_store_kernel<QT, CT><<<tokens, 128, 0, s>>>(proj, row_stride, k_col, v_col, cos_t, sin_t, rot_half,        \
                                                      interleaved, (QT*)q_out, (CT*)k_cache, (CT*)v_cache, token_req, \
                                                      positions, req_slot, block_table, table_width, page_size, hq, hkv, dim)
    if (q_dtype == CISR_BF16 && cache_dtype == CISR_BF16) CISR_ROPE(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == CISR_F32 && cache_dtype == CISR_F32) CISR_ROPE(float, float);
    else if (q_dtype == CISR_BF16 && cache_dtype == CISR_F32) CISR_ROPE(__nv_bfloat16, float);
    else CISR_ROPE(float, __nv_bfloat16);
#undef CISR_ROPE
    return launch_status();
}

// ---------------------------------------------------------------- page copy (copy-on-write of a shared page)
// Copies whole pages inside one pool: pool viewed as [n_planes, pages, page_elems]; pairs (src, dst) in `pairs`.
__global__ void page_copy_kernel(uint4* __restrict__ pool, const int* __restrict__ pairs, size_t plane_vec,
                                 size_t page_vec) {
    CISR_TRACE_SCOPE(TRACE_PAGE_COPY);
    const int pair = blockIdx.x, plane = blockIdx.y;
    const uint4* src = pool + plane * plane_vec + (size_t)pairs[2 * pair] * page_vec;
    uint4* dst = pool + plane * plane_vec + (size_t)pairs[2 * pair + 1] * page_vec;
    for (size_t i = threadIdx.x; i < page_vec; i += blockDim.x) dst[i] = src[i];
}

CISR_EXPORT int cisr_page_copy(void* pool, const int* pairs, int n_pairs, int n_planes, long long plane_bytes,
                               long long page_bytes, void* stream) {
    if (n_pairs <= 0) return 0;
    if (page_bytes % 16 || plane_bytes % 16) return -2;
    page_copy_kernel<<<dim3(n_pairs, n_planes), 128, 0, (cudaStream_t)stream>>>((uint4*)pool, pairs, plane_bytes / 16,
                                                                                 page_bytes / 16);
    return launch_status();
}

// ---------------------------------------------------------------- block table updates
// table[idx[i]] = val[i]; the host sends one value per entry, so the order does not matter.
// Launched plainly, and it never lets its successors start early: kernels further down the step read the table before
// their own wait on their predecessor, which is safe only because nothing after this kernel starts before it is done.
__global__ void table_update_kernel(int* __restrict__ table, const int* __restrict__ idx, const int* __restrict__ val, int n) {
    CISR_TRACE_SCOPE(TRACE_TABLE_UPDATE);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && idx[i] >= 0) table[idx[i]] = val[i];
}

CISR_EXPORT int cisr_table_update(int* table, const int* idx, const int* val, int n, void* stream) {
    if (n <= 0) return 0;
    table_update_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(table, idx, val, n);
    return launch_status();
}
