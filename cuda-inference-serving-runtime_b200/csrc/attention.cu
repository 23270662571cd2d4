// Causal grouped-query attention over the paged cache, in float arithmetic.
//
// Compiled once per (HEAD_DIM, STORAGE_BF16): HEAD_DIM any multiple of 16 up to 256;
// STORAGE_BF16=0 reads float queries and a float cache (the true 32-bit path),
// STORAGE_BF16=1 reads bfloat16 queries and a bfloat16 cache.  Scores, softmax
// statistics and the value sum are float in both.
//
//   attn_prefill : portions of any length; one CTA per (64-query tile, query head);
//                  flash-style online softmax over 64- or 32-key tiles gathered page
//                  by page through the block table.
//   attn_decode  : single new tokens; one CTA per (request, kv head, key range);
//                  all query heads of the group share each key/value tile; writes an
//                  unnormalised partial sum with its (max, denominator).
//   attn_merge   : log-sum-exp merge of the partials in a fixed order.
//
// Parity (formulas): kernels/ops.cu:88-123 (online softmax m, l, alpha, beta),
// kernels/ops.cu:35-86 (split + merge), runtime/reference.py:18-31 (grouping
// h -> h / (Hq/Hkv), scale, causal order) of nehanmohammed19/cuda-inference-serving-runtime.
// Cache layout: [pages, kv_heads, page_size, HEAD_DIM].
#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16, at most 256>"
#endif
#if (HEAD_DIM % 16) || (HEAD_DIM > 256) || (HEAD_DIM < 16)
#error "HEAD_DIM must be a multiple of 16 between 16 and 256"
#endif
#ifndef STORAGE_BF16
#define STORAGE_BF16 0
#endif

#if STORAGE_BF16
typedef __nv_bfloat16 st_t;
#else
typedef float st_t;
#endif

namespace {
constexpr int D = HEAD_DIM;
constexpr int VEC = 16 / sizeof(st_t);  // elements per 16-byte load
constexpr int NVEC = D / VEC;           // 16-byte loads per row

__device__ __forceinline__ void load_vec(const st_t* p, float* out) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
#if STORAGE_BF16
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
#else
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
    out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
#endif
}

// ------------------------------------------------------------------ prefill
constexpr int BM = 64;
constexpr int BN = (D <= 128) ? 64 : 32;
constexpr int NJ = BN / 16;  // score columns per thread
constexpr int ND = D / 16;   // output columns per thread
constexpr int QS = BM + 4, KS = BN + 4, PS = BM + 4;
constexpr int PREFILL_THREADS = 256;
constexpr size_t PREFILL_SMEM = sizeof(float) * (size_t)(D * QS + D * KS + BN * D + BN * PS);

__global__ void __launch_bounds__(PREFILL_THREADS)
attn_prefill_kernel(const st_t* __restrict__ q, st_t* __restrict__ out, const st_t* __restrict__ k_cache,
                    const st_t* __restrict__ v_cache, const int* __restrict__ req_slot,
                    const int* __restrict__ block_table, int table_width, const int* __restrict__ tile_req, const int* __restrict__ tile_q0,
                    const int* __restrict__ q_start, const int* __restrict__ q_len,
                    const int* __restrict__ ctx_len, int hq, int hkv, int page_size, float scale, int window) {
    CISR_TRACE_SCOPE(TRACE_ATTN_SIMT);
    extern __shared__ __align__(16) float smem[];
    float* Qs = smem;             // [D][QS]   transposed, pre-scaled
    float* Ks = Qs + D * QS;      // [D][KS]   transposed
    float* Vs = Ks + D * KS;      // [BN][D]
    float* Pt = Vs + BN * D;      // [BN][PS]  transposed probabilities

    const int tile = blockIdx.x, head = blockIdx.y;
    const int req = tile_req[tile], q0 = tile_q0[tile];
    const int rows = min(BM, q_len[req] - q0);
    const int tok0 = q_start[req] + q0;
    const int ctx = ctx_len[req];
    const int qpos0 = ctx - q_len[req] + q0;  // position of the tile's first query
    const int kvh = head / (hq / hkv);
    const int* table = block_table + (size_t)req_slot[req] * table_width;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;

    for (int e = tid; e < BM * NVEC; e += PREFILL_THREADS) {
        const int r = e / NVEC, c = (e - r * NVEC) * VEC;
        float v[VEC];
        if (r < rows) load_vec(q + ((size_t)(tok0 + r) * hq + head) * D + c, v);
        else {
#pragma unroll
            for (int u = 0; u < VEC; ++u) v[u] = 0.f;
        }
#pragma unroll
        for (int u = 0; u < VEC; ++u) Qs[(c + u) * QS + r] = v[u] * scale;
    }

    float o[4][ND], m_run[4], l_run[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m_run[i] = -INFINITY; l_run[i] = 0.f;
#pragma unroll
        for (int j = 0; j < ND; ++j) o[i][j] = 0.f;
    }

    const int k_end = qpos0 + rows;  // one past the last key any row of the tile sees
    int k_first = 0;
    if (window > 0) k_first = max(0, qpos0 - window + 1);
    for (int k0 = (k_first / BN) * BN; k0 < k_end; k0 += BN) {
        __syncthreads();  // previous tile's readers are done (also orders the Q stores on the first pass)
        for (int e = tid; e < BN * NVEC; e += PREFILL_THREADS) {
            const int r = e / NVEC, c = (e - r * NVEC) * VEC;
            const int kpos = k0 + r;
            float kv[VEC], vv[VEC];
            const int page = kpos < ctx ? table[kpos / page_size] : -1;  // -1 also marks a page the window has passed
            if (page >= 0) {
                const size_t base = (((size_t)page * hkv + kvh) * page_size + kpos % page_size) * D + c;
                load_vec(k_cache + base, kv);
                load_vec(v_cache + base, vv);
            } else {
#pragma unroll
                for (int u = 0; u < VEC; ++u) { kv[u] = 0.f; vv[u] = 0.f; }
            }
#pragma unroll
            for (int u = 0; u < VEC; ++u) { Ks[(c + u) * KS + r] = kv[u]; Vs[r * D + c + u] = vv[u]; }
        }
        __syncthreads();

        float s[4][NJ];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < NJ; ++j) s[i][j] = 0.f;
#pragma unroll 4
        for (int d = 0; d < D; ++d) {
            const float4 qv = *reinterpret_cast<const float4*>(Qs + d * QS + ty * 4);
            float kk[NJ];
            if (NJ == 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(Ks + d * KS + tx * 4);
                kk[0] = k4.x; kk[1] = k4.y; kk[NJ - 2] = k4.z; kk[NJ - 1] = k4.w;
            } else {
                const float2 k2 = *reinterpret_cast<const float2*>(Ks + d * KS + tx * 2);
                kk[0] = k2.x; kk[1] = k2.y;
            }
            const float qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < NJ; ++j) s[i][j] = fmaf(qq[i], kk[j], s[i][j]);
        }

        float p[4][NJ];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = ty * 4 + i;
            const int qpos = qpos0 + r;
            float tile_max = -INFINITY;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int kpos = k0 + tx * NJ + j;
                const bool ok = (r < rows) && (kpos <= qpos) && (window <= 0 || kpos + window > qpos);
                s[i][j] = ok ? s[i][j] : -INFINITY;
                tile_max = fmaxf(tile_max, s[i][j]);
            }
#pragma unroll
            for (int off = 8; off; off >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, off));
            const float m_new = fmaxf(m_run[i], tile_max);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = expf(m_run[i] - m_use);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) { p[i][j] = expf(s[i][j] - m_use); sum += p[i][j]; }
#pragma unroll
            for (int off = 8; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            l_run[i] = l_run[i] * alpha + sum;
            m_run[i] = m_new;
#pragma unroll
            for (int j = 0; j < ND; ++j) o[i][j] *= alpha;
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            *reinterpret_cast<float4*>(Pt + (tx * NJ + j) * PS + ty * 4) = make_float4(p[0][j], p[1][j], p[2][j], p[3][j]);
        __syncthreads();

#pragma unroll 4
        for (int t = 0; t < BN; ++t) {
            const float4 pv = *reinterpret_cast<const float4*>(Pt + t * PS + ty * 4);
            const float pp[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int j = 0; j < ND; ++j) {
                const float v = Vs[t * D + tx + 16 * j];
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i][j] = fmaf(pp[i], v, o[i][j]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
        const float inv = 1.f / l_run[i];
        st_t* dst = out + ((size_t)(tok0 + r) * hq + head) * D;
#pragma unroll
        for (int j = 0; j < ND; ++j) dst[tx + 16 * j] = from_float<st_t>(o[i][j] * inv);
    }
}

// ------------------------------------------------------------------ decode (split over key ranges)
constexpr int DEC_THREADS = 128;
constexpr int TK = (D * (int)sizeof(float) <= 256) ? 64 : ((D * (int)sizeof(float) <= 512) ? 32 : 16);
constexpr int KSD = D + 4;  // row stride of the key tile: 16-byte reads of consecutive rows fall in distinct banks

__host__ __device__ inline size_t decode_smem_floats(int group) {
    return (size_t)group * D        // q
           + (size_t)TK * KSD       // K tile
           + (size_t)TK * D         // V tile
           + (size_t)group * TK     // scores / probabilities
           + (size_t)group * D      // output accumulator
           + 3 * (size_t)group;     // running max, running denominator, rescale
}

__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_kernel(const st_t* __restrict__ q, const st_t* __restrict__ k_cache, const st_t* __restrict__ v_cache,
                   const int* __restrict__ req_slot, const int* __restrict__ block_table, int table_width, const int* __restrict__ dec_req,
                   const int* __restrict__ q_start, const int* __restrict__ ctx_len, float* __restrict__ partial,
                   float* __restrict__ stats, int hq, int hkv, int page_size, float scale, int window,
                   int split_size, int n_splits) {
    CISR_TRACE_SCOPE(TRACE_ATTN_SIMT);
    extern __shared__ __align__(16) float smem[];
    const int group = hq / hkv;
    float* qs = smem;                 // [group][D]
    float* Ks = qs + group * D;       // [TK][KSD]
    float* Vs = Ks + TK * KSD;        // [TK][D]
    float* ps = Vs + TK * D;          // [group][TK]
    float* Os = ps + group * TK;      // [group][D]
    float* m_s = Os + group * D;      // [group]
    float* l_s = m_s + group;
    float* a_s = l_s + group;

    const int slot = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int req = dec_req[slot];
    const int tok = q_start[req];
    const int ctx = ctx_len[req];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int* table = block_table + (size_t)req_slot[req] * table_width;

    int lo = split * split_size, hi = min(lo + split_size, ctx);
    if (window > 0) lo = max(lo, ctx - window);

    const size_t part_base = ((size_t)slot * hq + (size_t)kvh * group) * n_splits;  // + g * n_splits + split
    if (lo >= hi) {  // nothing in this range: the merge skips entries with denominator 0
        for (int g = tid; g < group; g += DEC_THREADS) {
            const size_t p = part_base + (size_t)g * n_splits + split;
            stats[2 * p] = -INFINITY; stats[2 * p + 1] = 0.f;
        }
        return;
    }

    for (int e = tid; e < group * NVEC; e += DEC_THREADS) {
        const int g = e / NVEC, c = (e - g * NVEC) * VEC;
        float v[VEC];
        load_vec(q + ((size_t)tok * hq + kvh * group + g) * D + c, v);
#pragma unroll
        for (int u = 0; u < VEC; ++u) { qs[g * D + c + u] = v[u] * scale; }
    }
    for (int e = tid; e < group * D; e += DEC_THREADS) Os[e] = 0.f;
    for (int g = tid; g < group; g += DEC_THREADS) { m_s[g] = -INFINITY; l_s[g] = 0.f; }

    for (int k0 = lo; k0 < hi; k0 += TK) {
        __syncthreads();
        for (int e = tid; e < TK * NVEC; e += DEC_THREADS) {
            const int r = e / NVEC, c = (e - r * NVEC) * VEC;
            const int kpos = k0 + r;
            float kv[VEC], vv[VEC];
            const int page = kpos < hi ? table[kpos / page_size] : -1;
            if (page >= 0) {
                const size_t base = (((size_t)page * hkv + kvh) * page_size + kpos % page_size) * D + c;
                load_vec(k_cache + base, kv);
                load_vec(v_cache + base, vv);
            } else {
#pragma unroll
                for (int u = 0; u < VEC; ++u) { kv[u] = 0.f; vv[u] = 0.f; }
            }
#pragma unroll
            for (int u = 0; u < VEC; ++u) { Ks[r * KSD + c + u] = kv[u]; Vs[r * D + c + u] = vv[u]; }
        }
        __syncthreads();

        for (int e = tid; e < group * TK; e += DEC_THREADS) {
            const int g = e / TK, t = e - g * TK;
            const float4* kr = reinterpret_cast<const float4*>(Ks + t * KSD);
            const float4* qr = reinterpret_cast<const float4*>(qs + g * D);
            float acc = 0.f;
#pragma unroll 4
            for (int d = 0; d < D / 4; ++d) {
                const float4 a = qr[d], b = kr[d];
                acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
                acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
            }
            ps[g * TK + t] = (k0 + t < hi) ? acc : -INFINITY;
        }
        __syncthreads();

        for (int g = warp; g < group; g += DEC_THREADS / 32) {
            float mx = -INFINITY;
            for (int t = lane; t < TK; t += 32) mx = fmaxf(mx, ps[g * TK + t]);
            mx = warp_max(mx);
            const float m_old = m_s[g];
            const float m_new = fmaxf(m_old, mx);  // finite: the range holds at least one key
            float sum = 0.f;
            for (int t = lane; t < TK; t += 32) {
                const float pr = expf(ps[g * TK + t] - m_new);
                ps[g * TK + t] = pr;
                sum += pr;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = expf(m_old - m_new);
                a_s[g] = alpha;
                l_s[g] = l_s[g] * alpha + sum;
                m_s[g] = m_new;
            }
        }
        __syncthreads();

        for (int e = tid; e < group * (D / 4); e += DEC_THREADS) {
            const int g = e / (D / 4), c = (e - g * (D / 4)) * 4;
            float4 acc = *reinterpret_cast<float4*>(Os + g * D + c);
            const float alpha = a_s[g];
            acc.x *= alpha; acc.y *= alpha; acc.z *= alpha; acc.w *= alpha;
            const float* pr = ps + g * TK;
#pragma unroll 4
            for (int t = 0; t < TK; ++t) {
                const float pv = pr[t];
                const float4 v = *reinterpret_cast<const float4*>(Vs + t * D + c);
                acc.x = fmaf(pv, v.x, acc.x); acc.y = fmaf(pv, v.y, acc.y);
                acc.z = fmaf(pv, v.z, acc.z); acc.w = fmaf(pv, v.w, acc.w);
            }
            *reinterpret_cast<float4*>(Os + g * D + c) = acc;
        }
    }
    __syncthreads();
    for (int e = tid; e < group * D; e += DEC_THREADS) {
        const int g = e / D, d = e - g * D;
        partial[(part_base + (size_t)g * n_splits + split) * D + d] = Os[e];
    }
    for (int g = tid; g < group; g += DEC_THREADS) {
        const size_t p = part_base + (size_t)g * n_splits + split;
        stats[2 * p] = m_s[g]; stats[2 * p + 1] = l_s[g];
    }
}

__global__ void attn_merge_kernel(const float* __restrict__ partial, const float* __restrict__ stats,
                                  st_t* __restrict__ out, const int* __restrict__ dec_req,
                                  const int* __restrict__ q_start, int hq, int n_splits) {
    CISR_TRACE_SCOPE(TRACE_ATTN_MERGE);
    const int slot = blockIdx.x, head = blockIdx.y;
    const size_t base = ((size_t)slot * hq + head) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s)
        if (stats[2 * (base + s) + 1] > 0.f) m = fmaxf(m, stats[2 * (base + s)]);
    const int tok = q_start[dec_req[slot]];
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float num = 0.f, den = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float l = stats[2 * (base + s) + 1];
            if (l > 0.f) {
                const float w = expf(stats[2 * (base + s)] - m);
                num = fmaf(w, partial[(base + s) * D + d], num);
                den = fmaf(w, l, den);
            }
        }
        out[((size_t)tok * hq + head) * D + d] = from_float<st_t>(den > 0.f ? num / den : 0.f);  // no keys at all: a padding row
    }
}
}  // namespace

CISR_EXPORT int cisr_attn_head_dim() { return D; }
CISR_EXPORT int cisr_attn_storage_bf16() { return STORAGE_BF16; }
CISR_EXPORT int cisr_attn_prefill_tile() { return BM; }

CISR_EXPORT int cisr_attn_prefill(const void* q, void* out, const void* k_cache, const void* v_cache,
                                  const int* req_slot, const int* block_table, int table_width, const int* tile_req, const int* tile_q0,
                                  int n_tiles, const int* q_start, const int* q_len, const int* ctx_len, int hq,
                                  int hkv, int page_size, float scale, int window, void* stream) {
    if (n_tiles <= 0) return 0;
    if (hq % hkv) return -2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREFILL_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    attn_prefill_kernel<<<dim3(n_tiles, hq), PREFILL_THREADS, PREFILL_SMEM, (cudaStream_t)stream>>>(
        (const st_t*)q, (st_t*)out, (const st_t*)k_cache, (const st_t*)v_cache, req_slot, block_table, table_width, tile_req,
        tile_q0, q_start, q_len, ctx_len, hq, hkv, page_size, scale, window);
    return launch_status();
}

// partial: float [n_dec, hq, n_splits, D]; stats: float [n_dec, hq, n_splits, 2]
CISR_EXPORT int cisr_attn_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                 const int* req_slot, const int* block_table, int table_width, const int* dec_req, int n_dec,
                                 const int* q_start, const int* ctx_len, float* partial, float* stats, int hq,
                                 int hkv, int page_size, float scale, int window, int split_size, int n_splits,
                                 void* stream) {
    if (n_dec <= 0) return 0;
    if (hq % hkv || split_size <= 0 || n_splits <= 0) return -2;
    const size_t smem = decode_smem_floats(hq / hkv) * sizeof(float);
    if (smem > 220 * 1024) return -3;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    cudaStream_t s = (cudaStream_t)stream;
    attn_decode_kernel<<<dim3(n_dec, hkv, n_splits), DEC_THREADS, smem, s>>>(
        (const st_t*)q, (const st_t*)k_cache, (const st_t*)v_cache, req_slot, block_table, table_width, dec_req, q_start,
        ctx_len, partial, stats, hq, hkv, page_size, scale, window, split_size, n_splits);
    int status = launch_status();
    if (status) return status;
    attn_merge_kernel<<<dim3(n_dec, hq), D < 128 ? 64 : 128, 0, s>>>(partial, stats, (st_t*)out, dec_req, q_start, hq, n_splits);
    return launch_status();
}
