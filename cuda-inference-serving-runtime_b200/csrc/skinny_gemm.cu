// Weight-streaming matrix products for steps with few tokens (decode): out[M, N] = a[M, K] * w[N, K]^T
// with M <= 64, bfloat16 operands, float accumulation on the tensor cores, fused with what
// surrounds the product so that a decode layer is five launches instead of ten:
//
//   prologue  ACT   : a is bfloat16 [M, K] in global memory
//             NORM  : a = rmsnorm(x + delta) * norm_w; CTA 0 also writes the residual sum to x_out when there is a
//                     delta (a different buffer than x, so no CTA reads what another has overwritten).  `rows`, when
//                     given, picks the rows of x (final norm).
//   epilogue  PLAIN : out float [M, N], written or added to (the residual form: out is the stream itself)
//             SWIGLU: w stacks gate rows [0, I) over up rows [I, 2I); out bfloat16 [M, I] = silu(g) * u
//             ROPE  : w stacks q, k and v heads; each CTA owns one head, rotates it (q and k) and writes q to
//                     q_out [M, Hq, D] and k, v into their cache pages (as elementwise.cu's rope_store does)
//
// The weight matrix is the A operand of mma.sync.m16n8k16 (16 output features by 16 k), the tokens are the
// 8-wide N dimension, so every weight element is read from global memory exactly once, straight into
// registers with 16-byte loads: lane (r = lane / 4, t = lane % 4) loads w[f0 + r][32c + 8t .. 8t + 7] and
// w[f0 + r + 8][same]; the two mma of a 32-wide chunk take k = 8t + 4j + {0,1} and 8t + 4j + {2,3}
// (j = 0, 1) as their "columns 2t + {0,1}" and "8 + 2t + {0,1}", and the token operand uses the same k
// permutation, so the sum over k is unchanged.
//
// A CTA is RT row tiles (16 features each) by KS splits of K, one warp each (the rotation kernel gives a warp two row
// tiles).  A warp first issues the loads of its first MAXC chunks of weights (they depend on no earlier kernel), then
// waits for the kernel before it (programmatic dependent launch), and the KS partial sums of a row tile are added in
// shared memory in a fixed order.
//
// The token operand, up to 16 tokens: with that permutation lane (r, t) needs exactly the eight values
// a[r][32c + 8t .. + 7] as they lie in memory, so every lane fetches them itself, for its warp's chunks only, right
// after the wait: one trip to memory and no pass through shared memory.  With the norm prologue the operand is
// (x + delta) * norm_w rounded to bfloat16; the row's 1 / rms is a common factor of the whole product, so it is applied
// to the finished sums, and the squares are added up per K split on the way and over the splits in the epilogue.
// More tokens are staged once per CTA in shared memory, normed there.
//
// Parity: these products are what runtime/blas.py:41-56 of the reference hands to cuBLAS with M = batch;
// the fused neighbours are kernels/execution.cu:12-24 (residual + norm), :7-10 (SwiGLU), :28-40 (rotation
// and cache write).  K must be a multiple of 8 (16-byte rows).
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
enum : int { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_ROPE = 2 };
#ifndef SKINNY_MAXC
#define SKINNY_MAXC 6
#endif
#ifndef SKINNY_KS
#define SKINNY_KS 8
#endif
// Chunks of 32 k whose weights a warp holds in registers at once: SKINNY_MAXC, or half of it where that covers the
// warp's whole share of K (kernels this brief pay for every instruction they fetch, also for the predicated-off ones).
constexpr int MAXC_FULL = SKINNY_MAXC, MAXC_HALF = (SKINNY_MAXC + 1) / 2;
bool g_pdl = false;

struct SkinnyArgs {
    const bf16* w; int n; int k;
    const bf16* act;                               // ACT prologue
    const float* x; const float* delta; const void* norm_w; int norm_w_bf16; float eps; float* x_out; const int* rows;
    int m; int rt; int ks;
    int sums_in_smem;                              // NORM prologue: x + delta staged as float in shared memory (one pass over global memory)
    float* out_f32; bf16* out_bf16; int inter;      // PLAIN / SWIGLU
    // ROPE
    const float* cos_t; const float* sin_t; int rot_half; int interleaved; bf16* q_out; bf16* k_cache; bf16* v_cache;
    const int* positions; const int* token_req; const int* req_slot; const int* block_table; int table_width; int page_size;
    int hq; int hkv; int dim;
    int accumulate;                                // PLAIN: out += product
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint4 load_weights(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// The token operand in shared memory: hs[MT * 8][ldh] bfloat16, rows >= m zero.  All warps take part.
// NORM prologue: `nw` holds the norm weights as float (fetched before the wait on the previous kernel).  With `sums`
// (float [MT * 8][k]) every row is read from global memory once: all of a lane's loads are issued before the first
// is used, the sum x + delta is kept in shared memory while the warp adds up its squares, and the second pass
// reads it from there.  Without `sums` (rows too long for shared memory) the second pass reads global memory again.
template <int MT>
__device__ void stage_tokens(const SkinnyArgs& a, bf16* hs, int ldh, const float* nw, float* sums) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const int k = a.k, k8 = k / 8;
    if (a.act) {
        constexpr int UA = 4;                      // loads in flight per thread: one trip to memory for up to 4 x 512 x 16 bytes
        const int total = MT * 8 * k8;
        for (int base = tid; base < total; base += UA * blockDim.x) {
            uint4 v[UA];
#pragma unroll
            for (int u = 0; u < UA; ++u) {
                const int e = base + u * blockDim.x, r = e / k8, c = (e - r * k8) * 8;
                v[u] = make_uint4(0, 0, 0, 0);
                if (e < total && r < a.m) v[u] = *reinterpret_cast<const uint4*>(a.act + (size_t)r * k + c);
            }
#pragma unroll
            for (int u = 0; u < UA; ++u) {
                const int e = base + u * blockDim.x, r = e / k8, c = (e - r * k8) * 8;
                if (e < total) *reinterpret_cast<uint4*>(hs + r * ldh + c) = v[u];
            }
        }
        return;
    }
    const int k4 = k / 4;
    constexpr int U = 6;                           // float4 loads of x (and of delta) in flight per lane
    for (int r = warp; r < MT * 8; r += nwarp) {
        bf16* dst = hs + r * ldh;
        if (r >= a.m) {
            for (int c = lane; c < k8; c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
            continue;
        }
        const size_t src = (size_t)(a.rows ? a.rows[r] : r) * k;
        const float4* xr = reinterpret_cast<const float4*>(a.x + src);
        const float4* dr = a.delta ? reinterpret_cast<const float4*>(a.delta + src) : nullptr;
        float4* row_sums = sums ? reinterpret_cast<float4*>(sums + (size_t)r * k) : nullptr;
        const bool write_x = a.x_out && blockIdx.x == 0;
        float sq = 0.f;
        for (int base = 0; base < k4; base += 32 * U) {
            float4 xv[U], dv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int c = base + lane + 32 * u;
                xv[u] = make_float4(0.f, 0.f, 0.f, 0.f); dv[u] = xv[u];
                if (c < k4) { xv[u] = xr[c]; if (dr) dv[u] = dr[c]; }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int c = base + lane + 32 * u;
                float4 v = xv[u];
                v.x += dv[u].x; v.y += dv[u].y; v.z += dv[u].z; v.w += dv[u].w;
                sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                if (c < k4) {
                    if (row_sums) row_sums[c] = v;
                    if (write_x) reinterpret_cast<float4*>(a.x_out + src)[c] = v;
                }
            }
        }
        sq = warp_sum(sq);
        const float scale = rsqrtf(sq / (float)k + a.eps);
        __syncwarp();                              // the lanes read back only what they wrote themselves; cheap insurance
#pragma unroll 4
        for (int c = lane; c < k4; c += 32) {
            float4 v;
            if (row_sums) {
                v = row_sums[c];
            } else {
                v = xr[c];
                if (dr) { const float4 d = dr[c]; v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w; }
            }
            const float4 wv = reinterpret_cast<const float4*>(nw)[c];
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale * wv.x, v.y * scale * wv.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * scale * wv.z, v.w * scale * wv.w);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo); packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst + 4 * c) = packed;
        }
    }
}

// RW: row tiles per warp (they share the warp's token operand).  The CTA's row tiles are RT * RW; a.rt counts warps.
template <int MT, int EPI, int MAXC, int RW>
__global__ void __launch_bounds__(EPI == EPI_PLAIN ? 256 : 512) skinny_kernel(const SkinnyArgs a) {
    CISR_TRACE_SCOPE(EPI == EPI_ROPE ? TRACE_SKINNY_ROPE : EPI == EPI_SWIGLU ? TRACE_SKINNY_SWIGLU : TRACE_SKINNY_PLAIN);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // Up to 16 tokens: every lane fetches its own share of the tokens straight from global memory as the mma's token
    // operand, no staging in shared memory (see the main loop).  More tokens: staged once per CTA.
    constexpr bool DIRECT = MT <= 2;
    const int ldh = a.k + 8;
    bf16* hs = reinterpret_cast<bf16*>(smem_raw);                // staged only: [MT * 8][ldh]
    float* red = DIRECT ? reinterpret_cast<float*>(smem_raw) : reinterpret_cast<float*>(hs + MT * 8 * ldh);   // [KS][RT * RW * 16][MT * 8]
    float* ssq = red + (size_t)a.ks * a.rt * RW * 16 * MT * 8;   // DIRECT, NORM: [KS][MT * 8] sums of squares of the K splits
    float* nw = ssq + (DIRECT ? a.ks * MT * 8 : 0);              // NORM: [k] norm weights as float
    float* sums = a.sums_in_smem ? nw + a.k : nullptr;           // staged NORM: [MT * 8][k] x + delta
    float* tables = nw + (a.act ? 0 : a.k) + (a.sums_in_smem ? (size_t)MT * 8 * a.k : 0);   // ROPE: [2][m][rot_half] cos, sin
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, t = lane & 3;
    const int RT = a.rt, KS = a.ks;
    const int rt = warp % RT, ks = warp / RT;
    const int k = a.k, chunks = (k + 31) / 32;

    bool ok_lo[RW], ok_hi[RW];
    const bf16* row_lo[RW]; const bf16* row_hi[RW];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
        const int tile = rt * RW + j;              // the warp's j-th row tile among the CTA's
        int f_lo, f_hi, n_lo;
        if (EPI == EPI_SWIGLU) { f_lo = (blockIdx.x * RT * RW + tile) * 8; f_hi = a.inter + f_lo; n_lo = a.inter; }   // rows 0-7 of a tile gate, 8-15 up
        else if (EPI == EPI_ROPE) { f_lo = blockIdx.x * a.dim + tile * 16; f_hi = f_lo + 8; n_lo = a.n; }
        else { f_lo = (blockIdx.x * RT * RW + tile) * 16; f_hi = f_lo + 8; n_lo = a.n; }
        ok_lo[j] = f_lo + r < n_lo; ok_hi[j] = f_hi + r < a.n;
        row_lo[j] = a.w + (size_t)(ok_lo[j] ? f_lo + r : 0) * k + 8 * t;
        row_hi[j] = a.w + (size_t)(ok_hi[j] ? f_hi + r : 0) * k + 8 * t;
    }

    // weights of the first batch of chunks: nothing here depends on an earlier kernel
    uint4 wl[RW][MAXC], wh[RW][MAXC];
    auto load_batch = [&](int base) {
#pragma unroll
        for (int j = 0; j < RW; ++j) {
#pragma unroll
            for (int i = 0; i < MAXC; ++i) {
                const int c = ks + (base + i) * KS;
                const bool in_k = c < chunks && c * 32 + 8 * t < k;
                wl[j][i] = make_uint4(0, 0, 0, 0); wh[j][i] = make_uint4(0, 0, 0, 0);
                if (in_k && ok_lo[j]) wl[j][i] = load_weights(row_lo[j] + c * 32);
                if (in_k && ok_hi[j]) wh[j][i] = load_weights(row_hi[j] + c * 32);
            }
        }
    };
    load_batch(0);
    // ROPE: where each token's key and value go is known from the step's metadata and the block table, which the
    // kernel before this one does not write: look it up now, three dependent loads off the path after the wait
    __shared__ long long cache_row[MT * 8];
    if (EPI == EPI_ROPE && tid < a.m) {
        const int pos = a.positions[tid];
        const int page = a.block_table[(size_t)a.req_slot[a.token_req[tid]] * a.table_width + pos / a.page_size];
        cache_row[tid] = page < 0 ? -1 : (long long)page * a.hkv * a.page_size + pos % a.page_size;
    }
    // The norm weights and the rotation tables (made at the start of the step) do not come from the kernel before either.
    if (!a.act) {
        for (int c = tid; c < a.k; c += blockDim.x)
            nw[c] = a.norm_w_bf16 ? __bfloat162float(((const bf16*)a.norm_w)[c]) : ((const float*)a.norm_w)[c];
    }
    if (EPI == EPI_ROPE && a.rot_half > 0) {
        const int n_rot = a.m * a.rot_half;
        for (int c = tid; c < n_rot; c += blockDim.x) { tables[c] = a.cos_t[c]; tables[n_rot + c] = a.sin_t[c]; }
    }
    if (EPI != EPI_ROPE) pdl_trigger();
    pdl_wait();
    CISR_TRACE_WAITED();
    if (!a.act) __syncthreads();                  // the norm weights are in shared memory
    // PLAIN, adding into `out`: what is there now (written by kernels that have finished) is requested before the
    // product, so the sum at the end does not wait for it
    float there = 0.f;
    if (EPI == EPI_PLAIN && a.accumulate) {
        const int rows_all = a.rt * RW * 16, mrow = tid / rows_all, f = blockIdx.x * rows_all + (tid - mrow * rows_all);
        if (mrow < a.m && f < a.n) there = a.out_f32[(size_t)mrow * a.n + f];
    }

    if (!DIRECT) {
        stage_tokens<MT>(a, hs, ldh, nw, sums);
        __syncthreads();
    }
    CISR_TRACE_MARK(0);
    // DIRECT: lane (r, t) holds token mt * 8 + r; its 8 values k = 32 c + 8 t .. + 7 of a chunk are the mma's token
    // operand as they lie in memory.  With the norm prologue the operand is (x + delta) * norm_w rounded to bfloat16,
    // the row's 1 / rms is a factor of the whole product and is applied to the sums at the end; the squares are added
    // up per K split here (by the warps of row tile 0) and over the splits there.
    float sq[MT];
    size_t src_row[MT];
    bool live[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int tok = mt * 8 + r;
        sq[mt] = 0.f;
        live[mt] = DIRECT && tok < a.m;
        src_row[mt] = (size_t)(live[mt] ? (a.act || !a.rows ? tok : a.rows[tok]) : 0) * k;
    }
    const bool write_x = DIRECT && !a.act && a.x_out && blockIdx.x == 0 && rt == 0;

    float acc[RW][MT][4];
#pragma unroll
    for (int j = 0; j < RW; ++j)
#pragma unroll
        for (int i = 0; i < MT; ++i) { acc[j][i][0] = acc[j][i][1] = acc[j][i][2] = acc[j][i][3] = 0.f; }
    for (int base = 0; ks + base * KS < chunks; base += MAXC) {
        if (base) load_batch(base);
        uint4 tok_b[DIRECT ? MAXC : 1][MT];
        if (DIRECT && a.act) {
#pragma unroll
            for (int i = 0; i < MAXC; ++i) {
                const int c = ks + (base + i) * KS, kb = c * 32 + 8 * t;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    tok_b[i][mt] = make_uint4(0, 0, 0, 0);
                    if (c < chunks && kb < k && live[mt]) tok_b[i][mt] = *reinterpret_cast<const uint4*>(a.act + src_row[mt] + kb);
                }
            }
        } else if (DIRECT) {
            float4 xv[MAXC][MT][2];
#pragma unroll
            for (int i = 0; i < MAXC; ++i) {                         // every load of the batch before the first use
                const int c = ks + (base + i) * KS, kb = c * 32 + 8 * t;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    xv[i][mt][0] = make_float4(0.f, 0.f, 0.f, 0.f); xv[i][mt][1] = xv[i][mt][0];
                    if (c < chunks && kb < k && live[mt]) {
                        const float4* xp = reinterpret_cast<const float4*>(a.x + src_row[mt] + kb);
                        xv[i][mt][0] = xp[0]; xv[i][mt][1] = xp[1];
                    }
                }
            }
            if (a.delta) {
#pragma unroll
                for (int i = 0; i < MAXC; ++i) {
                    const int c = ks + (base + i) * KS, kb = c * 32 + 8 * t;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        if (c < chunks && kb < k && live[mt]) {
                            const float4* dp = reinterpret_cast<const float4*>(a.delta + src_row[mt] + kb);
                            const float4 d0 = dp[0], d1 = dp[1];
                            float4& v0 = xv[i][mt][0]; float4& v1 = xv[i][mt][1];
                            v0.x += d0.x; v0.y += d0.y; v0.z += d0.z; v0.w += d0.w;
                            v1.x += d1.x; v1.y += d1.y; v1.z += d1.z; v1.w += d1.w;
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < MAXC; ++i) {
                const int c = ks + (base + i) * KS, kb = c * 32 + 8 * t;
                const bool in_k = c < chunks && kb < k;
                float4 n0 = make_float4(0.f, 0.f, 0.f, 0.f), n1 = n0;
                if (in_k) { n0 = *reinterpret_cast<const float4*>(nw + kb); n1 = *reinterpret_cast<const float4*>(nw + kb + 4); }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const float4 v0 = xv[i][mt][0], v1 = xv[i][mt][1];
                    sq[mt] += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
                    if (write_x && in_k && live[mt]) {
                        float4* xo = reinterpret_cast<float4*>(a.x_out + src_row[mt] + kb);
                        xo[0] = v0; xo[1] = v1;
                    }
                    tok_b[i][mt].x = pack2(v0.x * n0.x, v0.y * n0.y); tok_b[i][mt].y = pack2(v0.z * n0.z, v0.w * n0.w);
                    tok_b[i][mt].z = pack2(v1.x * n1.x, v1.y * n1.y); tok_b[i][mt].w = pack2(v1.z * n1.z, v1.w * n1.w);
                }
            }
        }
        // Every lane runs every mma (a warp-wide instruction must never sit under a lane-dependent condition);
        // lanes whose 8 columns lie beyond K, and chunks beyond the last, feed zeros on both sides.
#pragma unroll
        for (int i = 0; i < MAXC; ++i) {
            const int c = ks + (base + i) * KS;
            const int kb = c * 32 + 8 * t;
            const bool in_k = c < chunks && kb < k;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint4 b = make_uint4(0, 0, 0, 0);
                if (DIRECT) b = tok_b[i][mt];
                else if (in_k) b = *reinterpret_cast<const uint4*>(hs + (mt * 8 + r) * ldh + kb);   // k = kb .. kb + 7 of token mt*8 + r
#pragma unroll
                for (int j = 0; j < RW; ++j) {
                    mma_bf16(acc[j][mt], wl[j][i].x, wh[j][i].x, wl[j][i].y, wh[j][i].y, b.x, b.y);
                    mma_bf16(acc[j][mt], wl[j][i].z, wh[j][i].z, wl[j][i].w, wh[j][i].w, b.z, b.w);
                }
            }
        }
    }

    // ROPE: the kernel after this one is the attention, whose CTAs request their whole key range as soon as they start.
    // Let them start only now that this kernel's own tokens have arrived: started earlier, their tens of megabytes queue
    // in front of the few kilobytes that this kernel (and the one before it) wait for, which cost more than the earlier
    // start saved.
    if (EPI == EPI_ROPE) pdl_trigger();
    CISR_TRACE_MARK(1);
    // partial sums: red[ks][rt * 16 + row][token]
    const int rows_cta = RT * RW * 16, mw = MT * 8;
#pragma unroll
    for (int j = 0; j < RW; ++j) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float* dst = red + ((size_t)ks * rows_cta + (rt * RW + j) * 16) * mw + mt * 8 + 2 * t;
            dst[r * mw] = acc[j][mt][0]; dst[r * mw + 1] = acc[j][mt][1];
            dst[(r + 8) * mw] = acc[j][mt][2]; dst[(r + 8) * mw + 1] = acc[j][mt][3];
        }
    }
    if (DIRECT && !a.act && rt == 0) {              // the K split's share of each token's sum of squares
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float v = sq[mt];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0) ssq[ks * mw + mt * 8 + r] = v;
        }
    }
    __syncthreads();
    CISR_TRACE_MARK(2);
    // DIRECT with the norm prologue: 1 / rms of token `mrow`, the K splits in their fixed order
    auto inv_rms = [&](int mrow) {
        if (!DIRECT || a.act) return 1.f;
        float total = 0.f;
        for (int q = 0; q < KS; ++q) total += ssq[q * mw + mrow];
        return rsqrtf(total / (float)k + a.eps);
    };

    if (EPI == EPI_PLAIN) {
        for (int e = tid; e < rows_cta * a.m; e += blockDim.x) {
            const int mrow = e / rows_cta, row = e - mrow * rows_cta;
            const int f = blockIdx.x * rows_cta + row;
            if (f >= a.n) continue;
            float v = 0.f;
            for (int q = 0; q < KS; ++q) v += red[((size_t)q * rows_cta + row) * mw + mrow];
            v *= inv_rms(mrow);
            float* dst = a.out_f32 + (size_t)mrow * a.n + f;
            if (a.accumulate) v += e == tid ? there : *dst;          // the thread's first element was requested early
            *dst = v;
        }
    } else if (EPI == EPI_SWIGLU) {
        const int per = RT * RW * 8;               // features of this CTA
        for (int e = tid; e < per * a.m; e += blockDim.x) {
            const int mrow = e / per, col = e - mrow * per;
            const int f = blockIdx.x * per + col;
            if (f >= a.inter) continue;
            const int row = (col >> 3) * 16 + (col & 7);             // gate row of the feature in the CTA's tiles; up is 8 below
            float g = 0.f, u = 0.f;
            for (int q = 0; q < KS; ++q) {
                g += red[((size_t)q * rows_cta + row) * mw + mrow];
                u += red[((size_t)q * rows_cta + row + 8) * mw + mrow];
            }
            const float sc = inv_rms(mrow);
            g *= sc; u *= sc;
            a.out_bf16[(size_t)mrow * a.inter + f] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
        }
    } else {
        const int dim = a.dim, hh = blockIdx.x;
        for (int e = tid; e < dim * a.m; e += blockDim.x) {     // first the sum over the K splits, in place in split 0
            const int mrow = e / dim, row = e - mrow * dim;
            float v = 0.f;
            for (int q = 0; q < KS; ++q) v += red[((size_t)q * rows_cta + row) * mw + mrow];
            red[(size_t)row * mw + mrow] = v * inv_rms(mrow);
        }
        __syncthreads();
        const bool is_q = hh < a.hq, is_k = !is_q && hh < a.hq + a.hkv;
        const int rot = 2 * a.rot_half;
        for (int e = tid; e < a.m * dim; e += blockDim.x) {
            const int mrow = e / dim, d = e - mrow * dim;
            float v = red[(size_t)d * mw + mrow];
            if ((is_q || is_k) && d < rot) {
                int f, other; bool first;
                if (a.interleaved) { f = d >> 1; first = !(d & 1); other = first ? d + 1 : d - 1; }
                else { first = d < a.rot_half; f = first ? d : d - a.rot_half; other = first ? d + a.rot_half : d - a.rot_half; }
                const float c = tables[mrow * a.rot_half + f], s = tables[a.m * a.rot_half + mrow * a.rot_half + f];
                const float o = red[(size_t)other * mw + mrow];
                v = first ? v * c - o * s : v * c + o * s;
            }
            if (is_q) {
                a.q_out[((size_t)mrow * a.hq + hh) * dim + d] = __float2bfloat16_rn(v);
            } else {
                const long long at = cache_row[mrow];     // page * hkv * page_size + offset in the page
                if (at < 0) continue;                      // a padding row: its slot holds no pages
                const int kvh = is_k ? hh - a.hq : hh - a.hq - a.hkv;
                const size_t dst = ((size_t)at + (size_t)kvh * a.page_size) * dim + d;
                (is_k ? a.k_cache : a.v_cache)[dst] = __float2bfloat16_rn(v);
            }
        }
    }
}

int sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

template <int MT, int EPI, int MAXC, int RW>
int launch_sized(const SkinnyArgs& a, int grid, size_t smem, cudaStream_t s) {
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(skinny_kernel<MT, EPI, MAXC, RW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    return launch_kernel(skinny_kernel<MT, EPI, MAXC, RW>, dim3(grid), dim3(32 * a.rt * a.ks), smem, s, g_pdl, a);
}

// RW row tiles per warp, a.rt warps side by side, a.ks splits of K: a.rt * a.ks warps (at most 16)
template <int MT, int EPI, int RW>
int launch_tiles(SkinnyArgs& a, int grid, cudaStream_t s) {
    const int tiles = a.rt * RW;
    const size_t extra = (a.act ? 0 : sizeof(float) * (size_t)a.k) +
                         (EPI == EPI_ROPE ? sizeof(float) * 2 * (size_t)a.m * a.rot_half : 0);
    constexpr bool DIRECT = MT <= 2;                              // no staged tokens: the partial sums, the sums of squares, the norm weights
    const size_t staged = DIRECT ? 0 : sizeof(bf16) * (size_t)(MT * 8) * (a.k + 8);
    size_t smem = staged + sizeof(float) * ((size_t)a.ks * tiles * 16 * MT * 8 + (DIRECT ? a.ks * MT * 8 : 0)) + extra;
    if (smem > 220 * 1024 && a.ks > 1 && EPI == EPI_PLAIN) {   // long rows and many tokens: give up the K split for room
        a.ks = 1;
        smem = staged + sizeof(float) * ((size_t)tiles * 16 * MT * 8 + (DIRECT ? MT * 8 : 0)) + extra;
    }
    if (smem > 220 * 1024) return -3;
    const size_t sums_bytes = sizeof(float) * (size_t)(MT * 8) * a.k;
    a.sums_in_smem = !DIRECT && !a.act && smem + sums_bytes <= 100 * 1024;   // keep two CTAs per SM
    if (a.sums_in_smem) smem += sums_bytes;
    const int per_warp = ((a.k + 31) / 32 + a.ks - 1) / a.ks;         // chunks of K each warp multiplies
    if constexpr (RW > 1) return launch_sized<MT, EPI, MAXC_HALF, RW>(a, grid, smem, s);      // the caller checked the share
    else if (per_warp <= MAXC_HALF) return launch_sized<MT, EPI, MAXC_HALF, RW>(a, grid, smem, s);
    else return launch_sized<MT, EPI, MAXC_FULL, RW>(a, grid, smem, s);
}

template <int MT, int EPI>
int launch_epilogue(SkinnyArgs& a, cudaStream_t s) {
    if constexpr (EPI == EPI_ROPE) {
        const int grid = a.hq + 2 * a.hkv;                       // a CTA per head; at most 16 warps
        if constexpr (MT <= 2) {
            // two row tiles per warp where the head allows it and the weights of a warp's share of K still fit its
            // registers: twice the K splits, so half the chunks (and half the trips to memory) per warp
            const int rt = a.dim / 32, ks = max(1, min(SKINNY_KS, 16 / max(rt, 1)));
            if (a.dim % 32 == 0 && ((a.k + 31) / 32 + ks - 1) / ks <= MAXC_HALF) {
                a.rt = rt; a.ks = ks;
                return launch_tiles<MT, EPI, 2>(a, grid, s);
            }
        }
        a.rt = a.dim / 16; a.ks = max(1, min(4, 16 / a.rt));
        return launch_tiles<MT, EPI, 1>(a, grid, s);
    }
    if (EPI == EPI_SWIGLU) {
        // 8 features per CTA, or 16 where that many CTAs would not be resident at once (every CTA fetches all tokens)
        a.rt = (a.inter + 7) / 8 > sm_count() ? 2 : 1; a.ks = SKINNY_KS;
        return launch_tiles<MT, EPI, 1>(a, (a.inter + 8 * a.rt - 1) / (8 * a.rt), s);
    }
    if (MT <= 2) { a.rt = 1; a.ks = SKINNY_KS; return launch_tiles<MT, EPI, 1>(a, (a.n + 15) / 16, s); }
    a.rt = 4; a.ks = 2;                                           // more tokens: stage them once per 64 features
    return launch_tiles<MT, EPI, 1>(a, (a.n + 63) / 64, s);
}

template <int MT>
int launch(SkinnyArgs& a, int epilogue, cudaStream_t s) {
    if (epilogue == EPI_ROPE) return launch_epilogue<MT, EPI_ROPE>(a, s);
    if (epilogue == EPI_SWIGLU) return launch_epilogue<MT, EPI_SWIGLU>(a, s);
    return launch_epilogue<MT, EPI_PLAIN>(a, s);
}
}  // namespace

CISR_EXPORT int cisr_skinny_max_tokens() { return 64; }
CISR_EXPORT void cisr_skinny_set_pdl(int on) { g_pdl = on != 0; }

// One entry point; unused pointer groups are null.  Returns -2 for shapes it does not take (the caller then
// uses the library product and the separate kernels).
CISR_EXPORT int cisr_skinny_gemm(const void* w, int n, int k, const void* act, const float* x, const float* delta,
                                 const void* norm_w, int norm_w_dtype, float eps, float* x_out, const int* rows, int m,
                                 int epilogue, float* out_f32, void* out_bf16, int inter, const float* cos_t,
                                 const float* sin_t, int rot_half, int interleaved, void* q_out, void* k_cache,
                                 void* v_cache, const int* positions, const int* token_req, const int* req_slot,
                                 const int* block_table, int table_width, int page_size, int hq, int hkv, int dim,
                                 int accumulate, void* stream) {
    if (m <= 0) return 0;
    if (m > 64 || k % 8 || k <= 0 || n <= 0) return -2;
    if (epilogue == EPI_ROPE && (dim % 16 || dim > 256 || dim < 16 || n != (hq + 2 * hkv) * dim || 2 * rot_half > dim)) return -2;
    if (epilogue == EPI_SWIGLU && n != 2 * inter) return -2;
    SkinnyArgs a;
    a.w = (const bf16*)w; a.n = n; a.k = k; a.act = (const bf16*)act; a.x = x; a.delta = delta; a.norm_w = norm_w;
    a.norm_w_bf16 = norm_w_dtype == CISR_BF16; a.eps = eps; a.x_out = x_out; a.rows = rows; a.m = m; a.rt = 1; a.ks = 1;
    a.sums_in_smem = 0; a.accumulate = accumulate != 0 && epilogue == EPI_PLAIN;
    a.out_f32 = out_f32; a.out_bf16 = (bf16*)out_bf16; a.inter = inter; a.cos_t = cos_t; a.sin_t = sin_t;
    a.rot_half = rot_half; a.interleaved = interleaved; a.q_out = (bf16*)q_out; a.k_cache = (bf16*)k_cache;
    a.v_cache = (bf16*)v_cache; a.positions = positions; a.token_req = token_req; a.req_slot = req_slot;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size; a.hq = hq; a.hkv = hkv; a.dim = dim;
    cudaStream_t s = (cudaStream_t)stream;
    if (m <= 8) return launch<1>(a, epilogue, s);
    if (m <= 16) return launch<2>(a, epilogue, s);
    if (m <= 32) return launch<4>(a, epilogue, s);
    return launch<8>(a, epilogue, s);
}
