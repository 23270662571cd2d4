// Weight-streaming matrix product for steps with few tokens and large weight matrices (decode of wide models, and
// the vocabulary head of any model): out[M, N] = a[M, K] * w[N, K]^T, M <= 16, bfloat16 operands, float accumulation.
// The same prologues and epilogues as skinny_gemm.cu (activation or residual add + RMSNorm in; float out, SwiGLU,
// rotation + cache write out), built for bandwidth instead of latency:
//
//   * persistent: one CTA per SM walks "row blocks" (32, 64 or 128 weight rows by all of K); the tokens are staged
//     (and normalised) once per CTA, not once per 16 rows
//   * the weights stream through a ring of stages in shared memory, filled by tensor-map copies (cp.async.bulk.tensor,
//     128-byte swizzle).  Where K is whole 64-column groups the groups are one more dimension of the tensor map
//     ([64][rows][groups], strides {row, 128 bytes}) and a stage is ONE box: all the block's rows by sixteen k-slices'
//     worth of 32 KB (36 KB where nine groups are a whole block).  The copy engine's cost is per request: 4 KB boxes
//     stream at 2 TB/s, 16 KB boxes at 5 to 6, and a short launch gains again from 32 KB.  Otherwise a stage is
//     eight tiles of 16 rows x 64 k, fetched as one box per k-slice.
//     A producer warp keeps the ring full (up to 200 KB on the way per SM) and starts before the wait on the previous
//     kernel: weights do not depend on it
//   * eight consumer warps: warp w takes row tile w % RT of the block and the k-slices w / RT, w / RT + 8 / RT, ... of
//     every stage (RT = rows / 16), with ldmatrix for the weights (A operand of mma.sync.m16n8k16) and the tokens as the
//     8-wide N.  The k-slices of a row tile are added through shared memory in a fixed order, then the epilogue runs
//     while the producer already fetches the next block
//   * SWIGLU: a row tile is 8 gate rows and the 8 up rows of the same features (two 8-row boxes); ROPE: a block is the
//     matching slabs of a head's two halves, so a rotation pair never leaves its CTA
//
// Every wait on an mbarrier is bounded (tma.cuh); a warp whose wait ran out raises the CTA's abort flag and the
// device flag, every later wait is skipped, the barriers of the block structure are still reached, and the kernel
// returns without a result.
//
// Parity: the products that runtime/blas.py:41-56 of the reference hands to cuBLAS with M = batch, with the
// neighbours kernels/execution.cu:12-24 (residual + norm), :7-10 (SwiGLU), :28-40 (rotation and cache write) fused.
#include <stdlib.h>

#include "tma.cuh"

namespace {
typedef __nv_bfloat16 bf16;
enum : int { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_ROPE = 2 };
constexpr int CONSUMERS = 8;                      // consumer warps = boxes per stage
constexpr int THREADS = 32 * (CONSUMERS + 1);     // + the producer warp
constexpr int BOX_BYTES = 16 * 64 * 2;            // 16 rows x 64 k
constexpr int STAGE_BYTES = CONSUMERS * BOX_BYTES;
bool g_pdl = false;
int* g_error = nullptr;

struct StreamArgs {
    int n; int k;
    const bf16* act;                               // ACT prologue
    const float* x; const float* delta; const void* norm_w; int norm_w_bf16; float eps; float* x_out; const int* rows;
    int m; int block_rows; int n_blocks; int stages;
    float* out_f32; bf16* out_bf16; int inter;      // PLAIN / SWIGLU
    // ROPE
    const float* cos_t; const float* sin_t; int rot_half; int interleaved; bf16* q_out; bf16* k_cache; bf16* v_cache;
    const int* positions; const int* token_req; const int* req_slot; const int* block_table; int table_width; int page_size;
    int hq; int hkv; int dim;
    int accumulate;                                // PLAIN: out += product
    int grouped;                                   // the tensor map's last dimension counts 64-column groups: a stage is one box
    int stage_groups; int stage_bytes;             // k-slices (64 columns each) per stage, and the stage's size
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * CONSUMERS) : "memory"); }

// The token operand in shared memory: hs[m][ldh] bfloat16 (token columns >= m of the products read zeros instead).
// Consumer threads only.
__device__ void stage_tokens(const StreamArgs& a, bf16* hs, int ldh, int tid, float* scratch /* >= 8 floats */) {
    const int lane = tid & 31, warp = tid >> 5;
    const int k = a.k, k8 = k / 8;
    if (a.act) {
        for (int e = tid; e < a.m * k8; e += 32 * CONSUMERS) {
            const int r = e / k8, c = (e - r * k8) * 8;
            *reinterpret_cast<uint4*>(hs + r * ldh + c) = *reinterpret_cast<const uint4*>(a.act + (size_t)r * k + c);
        }
        return;
    }
    const int k4 = k / 4;
    constexpr int V = 8;                           // float4 per thread that the cooperative path keeps in registers
    if (a.m <= 2 && k4 <= V * 32 * CONSUMERS) {
        // One or two tokens (single-stream decode): all consumer warps share a row, every thread keeps its part of
        // x + delta in registers, so the row is one trip to memory deep instead of two passes by one warp.
        for (int r = 0; r < a.m; ++r) {
            const size_t src = (size_t)(a.rows ? a.rows[r] : r) * k;
            const float4* xr = reinterpret_cast<const float4*>(a.x + src);
            const float4* dr = a.delta ? reinterpret_cast<const float4*>(a.delta + src) : nullptr;
            float4 v[V];
            float sq = 0.f;
#pragma unroll
            for (int u = 0; u < V; ++u) {
                const int c = tid + u * 32 * CONSUMERS;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < k4) {
                    v[u] = xr[c];
                    if (dr) { const float4 d = dr[c]; v[u].x += d.x; v[u].y += d.y; v[u].z += d.z; v[u].w += d.w; }
                }
            }
#pragma unroll
            for (int u = 0; u < V; ++u) sq += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
            sq = warp_sum(sq);
            if (lane == 0) scratch[warp] = sq;
            consumer_sync();
            float total = 0.f;
            for (int w = 0; w < CONSUMERS; ++w) total += scratch[w];     // the same order in every thread
            consumer_sync();                      // scratch is free for the next row
            const float scale = rsqrtf(total / (float)k + a.eps);
            const bool write_x = a.x_out && blockIdx.x == 0;
            bf16* dst = hs + r * ldh;
#pragma unroll
            for (int u = 0; u < V; ++u) {
                const int c = tid + u * 32 * CONSUMERS;
                if (c >= k4) continue;
                if (write_x) reinterpret_cast<float4*>(a.x_out + src)[c] = v[u];
                float w0, w1, w2, w3;
                if (a.norm_w_bf16) {
                    const bf16* wp = (const bf16*)a.norm_w + 4 * c;
                    w0 = __bfloat162float(wp[0]); w1 = __bfloat162float(wp[1]); w2 = __bfloat162float(wp[2]); w3 = __bfloat162float(wp[3]);
                } else {
                    const float4 wv = reinterpret_cast<const float4*>(a.norm_w)[c];
                    w0 = wv.x; w1 = wv.y; w2 = wv.z; w3 = wv.w;
                }
                __nv_bfloat162 lo = __floats2bfloat162_rn(v[u].x * scale * w0, v[u].y * scale * w1);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v[u].z * scale * w2, v[u].w * scale * w3);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo); packed.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst + 4 * c) = packed;
            }
        }
        return;
    }
    for (int r = warp; r < a.m; r += CONSUMERS) {
        bf16* dst = hs + r * ldh;
        const size_t src = (size_t)(a.rows ? a.rows[r] : r) * k;
        const float4* xr = reinterpret_cast<const float4*>(a.x + src);
        const float4* dr = a.delta ? reinterpret_cast<const float4*>(a.delta + src) : nullptr;
        float sq = 0.f;
#pragma unroll 16
        for (int c = lane; c < k4; c += 32) {
            float4 v = xr[c];
            if (dr) { const float4 d = dr[c]; v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w; }
            sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        sq = warp_sum(sq);
        const float scale = rsqrtf(sq / (float)k + a.eps);
        const bool write_x = a.x_out && blockIdx.x == 0;
#pragma unroll 16
        for (int c = lane; c < k4; c += 32) {      // the second pass finds the row in L2; once per CTA, not per 16 rows
            float4 v = xr[c];
            if (dr) { const float4 d = dr[c]; v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w; }
            if (write_x) reinterpret_cast<float4*>(a.x_out + src)[c] = v;
            float w0, w1, w2, w3;
            if (a.norm_w_bf16) {
                const bf16* wp = (const bf16*)a.norm_w + 4 * c;
                w0 = __bfloat162float(wp[0]); w1 = __bfloat162float(wp[1]); w2 = __bfloat162float(wp[2]); w3 = __bfloat162float(wp[3]);
            } else {
                const float4 wv = reinterpret_cast<const float4*>(a.norm_w)[c];
                w0 = wv.x; w1 = wv.y; w2 = wv.z; w3 = wv.w;
            }
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale * w0, v.y * scale * w1);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * scale * w2, v.w * scale * w3);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo); packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst + 4 * c) = packed;
        }
    }
}

template <int MT, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
stream_kernel(const __grid_constant__ CUtensorMap map_w, const StreamArgs a, int* __restrict__ error) {
    CISR_TRACE_SCOPE(TRACE_STREAM_GEMM);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1024-byte aligned
    const int S = a.stages, ldh = a.k + 8;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)S * a.stage_bytes); // [S]: a stage's boxes have landed
    uint64_t* empty = full + S;                                                      // [S]: the consumers are done with it
    int* abort_flag = reinterpret_cast<int*>(empty + S);
    float* red = reinterpret_cast<float*>(abort_flag + 4);                           // [CONSUMERS][16][MT * 8]
    bf16* hs = reinterpret_cast<bf16*>(red + CONSUMERS * 16 * MT * 8);               // [m][ldh]
    float* tables = reinterpret_cast<float*>(hs + (size_t)a.m * ldh);                // ROPE: [2][m][rot_half] cos, sin
    __shared__ long long cache_row[MT * 8];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RT = a.block_rows / 16, KSUB = CONSUMERS / RT;      // row tiles of a block, k-slices of a stage
    const int k_boxes = (a.k + 63) / 64;
    const int SG = a.stage_groups;                                // k-slices of a stage: KSUB at a time, one per consumer warp
    const int k_stages = (k_boxes + SG - 1) / SG;                 // stages per block
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, CONSUMERS); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();
    pdl_trigger();

    if (warp == CONSUMERS) {
        // ------------------------------------------------------------ producer: keeps the ring full across blocks
        int it = 0;
        for (int block = blockIdx.x; block < a.n_blocks; block += gridDim.x) {
            for (int ks = 0; ks < k_stages; ++ks, ++it) {
                const int s = it % S;
                bool ok = true;
                if (it >= S && !*(volatile int*)abort_flag) ok = mbar_wait(empty + s, ((it / S) & 1) ^ 1);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) { atomicExch(error, 4); *(volatile int*)abort_flag = 1; }
                }
                if (*(volatile int*)abort_flag) continue;          // nothing more is requested; the loops still end
                unsigned char* stage = ring + (size_t)s * a.stage_bytes;
                if (lane == 0) mbar_expect_tx(full + s, (uint32_t)a.stage_bytes);
                __syncwarp();
                // One copy per k-slice: all row tiles of the block in one box.  Where a block's rows lie in two places
                // the tensor map has a dimension for that: [2 halves][inter rows][K] for the stacked gate and up
                // matrices, [heads][2 halves][D / 2 rows][K] for the stacked heads, and the box takes both halves.
                // Few large boxes keep the copy engine's per-request cost low.  A box beyond K or N is all zeros.
                if (a.grouped) {
                    // K in whole 64-column groups: the groups are one more dimension of the tensor map, and the stage's
                    // k-slices arrive as ONE box [k-slices][rows][64 columns] (the copy engine's cost is per request:
                    // a 16 KB box streams at nearly three times the rate of four 4 KB boxes)
                    if (lane == 0) {
                        const int half = a.block_rows / 2, g0 = ks * SG;
                        if (EPI == EPI_SWIGLU) {
                            tma_load_4d(stage, &map_w, 0, block * half, 0, g0, full + s);
                        } else if (EPI == EPI_ROPE) {
                            const int per_head = a.dim / a.block_rows, h = block / per_head, p = block - h * per_head;
                            tma_load_5d(stage, &map_w, 0, p * half, 0, h, g0, full + s);
                        } else {
                            tma_load_3d(stage, &map_w, 0, block * a.block_rows, g0, full + s);
                        }
                    }
                } else if (lane < KSUB) {
                    const int sub = lane, kc = (ks * KSUB + sub) * 64, half = a.block_rows / 2;
                    unsigned char* dst = stage + sub * a.block_rows * 128;
                    if (EPI == EPI_SWIGLU) {
                        tma_load_3d(dst, &map_w, kc, block * half, 0, full + s);
                    } else if (EPI == EPI_ROPE) {
                        const int per_head = a.dim / a.block_rows, h = block / per_head, p = block - h * per_head;
                        tma_load_4d(dst, &map_w, kc, p * half, 0, h, full + s);
                    } else {
                        tma_load_2d(dst, &map_w, kc, block * a.block_rows, full + s);
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    // ROPE: where each token's key and value go, and the rotation tables, come from the start of the step
    if (EPI == EPI_ROPE) {
        if (tid < a.m) {
            const int pos = a.positions[tid];
            const int page = a.block_table[(size_t)a.req_slot[a.token_req[tid]] * a.table_width + pos / a.page_size];
            cache_row[tid] = page < 0 ? -1 : (long long)page * a.hkv * a.page_size + pos % a.page_size;
        }
        const int n_rot = a.m * a.rot_half;
        for (int c = tid; c < n_rot; c += 32 * CONSUMERS) { tables[c] = a.cos_t[c]; tables[n_rot + c] = a.sin_t[c]; }
    }
    pdl_wait();
    CISR_TRACE_WAITED();
    stage_tokens(a, hs, ldh, tid, red);
    consumer_sync();
    CISR_TRACE_MARK(0);

    const int rt = warp % RT, sub = warp / RT;
    const int g = lane >> 2, t = lane & 3, mw = MT * 8;
    int it = 0;
    for (int block = blockIdx.x; block < a.n_blocks; block += gridDim.x) {
        float acc[MT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
        for (int ks = 0; ks < k_stages; ++ks, ++it) {
            const int s = it % S;
            bool ok = true;
            if (!*(volatile int*)abort_flag) ok = mbar_wait(full + s, (it / S) & 1);
            if (!__all_sync(0xffffffffu, ok)) {
                if (lane == 0) { atomicExch(error, 4); *(volatile int*)abort_flag = 1; }
            }
            if (*(volatile int*)abort_flag) continue;
            // the k-slice's region holds the block's rows in the order they were fetched: SWIGLU all gate rows then all
            // up rows (a tile's rows 0-7 and 8-15 lie half a region apart), otherwise tile after tile
            for (int slice = sub; slice < SG; slice += KSUB) {     // this warp's k-slices of the stage
            const unsigned char* region = ring + (size_t)s * a.stage_bytes + (size_t)slice * a.block_rows * 128;
            const int k0 = (ks * SG + slice) * 64;                 // beyond K: the box is zeros and so are the tokens read as 0
            if (k0 < a.k) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    uint32_t w4[4];
                    const int row = lane & 15, chunk = kk * 2 + (lane >> 4);
                    const int at = EPI == EPI_SWIGLU ? (row < 8 ? rt * 8 + row : a.block_rows / 2 + rt * 8 + row - 8) : rt * 16 + row;
                    ldmatrix_x4(w4, region + at * 128 + ((chunk ^ (row & 7)) << 4));
                    const int kb = k0 + kk * 16 + 2 * t;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint32_t b0 = 0, b1 = 0;
                        const bf16* tok = hs + (mt * 8 + g) * ldh + kb;
                        const bool row_ok = mt * 8 + g < a.m;
                        if (row_ok && kb < a.k) b0 = *reinterpret_cast<const uint32_t*>(tok);     // K is a multiple of 8: pairs are whole
                        if (row_ok && kb + 8 < a.k) b1 = *reinterpret_cast<const uint32_t*>(tok + 8);
                        mma_bf16(acc[mt], w4, b0, b1);
                    }
                }
            }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);
        }
        // this warp's k-slice of its row tile: red[warp][row][token]
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float* dst = red + ((size_t)warp * 16) * mw + mt * 8 + 2 * t;
            dst[g * mw] = acc[mt][0]; dst[g * mw + 1] = acc[mt][1];
            dst[(g + 8) * mw] = acc[mt][2]; dst[(g + 8) * mw + 1] = acc[mt][3];
        }
        consumer_sync();
        const bool usable = !*(volatile int*)abort_flag;
        // value of local row `lr` (row tile lr / 16) for token `mrow`: the k-slices in their fixed order
        auto summed = [&](int lr, int mrow) {
            const int tile = lr >> 4, r16 = lr & 15;
            float v = 0.f;
            for (int q = 0; q < KSUB; ++q) v += red[((size_t)(q * RT + tile) * 16 + r16) * mw + mrow];
            return v;
        };
        if (usable && EPI == EPI_PLAIN) {
            for (int e = tid; e < a.block_rows * a.m; e += 32 * CONSUMERS) {
                const int mrow = e / a.block_rows, lr = e - mrow * a.block_rows;
                const int f = block * a.block_rows + lr;
                if (f < a.n) {
                    float* dst = a.out_f32 + (size_t)mrow * a.n + f;
                    *dst = a.accumulate ? *dst + summed(lr, mrow) : summed(lr, mrow);
                }
            }
        } else if (usable && EPI == EPI_SWIGLU) {
            const int feats = a.block_rows / 2;                    // a row tile is 8 gate rows then their 8 up rows
            for (int e = tid; e < feats * a.m; e += 32 * CONSUMERS) {
                const int mrow = e / feats, lf = e - mrow * feats;
                const int f = block * feats + lf;
                if (f >= a.inter) continue;
                const int lr = (lf >> 3) * 16 + (lf & 7);
                const float gate = summed(lr, mrow), up = summed(lr + 8, mrow);
                a.out_bf16[(size_t)mrow * a.inter + f] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
            }
        } else if (usable) {
            const int per_head = a.dim / a.block_rows, hh = block / per_head, p = block - hh * per_head, half = a.block_rows / 2;
            const bool is_q = hh < a.hq, is_k = !is_q && hh < a.hq + a.hkv;
            for (int e = tid; e < a.m * a.block_rows; e += 32 * CONSUMERS) {
                const int mrow = e / a.block_rows, lr = e - mrow * a.block_rows;
                const bool low = lr < half;
                const int d = low ? p * half + lr : a.dim / 2 + p * half + (lr - half);     // position in the head
                float v = summed(lr, mrow);
                if (is_q || is_k) {
                    int f, other; bool first;
                    if (a.interleaved) { f = d >> 1; first = !(d & 1); other = first ? lr + 1 : lr - 1; }
                    else { first = low; f = first ? d : d - a.rot_half; other = first ? lr + half : lr - half; }
                    const float c = tables[mrow * a.rot_half + f], s = tables[a.m * a.rot_half + mrow * a.rot_half + f];
                    const float o = summed(other, mrow);
                    v = first ? v * c - o * s : v * c + o * s;
                }
                if (is_q) {
                    a.q_out[((size_t)mrow * a.hq + hh) * a.dim + d] = __float2bfloat16_rn(v);
                } else {
                    const long long at = cache_row[mrow];
                    if (at < 0) continue;                          // a padding row: its slot holds no pages
                    const int kvh = is_k ? hh - a.hq : hh - a.hq - a.hkv;
                    const size_t dst = ((size_t)at + (size_t)kvh * a.page_size) * a.dim + d;
                    (is_k ? a.k_cache : a.v_cache)[dst] = __float2bfloat16_rn(v);
                }
            }
        }
        consumer_sync();          // the sums are read: the next block may overwrite them
    }
}

// rows per block: the one that needs the fewest block-times (waves x rows); ties go to the larger block
// Number of row blocks: for SWIGLU a block of `rows` weight rows is rows / 2 features (their gate and up rows).
int count_blocks(const StreamArgs& a, int epilogue, int rows) {
    return epilogue == EPI_SWIGLU ? (a.inter + rows / 2 - 1) / (rows / 2) : (a.n + rows - 1) / rows;
}
int choose_block_rows(const StreamArgs& a, int sms, int epilogue) {
    int best = 0;
    long long best_cost = 0;
    for (int rows = 128; rows >= 32; rows /= 2) {
        if (epilogue == EPI_ROPE && (a.dim % rows)) continue;     // a block is a slab of one head
        const long long cost = (long long)((count_blocks(a, epilogue, rows) + sms - 1) / sms) * rows;
        if (!best || cost < best_cost) { best = rows; best_cost = cost; }
    }
    return best;
}

template <int MT, int EPI>
int launch(StreamArgs& a, const void* w, cudaStream_t s) {
    static int sms = 0;
    if (!sms) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    a.block_rows = choose_block_rows(a, sms, EPI);
    // tuning knobs for measurements: rows per block by epilogue, and (below) the depth of the ring
    if (const char* forced = getenv(EPI == EPI_SWIGLU ? "CISR_STREAM_ROWS_SWIGLU" : EPI == EPI_ROPE ? "CISR_STREAM_ROWS_ROPE" : "CISR_STREAM_ROWS")) {
        const int rows = atoi(forced);
        if ((rows == 32 || rows == 64 || rows == 128) && !(EPI == EPI_ROPE && (a.dim % rows))) a.block_rows = rows;
    }
    if (!a.block_rows) return -2;
    a.n_blocks = count_blocks(a, EPI, a.block_rows);
    const size_t fixed = 1024 /* alignment slack */ + 64 + sizeof(float) * CONSUMERS * 16 * MT * 8 +
                         sizeof(bf16) * (size_t)a.m * (a.k + 8) +
                         (EPI == EPI_ROPE ? sizeof(float) * 2 * (size_t)a.m * a.rot_half : 0);
    const size_t budget = 224 * 1024;
    // K in whole 64-column groups: a stage is one box of several k-slices per consumer warp, 32 KB (or 36 KB where that
    // is a whole block of nine groups): the copy engine's cost is per request, and short launches in particular
    // stream faster in few large requests.  Otherwise one box per k-slice and one k-slice per consumer warp: 16 KB.
    a.grouped = a.k % 64 == 0;
    const int ksub = CONSUMERS / (a.block_rows / 16), groups = (a.k + 63) / 64;
    a.stage_groups = ksub;
    if (a.grouped) {
        a.stage_groups = groups == 2 * ksub + 1 && a.block_rows == 32 ? groups : 2 * ksub;
        if (a.stage_groups > groups) a.stage_groups = groups > ksub ? groups : ksub;
    }
    a.stage_bytes = a.stage_groups * a.block_rows * 128;
    if (fixed + 3 * ((size_t)a.stage_bytes + 16) > budget) { a.stage_groups = ksub; a.stage_bytes = STAGE_BYTES; }
    if (fixed + 3 * ((size_t)a.stage_bytes + 16) > budget) return -2;       // rows too long for shared memory: not this kernel's
    a.stages = (int)((budget - fixed) / ((size_t)a.stage_bytes + 16));
    if (a.stages > 12) a.stages = 12;
    if (const char* forced = getenv("CISR_STREAM_STAGES")) { const int st = atoi(forced); if (st >= 2 && st < a.stages) a.stages = st; }
    const size_t smem = fixed + (size_t)a.stages * ((size_t)a.stage_bytes + 16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(stream_kernel<MT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap map_w;
    int status = 0;
        if (EPI == EPI_PLAIN && !a.grouped) {
        status = cached_map(&map_w, w, a.n, a.k, a.block_rows, 64);
    } else {
        // More dimensions than the matrix has: the 64-column groups of K as the last one (`grouped`), and where a block's
        // rows lie in two places one for the halves (see the producer)
        static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
        const MapKey key{w, a.n, a.k, a.block_rows, EPI + 16 * a.grouped + 64 * a.stage_groups};
        auto it = maps.find(key);
        if (it == maps.end()) {
            if (maps.size() > 4096) maps.clear();
            CUtensorMap map;
            const cuuint64_t row_bytes = (cuuint64_t)a.k * sizeof(bf16);
            const cuuint32_t half = (cuuint32_t)a.block_rows / 2;
            const cuuint64_t inner = a.grouped ? 64 : (cuuint64_t)a.k, groups = (cuuint64_t)a.k / 64;
            cuuint64_t dims[5], strides[4];
            cuuint32_t box[5];
            int rank;
            if (EPI == EPI_PLAIN) {
                dims[0] = inner; dims[1] = (cuuint64_t)a.n; strides[0] = row_bytes; box[0] = 64; box[1] = (cuuint32_t)a.block_rows;
                rank = 2;
            } else if (EPI == EPI_SWIGLU) {
                dims[0] = inner; dims[1] = (cuuint64_t)a.inter; dims[2] = 2;
                strides[0] = row_bytes; strides[1] = row_bytes * a.inter;
                box[0] = 64; box[1] = half; box[2] = 2;
                rank = 3;
            } else {
                dims[0] = inner; dims[1] = (cuuint64_t)a.dim / 2; dims[2] = 2; dims[3] = (cuuint64_t)(a.hq + 2 * a.hkv);
                strides[0] = row_bytes; strides[1] = row_bytes * (a.dim / 2); strides[2] = row_bytes * a.dim;
                box[0] = 64; box[1] = half; box[2] = 2; box[3] = 1;
                rank = 4;
            }
            if (a.grouped) { dims[rank] = groups; strides[rank - 1] = 128; box[rank] = (cuuint32_t)a.stage_groups; ++rank; }
            status = make_map_nd(&map, w, rank, dims, strides, box);
            if (!status) it = maps.emplace(key, map).first;
        }
        if (!status) map_w = it->second;
    }
    if (status) return status;
    const int grid = a.n_blocks < sms ? a.n_blocks : sms;
    return launch_kernel(stream_kernel<MT, EPI>, dim3(grid), dim3(THREADS), smem, s, g_pdl, map_w, a, g_error);
}

template <int MT>
int launch_any(StreamArgs& a, const void* w, int epilogue, cudaStream_t s) {
    if (epilogue == EPI_ROPE) return launch<MT, EPI_ROPE>(a, w, s);
    if (epilogue == EPI_SWIGLU) return launch<MT, EPI_SWIGLU>(a, w, s);
    return launch<MT, EPI_PLAIN>(a, w, s);
}
}  // namespace

CISR_EXPORT void cisr_stream_set_pdl(int on) { g_pdl = on != 0; }

// `error_flag`: one zeroed int in device memory that a kernel sets (to 4) when one of its waits ran out.
CISR_EXPORT int cisr_stream_init(int* error_flag) {
    if (int status = tma_load_encoder()) return status;
    g_error = error_flag;
    return 0;
}

// The argument list of cisr_skinny_gemm.  Returns -2 for shapes it does not take (more than 16 tokens, K not a
// multiple of 8, rows too long for shared memory, a rotation that does not pair d with d + dim / 2): the caller then
// uses the other kernels.
CISR_EXPORT int cisr_stream_gemm(const void* w, int n, int k, const void* act, const float* x, const float* delta,
                                 const void* norm_w, int norm_w_dtype, float eps, float* x_out, const int* rows, int m,
                                 int epilogue, float* out_f32, void* out_bf16, int inter, const float* cos_t,
                                 const float* sin_t, int rot_half, int interleaved, void* q_out, void* k_cache,
                                 void* v_cache, const int* positions, const int* token_req, const int* req_slot,
                                 const int* block_table, int table_width, int page_size, int hq, int hkv, int dim,
                                 int accumulate, void* stream) {
    if (m <= 0) return 0;
    if (!g_encode || !g_error) return -13;
    if (m > 16 || k % 8 || k <= 0 || n <= 0 || ((uintptr_t)w & 15)) return -2;
    if (epilogue == EPI_ROPE) {
        if (dim % 32 || dim > 256 || dim < 32 || n != (hq + 2 * hkv) * dim) return -2;
        if (2 * rot_half != dim) return -2;      // the whole head rotates: pairs (d, d + dim / 2), or neighbours when interleaved
    }
    if (epilogue == EPI_SWIGLU && (n != 2 * inter || inter % 8)) return -2;
    StreamArgs a;
    a.n = n; a.k = k; a.act = (const bf16*)act; a.x = x; a.delta = delta; a.norm_w = norm_w;
    a.norm_w_bf16 = norm_w_dtype == CISR_BF16; a.eps = eps; a.x_out = x_out; a.rows = rows; a.m = m;
    a.block_rows = 0; a.n_blocks = 0; a.stages = 0; a.accumulate = accumulate != 0 && epilogue == EPI_PLAIN;
    a.out_f32 = out_f32; a.out_bf16 = (bf16*)out_bf16; a.inter = inter; a.cos_t = cos_t; a.sin_t = sin_t;
    a.rot_half = rot_half; a.interleaved = interleaved; a.q_out = (bf16*)q_out; a.k_cache = (bf16*)k_cache;
    a.v_cache = (bf16*)v_cache; a.positions = positions; a.token_req = token_req; a.req_slot = req_slot;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size; a.hq = hq; a.hkv = hkv; a.dim = dim;
    cudaStream_t s = (cudaStream_t)stream;
    int status;
    if (m <= 8) status = launch_any<1>(a, w, epilogue, s);
    else status = launch_any<2>(a, w, epilogue, s);
    return status;
}
