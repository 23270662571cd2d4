// Causal grouped-query attention over the paged bfloat16 cache on the tensor cores
// (mma.sync m16n8k16, bf16 operands, float accumulation), for head sizes that are multiples
// of 16 up to 128.  Same entry points and argument lists as attention.cu, which remains the
// float path and the path for larger heads.
//
//   attn_prefill : one CTA (4 warps) per (64-query tile, query head).  K and V tiles of 64 keys
//                  are gathered page by page with cp.async into double-buffered shared memory;
//                  S = Q K^T and O += P V run on the tensor cores; the online softmax
//                  (runtime/reference.py:18-27, kernels/ops.cu:88-123 of the reference) stays
//                  in float registers.
//   attn_decode  : one CTA per (request, kv head, key range).  The query heads of the group are
//                  the rows of one 16-row tile; each of the 4 warps takes a 16-key slab of every
//                  64-key tile with its own running softmax, and the warps are merged by
//                  log-sum-exp at the end.  K/V tiles stream through a 3-stage cp.async pipeline.
//   attn_merge   : log-sum-exp merge of the key ranges in a fixed order (kernels/ops.cu:72-86).
//
// Scores are scaled by scale * log2(e) in float after the product and exponentials are base 2.
// Cache layout: [pages, kv_heads, page_size, HEAD_DIM].
#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16, at most 128>"
#endif
#if (HEAD_DIM % 16) || (HEAD_DIM > 128) || (HEAD_DIM < 16)
#error "the tensor-core attention takes HEAD_DIM in multiples of 16 from 16 to 128"
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int D = HEAD_DIM;
constexpr int KD = D / 16;      // k-steps of Q K^T
constexpr int ND = D / 8;       // n-tiles of the output
constexpr int BN = 64;          // keys per tile
constexpr int LDS = D + 8;      // shared-memory row stride in elements: ldmatrix rows fall into distinct banks
constexpr int CHUNKS = D / 8;   // 16-byte chunks per row
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
bool g_pdl = false;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x in one instruction (ex2.approx: 2 ulp, -inf -> 0); the probabilities are rounded to bfloat16 right after
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gather `rows` key (or value) rows starting at position k0 into a [BN][LDS] tile; rows at or beyond `limit`
// and rows whose page entry is -1 (a page the window has passed) are zero-filled.  `pages` holds the block
// table entries of the CTA's key range in shared memory, entry 0 being logical page `first_page`: looking a
// page up there costs nothing, while a lookup in global memory would sit in front of every copy.
template <int THREADS>
__device__ __forceinline__ void load_kv_tile(bf16* Kt, bf16* Vt, const bf16* __restrict__ k_cache,
                                             const bf16* __restrict__ v_cache, const int* pages, int first_page, int k0,
                                             int limit, int hkv, int kvh, int page_size, int tid) {
    for (int c = tid; c < BN * CHUNKS; c += THREADS) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const int kpos = k0 + r;
        const int page = kpos < limit ? pages[kpos / page_size - first_page] : -1;
        const bool ok = page >= 0;
        const size_t base = ok ? (((size_t)page * hkv + kvh) * page_size + kpos % page_size) * D + ch * 8 : 0;
        cp_async16(Kt + r * LDS + ch * 8, k_cache + base, ok);
        cp_async16(Vt + r * LDS + ch * 8, v_cache + base, ok);
    }
}

// ------------------------------------------------------------------ prefill
// NG warp groups of 4 warps share one 64-query tile: group g takes key tiles g, g + NG, ... with its own running
// softmax and its own double buffer, and the groups are merged by log-sum-exp at the end.  A causal prompt's last
// query tile has the longest key loop of the whole launch; splitting it over groups shortens that tail and puts
// more warps on each SM.
constexpr int BM = 64;
#ifndef PREFILL_GROUPS
#define PREFILL_GROUPS (HEAD_DIM <= 64 ? 4 : 2)
#endif
constexpr int NG = PREFILL_GROUPS;
constexpr int PREFILL_THREADS = 128 * NG;
constexpr size_t PREFILL_MERGE_BYTES = sizeof(float) * (size_t)(NG - 1) * BM * (D + 2);
#ifndef PREFILL_BUFS
#define PREFILL_BUFS 2
#endif
constexpr int NB = PREFILL_BUFS;       // key/value buffers per group: 2 overlaps a group's own loads with its math; 1 halves
                                       // the shared memory so two CTAs fit an SM and overlap each other instead
constexpr size_t PREFILL_PIPE_BYTES = sizeof(bf16) * (size_t)(NG * NB * 2 * BN * LDS);
constexpr size_t PREFILL_SMEM = ((sizeof(bf16) * (size_t)(BM * LDS) +
                                  (PREFILL_PIPE_BYTES > PREFILL_MERGE_BYTES ? PREFILL_PIPE_BYTES : PREFILL_MERGE_BYTES) + 15) / 16) * 16;

__device__ __forceinline__ void group_sync(int group) { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }

__global__ void __launch_bounds__(PREFILL_THREADS)
attn_prefill_mma_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ k_cache,
                        const bf16* __restrict__ v_cache, const int* __restrict__ req_slot,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ tile_req,
                        const int* __restrict__ tile_q0, const int* __restrict__ q_start, const int* __restrict__ q_len,
                        const int* __restrict__ ctx_len, int hq, int hkv, int page_size, float scale, int window) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);   // [BM][LDS]
    bf16* pipe = Qs + BM * LDS;                     // [NG][2][K tile | V tile]
    float* merge = reinterpret_cast<float*>(pipe);  // reused after the loops: [NG - 1][BM][D + 2]
    int* pages = reinterpret_cast<int*>(smem_raw + PREFILL_SMEM);   // block table entries of this tile's key range

    const int tile = blockIdx.x, head = blockIdx.y;
    const int req = tile_req[tile], q0 = tile_q0[tile];
    const int rows = min(BM, q_len[req] - q0);
    const int tok0 = q_start[req] + q0;
    const int ctx = ctx_len[req];
    const int qpos0 = ctx - q_len[req] + q0;
    const int kvh = head / (hq / hkv);
    const int* table = block_table + (size_t)req_slot[req] * table_width;
    const int tid = threadIdx.x, lane = tid & 31;
    const int group = tid >> 7, gtid = tid & 127, warp = gtid >> 5;     // warp: which 16 query rows, within the group

    for (int c = tid; c < BM * CHUNKS; c += PREFILL_THREADS) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const bool ok = r < rows;
        cp_async16(Qs + r * LDS + ch * 8, q + ((size_t)(tok0 + (ok ? r : 0)) * hq + head) * D + ch * 8, ok);
    }
    cp_async_commit();
    const int k_end = qpos0 + rows;
    int k_first = 0;
    if (window > 0) k_first = max(0, qpos0 - window + 1);
    const int k_begin = (k_first / BN) * BN;
    const int n_tiles = (k_end - k_begin + BN - 1) / BN;
    const int first_page = k_begin / page_size;
    for (int i = tid; i <= (k_end - 1) / page_size - first_page; i += PREFILL_THREADS) pages[i] = table[first_page + i];
    cp_async_wait<0>();
    __syncthreads();                              // Q and the page entries are in shared memory

    uint32_t qf[KD][4];
#pragma unroll
    for (int kk = 0; kk < KD; ++kk)
        ldmatrix_x4(qf[kk], Qs + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
    float o[ND][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < ND; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    const float scale2 = scale * LOG2E;

    bf16* gbuf = pipe + (size_t)group * NB * 2 * BN * LDS;      // this group's [K tile | V tile] buffers
    if (group < n_tiles)
        load_kv_tile<128>(gbuf, gbuf + BN * LDS, k_cache, v_cache, pages, first_page, k_begin + group * BN, k_end, hkv, kvh,
                          page_size, gtid);
    cp_async_commit();

    for (int t = group, it = 0; t < n_tiles; t += NG, ++it) {
        const int k0 = k_begin + t * BN;
        const int buf = NB == 2 ? (it & 1) : 0;
        cp_async_wait<0>();
        group_sync(group);                    // tile t has landed; the group is done with the other buffer
        if (NB == 2 && t + NG < n_tiles) {
            bf16* nb = gbuf + (buf ^ 1) * 2 * BN * LDS;
            load_kv_tile<128>(nb, nb + BN * LDS, k_cache, v_cache, pages, first_page, k0 + NG * BN, k_end, hkv, kvh, page_size,
                              gtid);          // keys from k_end on are masked for every row
        }
        cp_async_commit();
        const bf16* Kt = gbuf + buf * 2 * BN * LDS;
        const bf16* Vt = Kt + BN * LDS;

        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < KD; ++kk) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, Kt + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + kk * 16 + 8 * ((lane >> 3) & 1));
                mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
            }
        }

        // Mask only where a tile can be cut by the causal edge, the window's edge or the tile's row count; most
        // tiles of a long prompt lie wholly inside and skip the per-element test.
        const int warp_row0 = warp * 16;
        const bool inside = (k0 + BN - 1 <= qpos0 + warp_row0) && (warp_row0 + 15 < rows) &&
                            (window <= 0 || k0 + window > qpos0 + warp_row0 + 15);
        float tile_max[2] = {-INFINITY, -INFINITY};
        if (inside) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                tile_max[0] = fmaxf(tile_max[0], fmaxf(s[nt][0], s[nt][1]));
                tile_max[1] = fmaxf(tile_max[1], fmaxf(s[nt][2], s[nt][3]));
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = warp_row0 + (lane >> 2) + 8 * (e >> 1);
                    const int kpos = k0 + nt * 8 + 2 * (lane & 3) + (e & 1);
                    const int qpos = qpos0 + row;
                    const bool ok = (row < rows) && (kpos <= qpos) && (window <= 0 || kpos + window > qpos);
                    const float v = ok ? s[nt][e] : -INFINITY;
                    s[nt][e] = v;
                    tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                }
            }
        }
        // the running max is kept in scaled units (score * scale * log2 e); p = 2^(s * scale2 - m) is one fma and one ex2
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = tile_max[h];
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx * scale2);      // scale2 > 0, so the max commutes with the scaling
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[h] = fast_exp2(m_run[h] - m_use);
            m_run[h] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float p0 = fast_exp2(fmaf(s[nt][2 * h], scale2, -m_use)), p1 = fast_exp2(fmaf(s[nt][2 * h + 1], scale2, -m_use));
                s[nt][2 * h] = p0; s[nt][2 * h + 1] = p1;
                sum += p0 + p1;
            }
            l_run[h] = l_run[h] * alpha[h] + sum;   // per-thread part of the row sum; the quad is summed at the end
        }
#pragma unroll
        for (int i = 0; i < ND; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < ND / 2; ++dp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, Vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                mma_bf16(o[2 * dp], pa, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
            }
        }
        if (NB == 1 && t + NG < n_tiles) {
            group_sync(group);                // every warp of the group is done with the only buffer
            load_kv_tile<128>(gbuf, gbuf + BN * LDS, k_cache, v_cache, pages, first_page, k0 + NG * BN, k_end, hkv, kvh, page_size, gtid);
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {      // whole-row denominators
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();                   // every group is done with its buffers: they become the merge area

    // groups 1.. hand their (output, max, denominator) to group 0 through shared memory, thread to same-placed thread
    if (NG > 1 && group > 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float* dst = merge + ((size_t)(group - 1) * BM + warp * 16 + (lane >> 2) + 8 * h) * (D + 2);
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                dst[i * 8 + 2 * (lane & 3)] = o[i][2 * h];
                dst[i * 8 + 2 * (lane & 3) + 1] = o[i][2 * h + 1];
            }
            if ((lane & 3) == 0) { dst[D] = m_run[h]; dst[D + 1] = l_run[h]; }
        }
    }
    if (NG > 1) __syncthreads();
    if (group > 0) return;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + (lane >> 2) + 8 * h;
        float m = m_run[h], l = l_run[h];
#pragma unroll
        for (int g = 1; g < NG; ++g) m = fmaxf(m, merge[((size_t)(g - 1) * BM + row) * (D + 2) + D]);
        const float m_use = (m == -INFINITY) ? 0.f : m;
        const float w0 = exp2f(m_run[h] - m_use);
        l *= w0;
#pragma unroll
        for (int i = 0; i < ND; ++i) { o[i][2 * h] *= w0; o[i][2 * h + 1] *= w0; }
#pragma unroll
        for (int g = 1; g < NG; ++g) {
            const float* src = merge + ((size_t)(g - 1) * BM + row) * (D + 2);
            const float wg = exp2f(src[D] - m_use);     // a group without tiles has max -inf: weight 0
            l += wg * src[D + 1];
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                o[i][2 * h] += wg * src[i * 8 + 2 * (lane & 3)];
                o[i][2 * h + 1] += wg * src[i * 8 + 2 * (lane & 3) + 1];
            }
        }
        if (row < rows) {
            const float inv = 1.f / l;
            bf16* dst = out + ((size_t)(tok0 + row) * hq + head) * D + 2 * (lane & 3);
#pragma unroll
            for (int i = 0; i < ND; ++i)
                *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        }
    }
}

// ------------------------------------------------------------------ decode
constexpr int DEC_THREADS = 128;
#ifndef DEC_STAGES
#define DEC_STAGES 3
#endif
constexpr int STAGES = DEC_STAGES;   // key/value tiles in flight per CTA: enough bytes on the way to keep HBM busy
constexpr size_t DEC_TILE_BYTES = sizeof(bf16) * (size_t)(2 * BN * LDS);
constexpr size_t DEC_MERGE_BYTES = sizeof(float) * (size_t)(4 * 16 * (D + 2));
constexpr size_t DEC_PIPE_BYTES = STAGES * DEC_TILE_BYTES > DEC_MERGE_BYTES ? STAGES * DEC_TILE_BYTES : DEC_MERGE_BYTES;
constexpr size_t DEC_SMEM = ((sizeof(bf16) * (size_t)(16 * LDS) + DEC_PIPE_BYTES + 15) / 16) * 16;

__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                       const int* __restrict__ req_slot, const int* __restrict__ block_table, int table_width,
                       const int* __restrict__ dec_req, const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                       float* __restrict__ partial, float* __restrict__ stats, int hq, int hkv, int page_size,
                       float scale, int window, int split_size, int n_splits, int row0) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                    // [16][LDS]
    bf16* pipe = Qs + 16 * LDS;                                      // [STAGES][K tile | V tile]
    float* merge = reinterpret_cast<float*>(pipe);                   // reused after the loop: [4][16][D + 2]
    int* pages = reinterpret_cast<int*>(smem_raw + DEC_SMEM);        // block table entries of this CTA's key range

    // Under programmatic dependent launch everything up to pdl_wait() overlaps the kernel before this one (the q/k/v
    // projection of the same layer).  That kernel writes only this step's token: the query, and the key and value at
    // position ctx - 1.  Request metadata, block tables and all older keys and values are safe to read before the wait.
    pdl_trigger();
    const int group = hq / hkv;
    const int rows = min(16, group - row0);                          // query heads of the group handled by this launch
    const int slot = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int req = dec_req[slot];
    const int tok = q_start[req];
    const int ctx = ctx_len[req];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int* table = block_table + (size_t)req_slot[req] * table_width;

    int lo = split * split_size;
    const int hi = min(lo + split_size, ctx);
    if (window > 0) lo = max(lo, ctx - window);
    const size_t part_base = ((size_t)slot * hq + (size_t)kvh * group + row0) * n_splits;
    if (lo >= hi) {      // nothing in this range (the same for every thread): the merge skips a zero denominator
        pdl_wait();
        for (int g = tid; g < rows; g += DEC_THREADS) {
            const size_t p = part_base + (size_t)g * n_splits + split;
            stats[2 * p] = -INFINITY; stats[2 * p + 1] = 0.f;
        }
        return;
    }
    const int n_tiles = (hi - lo + BN - 1) / BN;
    const int first_page = lo / page_size;
    for (int i = tid; i <= (hi - 1) / page_size - first_page; i += DEC_THREADS) pages[i] = table[first_page + i];
    __syncthreads();
    // the first tiles can start early unless they hold the newest key
    const bool early = !(hi == ctx && ctx - 1 < lo + (STAGES - 1) * BN);
    if (early) {
#pragma unroll
        for (int st = 0; st < STAGES - 1; ++st) {
            if (st < n_tiles) {
                bf16* Kt = pipe + st * 2 * BN * LDS;
                load_kv_tile<DEC_THREADS>(Kt, Kt + BN * LDS, k_cache, v_cache, pages, first_page, lo + st * BN, hi, hkv, kvh, page_size, tid);
            }
            cp_async_commit();
        }
    }
    pdl_wait();
    for (int c = tid; c < 16 * CHUNKS; c += DEC_THREADS) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const bool ok = r < rows;
        cp_async16(Qs + r * LDS + ch * 8, q + ((size_t)tok * hq + kvh * group + row0 + (ok ? r : 0)) * D + ch * 8, ok);
    }
    if (early) {
        cp_async_commit();           // the query is a group of its own, behind the early tiles
    } else {
#pragma unroll
        for (int st = 0; st < STAGES - 1; ++st) {
            if (st < n_tiles) {
                bf16* Kt = pipe + st * 2 * BN * LDS;
                load_kv_tile<DEC_THREADS>(Kt, Kt + BN * LDS, k_cache, v_cache, pages, first_page, lo + st * BN, hi, hkv, kvh, page_size, tid);
            }
            cp_async_commit();       // the query travels in the first tile's group
        }
    }

    uint32_t qf[KD][4];
    float o[ND][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < ND; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    const float scale2 = scale * LOG2E;

    for (int t = 0; t < n_tiles; ++t) {
        if (t == 0 && early) cp_async_wait<0>();       // the early tiles and the query, all issued long ago
        else cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nt = t + STAGES - 1;
            if (nt < n_tiles) {
                bf16* Kt = pipe + (nt % STAGES) * 2 * BN * LDS;
                load_kv_tile<DEC_THREADS>(Kt, Kt + BN * LDS, k_cache, v_cache, pages, first_page, lo + nt * BN, hi, hkv, kvh, page_size, tid);
            }
            cp_async_commit();
        }
        if (t == 0) {
#pragma unroll
            for (int kk = 0; kk < KD; ++kk)
                ldmatrix_x4(qf[kk], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
        }
        const bf16* Kt = pipe + (t % STAGES) * 2 * BN * LDS;
        const bf16* Vt = Kt + BN * LDS;
        const int k0 = lo + t * BN + warp * 16;        // this warp's 16-key slab of the tile

        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int kk = 0; kk < KD; ++kk) {
            uint32_t b[4];
            ldmatrix_x4(b, Kt + (warp * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + kk * 16 + 8 * ((lane >> 3) & 1));
            mma_bf16(s[0], qf[kk], b[0], b[1]);
            mma_bf16(s[1], qf[kk], b[2], b[3]);
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kpos = k0 + nt * 8 + 2 * (lane & 3) + (e & 1);
                const float v = kpos < hi ? s[nt][e] * scale2 : -INFINITY;
                s[nt][e] = v;
                tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = tile_max[h];
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[h] = exp2f(m_run[h] - m_use);
            m_run[h] = m_new;
            const float p0 = exp2f(s[0][2 * h] - m_use), p1 = exp2f(s[0][2 * h + 1] - m_use);
            const float p2 = exp2f(s[1][2 * h] - m_use), p3 = exp2f(s[1][2 * h + 1] - m_use);
            s[0][2 * h] = p0; s[0][2 * h + 1] = p1; s[1][2 * h] = p2; s[1][2 * h + 1] = p3;
            l_run[h] = l_run[h] * alpha[h] + (p0 + p1 + p2 + p3);
        }
#pragma unroll
        for (int i = 0; i < ND; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]); pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]); pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < ND / 2; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, Vt + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
            mma_bf16(o[2 * dp], pa, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();          // every warp is done with the pipeline buffers: they become the merge area

    // per-warp results: merge[warp][row][0..D) = unnormalised output, [D] = running max (base 2), [D+1] = denominator
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = (lane >> 2) + 8 * h;
        float* dst = merge + ((size_t)warp * 16 + row) * (D + 2);
#pragma unroll
        for (int i = 0; i < ND; ++i) {
            dst[i * 8 + 2 * (lane & 3)] = o[i][2 * h];
            dst[i * 8 + 2 * (lane & 3) + 1] = o[i][2 * h + 1];
        }
        if ((lane & 3) == 0) { dst[D] = m_run[h]; dst[D + 1] = l; }
    }
    __syncthreads();
    for (int e = tid; e < rows * D; e += DEC_THREADS) {
        const int g = e / D, d = e - g * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, merge[((size_t)w * 16 + g) * (D + 2) + D]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = merge + ((size_t)w * 16 + g) * (D + 2);
            const float wgt = src[D] == -INFINITY ? 0.f : exp2f(src[D] - m);
            num = fmaf(wgt, src[d], num);
            den = fmaf(wgt, src[D + 1], den);
        }
        const size_t p = part_base + (size_t)g * n_splits + split;
        partial[p * D + d] = num;
        if (d == 0) { stats[2 * p] = m * LN2; stats[2 * p + 1] = den; }   // the merge kernel works in natural logarithms
    }
}

__global__ void attn_merge_kernel(const float* __restrict__ partial, const float* __restrict__ stats,
                                  bf16* __restrict__ out, const int* __restrict__ dec_req,
                                  const int* __restrict__ q_start, int hq, int n_splits) {
    pdl_trigger();
    const int slot = blockIdx.x, head = blockIdx.y;
    const size_t base = ((size_t)slot * hq + head) * n_splits;
    const int tok = q_start[dec_req[slot]];       // request metadata does not come from the kernel before
    pdl_wait();
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s)
        if (stats[2 * (base + s) + 1] > 0.f) m = fmaxf(m, stats[2 * (base + s)]);
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
        out[((size_t)tok * hq + head) * D + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);   // no keys: a padding row
    }
}
}  // namespace

CISR_EXPORT int cisr_attn_head_dim() { return D; }
CISR_EXPORT void cisr_attn_set_pdl(int on) { g_pdl = on != 0; }
CISR_EXPORT int cisr_attn_storage_bf16() { return 1; }
CISR_EXPORT int cisr_attn_prefill_tile() { return BM; }

CISR_EXPORT int cisr_attn_prefill(const void* q, void* out, const void* k_cache, const void* v_cache,
                                  const int* req_slot, const int* block_table, int table_width, const int* tile_req,
                                  const int* tile_q0, int n_tiles, const int* q_start, const int* q_len,
                                  const int* ctx_len, int hq, int hkv, int page_size, float scale, int window,
                                  void* stream) {
    if (n_tiles <= 0) return 0;
    if (hq % hkv) return -2;
    const size_t smem = PREFILL_SMEM + sizeof(int) * ((size_t)table_width + 4);    // a tile's key range spans at most the table
    if (smem > 220 * 1024) return -3;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    attn_prefill_mma_kernel<<<dim3(n_tiles, hq), PREFILL_THREADS, smem, (cudaStream_t)stream>>>(
        (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache, req_slot, block_table, table_width,
        tile_req, tile_q0, q_start, q_len, ctx_len, hq, hkv, page_size, scale, window);
    return launch_status();
}

CISR_EXPORT int cisr_attn_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                 const int* req_slot, const int* block_table, int table_width, const int* dec_req,
                                 int n_dec, const int* q_start, const int* ctx_len, float* partial, float* stats, int hq,
                                 int hkv, int page_size, float scale, int window, int split_size, int n_splits,
                                 void* stream) {
    if (n_dec <= 0) return 0;
    if (hq % hkv || split_size <= 0 || n_splits <= 0) return -2;
    const size_t smem = DEC_SMEM + sizeof(int) * ((size_t)split_size / page_size + 4);   // + the range's block table entries
    if (smem > 220 * 1024) return -3;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int group = hq / hkv;
    for (int row0 = 0; row0 < group; row0 += 16) {     // groups wider than one 16-row tile take several launches
        int status = launch_kernel(attn_decode_mma_kernel, dim3(n_dec, hkv, n_splits), dim3(DEC_THREADS), smem, s, g_pdl,
                                   (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, req_slot, block_table,
                                   table_width, dec_req, q_start, ctx_len, partial, stats, hq, hkv, page_size, scale,
                                   window, split_size, n_splits, row0);
        if (status) return status;
    }
    return launch_kernel(attn_merge_kernel, dim3(n_dec, hq), dim3(D < 128 ? 64 : 128), 0, s, g_pdl, (const float*)partial,
                         (const float*)stats, (bf16*)out, dec_req, q_start, hq, n_splits);
}
