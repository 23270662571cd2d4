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
#if HEAD_DIM % 64 == 0
#include "tma.cuh"
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
    CISR_TRACE_SCOPE(TRACE_ATTN_PREFILL);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);   // [BM][LDS]
    bf16* pipe = Qs + BM * LDS;                     // [NG][2][K tile | V tile]
    float* merge = reinterpret_cast<float*>(pipe);  // reused after the loops: [NG - 1][BM][D + 2]
    int* pages = reinterpret_cast<int*>(smem_raw + PREFILL_SMEM);   // block table entries of this tile's key range

    pdl_trigger();
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
    {   // the step's metadata and block tables are older than the kernel before this one: stage the pages ahead of the wait
        const int k_end_ = qpos0 + rows;
        const int k_begin_ = ((window > 0 ? max(0, qpos0 - window + 1) : 0) / BN) * BN;
        const int first_page_ = k_begin_ / page_size;
        for (int i = tid; i <= (k_end_ - 1) / page_size - first_page_; i += PREFILL_THREADS) pages[i] = table[first_page_ + i];
    }
    pdl_wait();          // the queries, and this step's keys and values, come from the kernel before
    CISR_TRACE_WAITED();

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

// Where 16-byte chunk `chunk` of key row `row` of a tile gathered by cp.async lies: rows LDS elements apart.
struct PaddedTile {
    const bf16* k; const bf16* v;
    __device__ __forceinline__ const void* k_at(int row, int chunk) const { return k + row * LDS + chunk * 8; }
    __device__ __forceinline__ const void* v_at(int row, int chunk) const { return v + row * LDS + chunk * 8; }
};
// A warp's share of one 64-key tile: its 16-key slab against the group's query rows, with the running softmax.
// k0 is the position of the slab's first key; keys outside [lo, hi) are masked.
template <typename Tile>
__device__ __forceinline__ void decode_slab(const Tile& tile, const uint32_t (&qf)[KD][4], float (&o)[ND][4], float (&m_run)[2],
                                            float (&l_run)[2], int k0, int lo, int hi, float scale2, int warp, int lane) {
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < KD; ++kk) {
        uint32_t b[4];
        ldmatrix_x4(b, tile.k_at(warp * 16 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
        mma_bf16(s[0], qf[kk], b[0], b[1]);
        mma_bf16(s[1], qf[kk], b[2], b[3]);
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kpos = k0 + nt * 8 + 2 * (lane & 3) + (e & 1);
            const float v = (kpos < hi && kpos >= lo) ? s[nt][e] * scale2 : -INFINITY;
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
        ldmatrix_x4_trans(b, tile.v_at(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dp * 2 + (lane >> 4)));
        mma_bf16(o[2 * dp], pa, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
    }
}

// Each warp's result into the merge area: merge[warp][row][0..D) = unnormalised output, [D] = running max (base 2),
// [D+1] = denominator.  `merge` is [4][16][D + 2] floats of shared memory that no warp still reads as a tile.
__device__ __forceinline__ void warps_to_merge_area(float* merge, const float (&o)[ND][4], const float (&m_run)[2],
                                                    const float (&l_run)[2], int warp, int lane, int rows) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = (lane >> 2) + 8 * h;
        if (row >= rows) continue;                // a padding row of the 16-row tile: nobody reads it
        float* dst = merge + ((size_t)warp * 16 + row) * (D + 2);
#pragma unroll
        for (int i = 0; i < ND; ++i) {
            dst[i * 8 + 2 * (lane & 3)] = o[i][2 * h];
            dst[i * 8 + 2 * (lane & 3) + 1] = o[i][2 * h + 1];
        }
        if ((lane & 3) == 0) { dst[D] = m_run[h]; dst[D + 1] = l; }
    }
}
// Element d of query row g of the CTA: the four warps' results merged by log-sum-exp, in a fixed order.
// Returns the numerator; m (base 2) and den are the row's running max and denominator.
__device__ __forceinline__ float merged_element(const float* merge, int g, int d, float& m, float& den) {
    m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, merge[((size_t)w * 16 + g) * (D + 2) + D]);
    float num = 0.f;
    den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float* src = merge + ((size_t)w * 16 + g) * (D + 2);
        const float wgt = src[D] == -INFINITY ? 0.f : exp2f(src[D] - m);
        num = fmaf(wgt, src[d], num);
        den = fmaf(wgt, src[D + 1], den);
    }
    return num;
}
// The CTA's result written as its key range's partial sum (the merge kernel works in natural logarithms).
__device__ __forceinline__ void decode_finish(float* merge, const float (&o)[ND][4], const float (&m_run)[2], const float (&l_run)[2],
                                              float* __restrict__ partial, float* __restrict__ stats, size_t part_base,
                                              int rows, int n_splits, int split, int tid) {
    warps_to_merge_area(merge, o, m_run, l_run, tid >> 5, tid & 31, rows);
    __syncthreads();
    for (int e = tid; e < rows * D; e += DEC_THREADS) {
        const int g = e / D, d = e - g * D;
        float m, den;
        const float num = merged_element(merge, g, d, m, den);
        const size_t p = part_base + (size_t)g * n_splits + split;
        partial[p * D + d] = num;
        if (d == 0) { stats[2 * p] = m * LN2; stats[2 * p + 1] = den; }
    }
}

__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                       const int* __restrict__ req_slot, const int* __restrict__ block_table, int table_width,
                       const int* __restrict__ dec_req, const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                       float* __restrict__ partial, float* __restrict__ stats, int hq, int hkv, int page_size,
                       float scale, int window, int split_size, int n_splits, int row0) {
    CISR_TRACE_SCOPE(TRACE_ATTN_DECODE_GATHER);
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
    CISR_TRACE_WAITED();
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
        decode_slab(PaddedTile{Kt, Kt + BN * LDS}, qf, o, m_run, l_run, lo + t * BN + warp * 16, lo, hi, scale2, warp, lane);
    }
    cp_async_wait<0>();
    __syncthreads();          // every warp is done with the pipeline buffers: they become the merge area
    decode_finish(merge, o, m_run, l_run, partial, stats, part_base, rows, n_splits, split, tid);
}

#if HEAD_DIM % 64 == 0
// ------------------------------------------------------------------ decode, tiles staged by tensor-map copies
// The same result with another division of the work.  Each of the four warps owns whole tiles of TK keys (tiles
// w, w + 4, ... of the CTA's key range) with its own running softmax, its own 16 KB stage of shared memory and its
// own mbarrier; it requests its next tile itself as soon as it is done with the current one, so the loop has no
// CTA-wide barrier, and the tile's independent score columns give the tensor cores work to overlap.  A tile arrives
// by cp.async.bulk.tensor: one copy per page (and per 64 columns), issued by the lanes of the owning warp, instead
// of a 16-byte cp.async per thread with its own address arithmetic.  Every warp requests its first tile before the
// wait on the previous kernel (older keys do not come from it).
//
// The cache is one 2-D tensor [pages * kv_heads * page_size, D] read in boxes of min(page_size, TK) rows by 64
// columns with the 128-byte swizzle; the page size must be a multiple of 8 that divides TK or is a multiple of it.
// A page the window has passed (table entry -1) is fetched from beyond the tensor, which TMA fills with zeros.
constexpr int NSUB = D / 64;
constexpr int TK = 4096 / D;                        // keys per tile: 64 or 32, so that a tile's keys are 8 KB
constexpr int TKT = TK / 8;                         // score n-tiles per tile
constexpr int SUB_BYTES = TK * 128;                 // one TK-key x 64-column sub-tile
constexpr int TMA_TILE_BYTES = 2 * NSUB * SUB_BYTES;                 // keys then values: 16 KB
static_assert(4 * (size_t)TMA_TILE_BYTES >= DEC_MERGE_BYTES, "the merge area reuses the warps' stages");
constexpr size_t TMA_SMEM_FIXED = 1024 /* alignment slack */ + 4 * (size_t)TMA_TILE_BYTES + sizeof(bf16) * 16 * LDS + 64;

__device__ __forceinline__ int swizzled(int row, int chunk) {      // byte offset of 16-byte chunk `chunk` of key row `row`
    return (chunk >> 3) * SUB_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// Thread-block clusters: the CTAs of one (request, kv head) that share a cluster exchange their partial sums through
// distributed shared memory, each CTA finishing a slice of the output columns, so a step whose key ranges fit one
// cluster (up to 16) needs no merge kernel and no round trip of the partial sums through global memory.  The
// cluster barrier is the hardware's (all CTAs of a cluster are resident together); every CTA reaches it on every path.
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t shared_of_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void store_cluster(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

#ifdef DEC_TRACE
// Development aid (not built into the engine's libraries): clock stamps of thread 0 of every CTA of the last launch.
__device__ unsigned long long g_trace[8192][10];
__device__ __forceinline__ void stamp(int i) {
    if (threadIdx.x == 0) {
        const int b = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        if (b < 8192) {
            g_trace[b][i] = clock64();
            if (i == 0 || i == 7) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); g_trace[b][8 + (i ? 1 : 0)] = t; }
        }
    }
}
#define STAMP(i) stamp(i)
#else
#define STAMP(i)
#endif

// cluster: CTAs per cluster along the key ranges (1: none).  n_parts = n_splits / cluster partial sums per query head
// remain; with one, the first CTA writes the finished rows to `out`, otherwise partial sums for the merge kernel.
// STAGES: tiles a warp has on the way at once (each in its own 16 KB stage).  With one, a warp whose share is two tiles
// (ranges of 256 keys at head size 128) requests the second only after the first is used; with two, both are requested
// before the wait on the kernel before, at twice the shared memory: for launches of no more CTAs than the device has
// SMs, where that memory is idle anyway.  The sums are the same either way.
template <int STAGES>
__global__ void __launch_bounds__(DEC_THREADS, STAGES == 1 ? 3 : 1)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ k_cache,
                       const bf16* __restrict__ v_cache, int cache_rows, const int* __restrict__ req_slot,
                       const int* __restrict__ block_table, int table_width, const int* __restrict__ dec_req,
                       const int* __restrict__ q_start, const int* __restrict__ ctx_len, float* __restrict__ partial,
                       float* __restrict__ stats, int hq, int hkv, int page_size, float scale, int window, int split_size,
                       int cluster, int n_parts, int row0, int* __restrict__ error) {
    CISR_TRACE_SCOPE(TRACE_ATTN_DECODE_TMA);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1024-byte aligned
    float* merge = reinterpret_cast<float*>(ring);                   // reused after the loop: [4][16][D + 2]
    bf16* Qs = reinterpret_cast<bf16*>(ring + 4 * STAGES * (size_t)TMA_TILE_BYTES);   // [16][LDS]
    uint64_t* full = reinterpret_cast<uint64_t*>(Qs + 16 * LDS);     // [4][STAGES]: a warp's tile has landed
    int* failed = reinterpret_cast<int*>(full + 4 * STAGES);
    float* gathered = reinterpret_cast<float*>(failed + 4);          // [cluster][rows][D / cluster + 2]: this CTA's share of the cluster's results

    STAMP(0);
    pdl_trigger();
    const int group = hq / hkv;
    const int rows = min(16, group - row0);
    int* pages = reinterpret_cast<int*>(gathered + (cluster > 1 ? (size_t)cluster * rows * ((D + cluster - 1) / cluster + 2) : 0));   // block table entries of the key range
    const int slot = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int req = dec_req[slot];
    const int tok = q_start[req];
    const int ctx = ctx_len[req];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int* table = block_table + (size_t)req_slot[req] * table_width;

    int lo = split * split_size;                                     // a multiple of TK (checked by the launcher)
    const int hi = min(lo + split_size, ctx);
    if (window > 0) lo = max(lo, ctx - window);
    const size_t part_base = ((size_t)slot * hq + (size_t)kvh * group + row0) * n_parts;
    const bool empty = lo >= hi;              // nothing in this range (the same for every thread)
    if (empty && cluster == 1) {              // the merge skips a zero denominator
        pdl_wait();
        for (int g = tid; g < rows; g += DEC_THREADS) {
            const size_t p = part_base + (size_t)g * n_parts + split;
            stats[2 * p] = -INFINITY; stats[2 * p + 1] = 0.f;
        }
        return;
    }
    float o[ND][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < ND; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    if (tid == 0) *failed = 0;

    if (!empty) {
    const int base = lo & ~(TK - 1);          // tiles start on multiples of TK keys, so a tile is whole pages (or part of one)
    const int n_tiles = (hi - base + TK - 1) / TK;
    const int first_page = base / page_size;
    for (int i = tid; i <= (hi - 1) / page_size - first_page; i += DEC_THREADS) pages[i] = table[first_page + i];
    if (tid == 0) {
        for (int w = 0; w < 4 * STAGES; ++w) mbar_init(full + w, 1);
        mbar_init_fence();
    }
    __syncthreads();
    STAMP(1);

    // Tile t into this warp's stage: lane b fetches box b (K or V, 64-column half, run of box_rows keys).
    const int box_rows = min(page_size, TK), boxes = TK / box_rows;
    auto fetch = [&](int t, int slot) {
        unsigned char* stage = ring + (size_t)(warp * STAGES + slot) * TMA_TILE_BYTES;
        uint64_t* bar = full + warp * STAGES + slot;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)TMA_TILE_BYTES);
        __syncwarp();
        for (int b = lane; b < 2 * NSUB * boxes; b += 32) {
            const int i = b % boxes, sub = (b / boxes) % NSUB, is_v = b / (boxes * NSUB);
            const int kpos = base + t * TK + i * box_rows;
            const int page = kpos < hi ? pages[kpos / page_size - first_page] : -1;
            const int row = page < 0 ? cache_rows : (page * hkv + kvh) * page_size + kpos % page_size;
            tma_load_2d(stage + (is_v * NSUB + sub) * SUB_BYTES + i * box_rows * 128, is_v ? &map_v : &map_k, sub * 64, row, bar);
        }
    };
    // Older keys do not come from the kernel before this one, only the newest (position ctx - 1) does.  Every warp's
    // first tile is requested now; in the tile that holds the newest key that one row arrives stale and is fetched
    // again, by ordinary loads, once the kernel before has finished.
    const int newest = hi == ctx ? n_tiles - 1 : -1;
#pragma unroll
    for (int i = 0; i < STAGES; ++i)
        if (warp + 4 * i < n_tiles) fetch(warp + 4 * i, i);
    const bool newest_early = newest >= 0 && newest / 4 < STAGES;    // the newest key's tile was requested before the wait
    STAMP(2);
    pdl_wait();
    CISR_TRACE_WAITED();
    STAMP(3);
    uint4 newest_k = make_uint4(0, 0, 0, 0), newest_v = newest_k;
    if (newest_early && warp == (newest & 3) && lane < NSUB * 8) {
        const int pos = ctx - 1, page = pages[pos / page_size - first_page];
        if (page >= 0) {
            const size_t at = (((size_t)page * hkv + kvh) * page_size + pos % page_size) * D + lane * 8;
            newest_k = __ldcg(reinterpret_cast<const uint4*>(k_cache + at));     // from L2: no stale line of an earlier step
            newest_v = __ldcg(reinterpret_cast<const uint4*>(v_cache + at));
        }
    }
    for (int c = tid; c < 16 * CHUNKS; c += DEC_THREADS) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const bool ok = r < rows;
        cp_async16(Qs + r * LDS + ch * 8, q + ((size_t)tok * hq + kvh * group + row0 + (ok ? r : 0)) * D + ch * 8, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();                                                 // the query rows are in shared memory
    STAMP(4);
    CISR_TRACE_MARK(0);

    uint32_t qf[KD][4];
#pragma unroll
    for (int kk = 0; kk < KD; ++kk)
        ldmatrix_x4(qf[kk], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
    const float scale2 = scale * LOG2E;

    for (int t = warp, it = 0; t < n_tiles; t += 4, ++it) {
        const int slot = it % STAGES;
        const uint32_t parity = (uint32_t)(it / STAGES) & 1;
        unsigned char* stage = ring + (size_t)(warp * STAGES + slot) * TMA_TILE_BYTES;
        uint64_t* bar = full + warp * STAGES + slot;
        const unsigned char* Ks = stage;
        unsigned char* Vs = stage + NSUB * SUB_BYTES;
        if (!__all_sync(0xffffffffu, mbar_wait(bar, parity))) {      // the lanes agree on whether the wait ran out
            if (lane == 0) { atomicExch(error, 3); *failed = 1; }
            mbar_wait(bar, parity);      // one more bounded chance for the copy to land before the stage is given up
            break;
        }
        if (it == 0) { STAMP(5); CISR_TRACE_MARK(1); }
        const int k0 = base + t * TK;
        if (newest_early && t == newest) {        // the newest key's row over the stale one the early copy brought
            if (lane < NSUB * 8) {
                const int r = ctx - 1 - k0;
                *reinterpret_cast<uint4*>(stage + swizzled(r, lane)) = newest_k;
                *reinterpret_cast<uint4*>(Vs + swizzled(r, lane)) = newest_v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }
        if (k0 + TK > hi) {
            // Value rows beyond the newest key were never written, or are left over from another request: whatever
            // they hold must not meet the zero probabilities of those keys (0 * NaN).
            for (int e = lane; e < TK * NSUB * 8; e += 32) {
                const int r = e / (NSUB * 8), c = e - r * (NSUB * 8);
                if (k0 + r >= hi) *reinterpret_cast<uint4*>(Vs + swizzled(r, c)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // ordered before a tensor-map copy that refills the stage
            __syncwarp();
        }
        float s[TKT][4];
#pragma unroll
        for (int nt = 0; nt < TKT; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < KD; ++kk) {
#pragma unroll
            for (int np = 0; np < TKT / 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, Ks + swizzled(np * 16 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
            }
        }
        const bool edge = k0 < lo || k0 + TK > hi;                   // the same for the whole warp
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < TKT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nt][e] * scale2;
                if (edge) {
                    const int kpos = k0 + nt * 8 + 2 * (lane & 3) + (e & 1);
                    if (kpos >= hi || kpos < lo) v = -INFINITY;
                }
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
            alpha[h] = fast_exp2(m_run[h] - m_use);
            m_run[h] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < TKT; ++nt) {
                const float p0 = fast_exp2(s[nt][2 * h] - m_use), p1 = fast_exp2(s[nt][2 * h + 1] - m_use);
                s[nt][2 * h] = p0; s[nt][2 * h + 1] = p1;
                sum += p0 + p1;
            }
            l_run[h] = l_run[h] * alpha[h] + sum;
        }
#pragma unroll
        for (int i = 0; i < ND; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
#pragma unroll
        for (int j = 0; j < TK / 16; ++j) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * j][0], s[2 * j][1]); pa[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
            pa[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]); pa[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
            for (int dp = 0; dp < ND / 2; ++dp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, Vs + swizzled(j * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dp * 2 + (lane >> 4)));
                mma_bf16(o[2 * dp], pa, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();                                                // every lane has read the stage
        if (t + 4 * STAGES < n_tiles) fetch(t + 4 * STAGES, slot);
    }
    } else {
        pdl_wait();
    }
    __syncthreads();          // every warp is done with its stage: the stages become the merge area
    STAMP(6);
    CISR_TRACE_MARK(2);
    if (cluster == 1) {
        if (*failed) return;  // a copy never arrived; the host reads the error flag
        decode_finish(merge, o, m_run, l_run, partial, stats, part_base, rows, n_parts, split, tid);
        STAMP(7);
        return;
    }

    // All-to-all over the cluster: CTA r finishes output columns [r * cols, (r + 1) * cols) of every query row, so each
    // CTA sends every other CTA that slice of its rows (and the rows' max and denominator).  A CTA without keys, or
    // one that gave up, sends a zero weight.  Layout in the receiver: [sender][row][cols + 2].
    const bool have = !empty && !*failed;
    if (have) warps_to_merge_area(merge, o, m_run, l_run, warp, lane, rows);
    __syncthreads();
    const uint32_t rank = cluster_rank();
    const int cols = (D + cluster - 1) / cluster, stride = cols + 2;
    const uint32_t mine = smem_u32(gathered) + (uint32_t)(rank * rows * stride * sizeof(float));   // this sender's block, in any receiver
    for (int e = tid; e < rows * D; e += DEC_THREADS) {
        const int g = e / D, d = e - g * D;
        float m = -INFINITY, den = 0.f, num = 0.f;
        if (have) num = merged_element(merge, g, d, m, den);
        const int dest = d / cols, c = d - dest * cols;
        const uint32_t there = shared_of_rank(mine, (uint32_t)dest) + (uint32_t)((g * stride + c) * sizeof(float));
        store_cluster(there, num);
        if (c == 0) {
            store_cluster(there + (uint32_t)(cols * sizeof(float)), m);
            store_cluster(there + (uint32_t)((cols + 1) * sizeof(float)), den);
        }
    }
    cluster_barrier();
    const int part = split / cluster;
    for (int e = tid; e < rows * cols; e += DEC_THREADS) {
        const int g = e / cols, c = e - g * cols, d = (int)rank * cols + c;
        if (d >= D) continue;
        float m = -INFINITY;
        for (int r = 0; r < cluster; ++r) m = fmaxf(m, gathered[((size_t)r * rows + g) * stride + cols]);
        float num = 0.f, den = 0.f;
        for (int r = 0; r < cluster; ++r) {              // in the order of the key ranges
            const float* src = gathered + ((size_t)r * rows + g) * stride;
            const float wgt = src[cols] == -INFINITY ? 0.f : exp2f(src[cols] - m);
            num = fmaf(wgt, src[c], num);
            den = fmaf(wgt, src[cols + 1], den);
        }
        if (n_parts == 1) {
            out[((size_t)tok * hq + kvh * group + row0 + g) * D + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
        } else {
            const size_t p = part_base + (size_t)g * n_parts + part;
            partial[p * D + d] = num;
            if (d == 0) { stats[2 * p] = m * LN2; stats[2 * p + 1] = den; }
        }
    }
}
#endif

// Log-sum-exp merge of the key ranges.  A thread owns one output dimension; it requests the first sixteen ranges'
// partial sums at once, together with the ranges' statistics, so the kernel is one trip to memory deep; the weights
// are computed once into shared memory and the sum runs over the ranges in their fixed order.
__global__ void attn_merge_kernel(const float* __restrict__ partial, const float* __restrict__ stats,
                                  bf16* __restrict__ out, const int* __restrict__ dec_req,
                                  const int* __restrict__ q_start, int hq, int n_splits) {
    CISR_TRACE_SCOPE(TRACE_ATTN_MERGE);
    extern __shared__ float weights[];            // [n_splits] weights, then [n_splits] weighted denominators
    __shared__ float scratch[32];
    pdl_trigger();
    const int slot = blockIdx.x, head = blockIdx.y;
    const size_t base = ((size_t)slot * hq + head) * n_splits;
    const int tok = q_start[dec_req[slot]];       // request metadata does not come from the kernel before
    pdl_wait();
    CISR_TRACE_WAITED();
    const int d = threadIdx.x;                    // blockDim.x >= D: threads beyond D only help with the statistics
    float first[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) first[j] = (d < D && j < n_splits) ? partial[(base + j) * D + d] : 0.f;
    float m = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {
        const float2 ml = reinterpret_cast<const float2*>(stats)[base + s];
        weights[s] = ml.x; weights[n_splits + s] = ml.y;
        if (ml.y > 0.f) m = fmaxf(m, ml.x);
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
    __syncthreads();
    CISR_TRACE_MARK(0);
    m = -INFINITY;
    for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w) m = fmaxf(m, scratch[w]);
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {          // the thread that stored them
        const float l = weights[n_splits + s];
        const float w = l > 0.f ? expf(weights[s] - m) : 0.f;           // a range without keys weighs nothing
        weights[s] = w;
        weights[n_splits + s] = l > 0.f ? w * l : 0.f;
    }
    __syncthreads();
    CISR_TRACE_MARK(1);
    if (d >= D) return;
    float den = 0.f, num = 0.f;                   // every thread sums in the same order: the same denominator in all
    for (int s = 0; s < n_splits; ++s) den += weights[n_splits + s];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float w = j < n_splits ? weights[j] : 0.f;
        num = fmaf(w, w > 0.f ? first[j] : 0.f, num);                   // what an empty range left there is not a number to use
    }
    for (int s0 = 16; s0 < n_splits; s0 += 16) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = s0 + j < n_splits ? partial[(base + s0 + j) * D + d] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float w = s0 + j < n_splits ? weights[s0 + j] : 0.f;
            num = fmaf(w, w > 0.f ? v[j] : 0.f, num);
        }
    }
    out[((size_t)tok * hq + head) * D + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);   // no keys: a padding row
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
    return launch_kernel(attn_prefill_mma_kernel, dim3(n_tiles, hq), dim3(PREFILL_THREADS), smem, (cudaStream_t)stream, g_pdl,
                         (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache, req_slot, block_table,
                         table_width, tile_req, tile_q0, q_start, q_len, ctx_len, hq, hkv, page_size, scale, window);
}

CISR_EXPORT int cisr_attn_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                 const int* req_slot, const int* block_table, int table_width, const int* dec_req,
                                 int n_dec, const int* q_start, const int* ctx_len, float* partial, float* stats, int hq,
                                 int hkv, int page_size, float scale, int window, int split_size, int n_splits,
                                 int merge, void* stream) {
    // merge == 0: the ranges' partial sums and statistics are left in `partial` and `stats` for the caller's own merge
    // (merge_proj.cu merges them in the prologue of the output projection); `out` is then not written.
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
    if (!merge) return 0;
    return launch_kernel(attn_merge_kernel, dim3(n_dec, hq), dim3(D <= 64 ? 64 : 128), sizeof(float) * 2 * (size_t)n_splits, s, g_pdl,
                         (const float*)partial, (const float*)stats, (bf16*)out, dec_req, q_start, hq, n_splits);
}

// 1 when this library has the variant that stages tiles by tensor-map copies, and it takes this page and range size.
CISR_EXPORT int cisr_attn_decode_tma_ok(int page_size, int split_size) {
#if HEAD_DIM % 64 == 0
    return page_size > 0 && page_size % 8 == 0 && (TK % page_size == 0 || page_size % TK == 0) && split_size > 0 &&
           split_size % TK == 0;
#else
    return 0;
#endif
}

#if HEAD_DIM % 64 == 0
namespace { int* g_error = nullptr; bool g_clusters = false; int g_last_launches = 0; }

// `error_flag`: one zeroed int in device memory that a kernel sets when a wait on a copy ran out.
CISR_EXPORT int cisr_attn_tma_init(int* error_flag) {
    if (int status = tma_load_encoder()) return status;
    g_error = error_flag;
    return 0;
}

// As cisr_attn_decode, for caches of `n_pages` pages whose address is 16-byte aligned.  Key ranges are grouped into
// thread-block clusters of up to 16 where the device can hold such clusters; when one cluster covers all ranges
// the finished rows go straight to `out` and no merge kernel runs.
CISR_EXPORT int cisr_attn_decode_tma(const void* q, void* out, const void* k_cache, const void* v_cache, int n_pages,
                                     const int* req_slot, const int* block_table, int table_width, const int* dec_req,
                                     int n_dec, const int* q_start, const int* ctx_len, float* partial, float* stats,
                                     int hq, int hkv, int page_size, float scale, int window, int split_size,
                                     int n_splits, int merge, void* stream) {
    if (n_dec <= 0) return 0;
    if (!g_encode || !g_error) return -13;
    if (!merge && g_clusters) return -2;      // the caller's own merge needs every range's partial sum
    if (hq % hkv || n_splits <= 0 || !cisr_attn_decode_tma_ok(page_size, split_size)) return -2;
    const long long cache_rows = (long long)n_pages * hkv * page_size;
    if (cache_rows <= 0 || cache_rows >= (1ll << 31) || (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15)) return -2;
    const int box_rows = page_size < TK ? page_size : TK;
    CUtensorMap map_k, map_v;
    int status = cached_map(&map_k, k_cache, cache_rows, D, box_rows, 64);
    if (status) return status;
    if ((status = cached_map(&map_v, v_cache, cache_rows, D, box_rows, 64))) return status;
    const int group = hq / hkv, rows_max = group < 16 ? group : 16;
    const size_t smem_plain = TMA_SMEM_FIXED + sizeof(int) * ((size_t)split_size / page_size + 8);
    constexpr size_t SMEM_CAP = 110 * 1024;  // two CTAs per SM at the very least; the usual need is below 72 KB (three)
    constexpr size_t SMEM_CAP_DEEP = 200 * 1024;
    if (smem_plain > SMEM_CAP) return -3;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_CAP);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(attn_decode_tma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_CAP_DEEP);
        if (e != cudaSuccess) return (int)e;
        cudaFuncSetAttribute(attn_decode_tma_kernel<1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);   // clusters of more than 8
        cudaGetLastError();
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 0;
        configured = true;
    }
    // the largest cluster size that divides the number of ranges, fits shared memory and can be resident
    int cluster = 1;
    size_t smem = smem_plain;
    static int resident[17] = {};            // per cluster size: 0 unknown, 1 yes, -1 no (asked with the largest shared memory)
    for (int c = 16; c >= 2 && g_clusters; --c) {
        if (n_splits % c) continue;
        const size_t need = smem_plain + sizeof(float) * (size_t)c * rows_max * ((D + c - 1) / c + 2);
        if (need > SMEM_CAP) continue;
        if (!resident[c]) {
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(1, 1, c); config.blockDim = dim3(DEC_THREADS); config.dynamicSmemBytes = SMEM_CAP;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)c;
            config.attrs = attr; config.numAttrs = 1;
            int n = 0;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, attn_decode_tma_kernel<1>, &config);
            cudaGetLastError();
            resident[c] = (e == cudaSuccess && n >= 1) ? 1 : -1;
        }
        if (resident[c] < 0) continue;
        cluster = c;
        smem = need;
        break;
    }
    const int n_parts = n_splits / cluster;
    cudaStream_t s = (cudaStream_t)stream;
    g_last_launches = (group + 15) / 16 + (((n_parts == 1 && cluster > 1) || !merge) ? 0 : 1);
    // a warp's share of a range is more than one tile, and the launch leaves most of the device's shared memory idle
    const size_t smem_deep = smem + 4 * (size_t)TMA_TILE_BYTES;
    const bool deep = cluster == 1 && split_size > 4 * TK && (long long)n_dec * hkv * n_splits <= sms && smem_deep <= SMEM_CAP_DEEP;
    for (int row0 = 0; row0 < group; row0 += 16) {
        if (deep)
            status = launch_kernel_cluster(attn_decode_tma_kernel<2>, dim3(n_dec, hkv, n_splits), dim3(DEC_THREADS), smem_deep, s, g_pdl, 1,
                                           map_k, map_v, (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,
                                           (int)cache_rows, req_slot, block_table, table_width,
                                           dec_req, q_start, ctx_len, partial, stats, hq, hkv, page_size, scale, window, split_size,
                                           1, n_parts, row0, g_error);
        else
            status = launch_kernel_cluster(attn_decode_tma_kernel<1>, dim3(n_dec, hkv, n_splits), dim3(DEC_THREADS), smem, s, g_pdl, cluster,
                                           map_k, map_v, (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,
                                           (int)cache_rows, req_slot, block_table, table_width,
                                           dec_req, q_start, ctx_len, partial, stats, hq, hkv, page_size, scale, window, split_size,
                                           cluster, n_parts, row0, g_error);
        if (status) return status;
    }
    if ((n_parts == 1 && cluster > 1) || !merge) return 0;
    return launch_kernel(attn_merge_kernel, dim3(n_dec, hq), dim3(D <= 64 ? 64 : 128), sizeof(float) * 2 * (size_t)n_parts, s, g_pdl,
                         (const float*)partial, (const float*)stats, (bf16*)out, dec_req, q_start, hq, n_parts);
}

#ifdef DEC_TRACE
CISR_EXPORT int cisr_attn_trace_read(void* host, int bytes) { return (int)cudaMemcpyFromSymbol(host, g_trace, (size_t)bytes); }
#endif

// Kernels launched by the last cisr_attn_decode_tma call (the merge kernel is left out when one cluster covers all ranges).
CISR_EXPORT int cisr_attn_decode_tma_launches() { return g_last_launches; }

// 0 turns the clusters off (every key range then writes its partial sum and the merge kernel runs).
CISR_EXPORT void cisr_attn_set_clusters(int on) { g_clusters = on != 0; }
#endif
