// Decode steps: the log-sum-exp merge of the attention's key ranges and the output projection in ONE launch.
//
// The split decode attention leaves, per (request, query head, key range), an unnormalised partial output and its
// softmax statistics.  Merging them is a kernel of a few kilobytes, and the projection that follows reads the merged
// rows at once: as two launches they cost two trips through the launch chain and an extra trip through L2.  Here a
// thread-block cluster does both.  The cluster's CTAs split K by query heads: CTA c merges its own heads (it reads
// only their partial sums), multiplies them with its K-slice of the weights for the cluster's FT output features,
// and the K-slices are then summed through distributed shared memory, in the fixed order of the CTAs, each CTA
// finishing FT / C of the features.
//
//   grid (ceil(N / FT), 1, C), cluster (1, 1, C), 512 threads: all merge; warp w < 4 owns output features [16 w, 16 w + 16) of the tile
//   * before the wait on the attention kernel: the CTA's weights go to registers (mma.sync A fragments, as in
//     skinny_gemm.cu: lane (r, t) loads w[f0 + r][32 c + 8 t ..] and w[f0 + r + 8][..] with 16-byte loads)
//   * merge: exactly the arithmetic of attn_merge_kernel (attention_mma.cu): m = max of the ranges' maxima, weights
//     expf(m_s - m), denominator = the weights times the ranges' denominators added in range order, numerator by fmaf
//     in range order, the quotient rounded to bfloat16 once.  So a step gives the same bits through either path.
//   * products on mma.sync.m16n8k16 with the tokens as the 8-wide N (up to 16 tokens)
//   * every CTA sends its partial products of a feature to the CTA that finishes that feature (st.shared::cluster,
//     straight from the accumulator registers), one barrier.cluster, then CTA r adds the C contributions to its
//     FT / C features in the order c = 0 .. C - 1 from its own shared memory and writes float rows of `out`.
//     The cluster barrier is the hardware's: nothing here polls.
//
// Taken for steps made of single new tokens only, bfloat16, with up to 16 query-head slices of at most 256
// columns; everything else keeps the separate merge kernel and the weight-streaming products.
//
// Parity: kernels/ops.cu:72-86 (merge_attention) followed by the output projection of runtime/model.py:114-115.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int THREADS = 512;          // sixteen warps merge; the first four then own one 16-feature tile each
constexpr int FT = 64;                 // output features per CTA: one 16-row tile per warp
constexpr int MAX_SLICE = 256;         // K columns per CTA at most (the weights of a warp's tile stay in registers)
bool g_pdl = false;

struct MergeProjArgs {
    const float* partial; const float* stats; int n_splits;       // [n_dec, hq, n_splits, dim], [n_dec, hq, n_splits, 2]
    const int* dec_req; const int* q_start; int n_dec;            // row of request i's token: q_start[dec_req[i]]
    int hq; int dim; int heads_per_cta;
    const bf16* w; int n;                                          // [n, hq * dim]
    float* out;                                                    // [tokens, n]
    int accumulate;                                                // out += the product (out is the residual stream)
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 load_weights(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t smem_u32_of(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t shared_of_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void store_cluster(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One element (request, head, dimension) of the merged rows: both sums run over the ranges in their order, as in
// attn_merge_kernel.  FIRST_READY: the first SB ranges' partial sums are already in `first` (requested earlier).
constexpr int SB = 16;                 // ranges per batch of loads
template <bool FIRST_READY>
__device__ __forceinline__ void merge_element(const MergeProjArgs& a, int e, int heads, int head0, int ns, int nsp, int ldh,
                                              const float* wsm, bf16* hs, const float (&first)[SB]) {
    const int p = e / a.dim, d = e - p * a.dim, i = p / heads, hj = p - i * heads;
    const size_t base = ((size_t)i * a.hq + head0 + hj) * ns;
    const float4* wgt = reinterpret_cast<const float4*>(wsm + (size_t)p * 2 * nsp);
    float den = 0.f, num = 0.f;
    for (int s0 = 0; s0 < ns; s0 += SB) {
        float4 w4[SB / 4], wl4[SB / 4];
#pragma unroll
        for (int q = 0; q < SB / 4; ++q) {
            const bool in = s0 + 4 * q < nsp;
            w4[q] = in ? wgt[(s0 >> 2) + q] : make_float4(0.f, 0.f, 0.f, 0.f);
            wl4[q] = in ? wgt[(nsp >> 2) + (s0 >> 2) + q] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float v[SB];
        if (FIRST_READY && s0 == 0) {
#pragma unroll
            for (int sp = 0; sp < SB; ++sp) v[sp] = first[sp];
        } else {
#pragma unroll
            for (int sp = 0; sp < SB; ++sp) v[sp] = s0 + sp < ns ? a.partial[(base + s0 + sp) * a.dim + d] : 0.f;
        }
        const float* w = reinterpret_cast<const float*>(w4);
        const float* wl = reinterpret_cast<const float*>(wl4);
#pragma unroll
        for (int sp = 0; sp < SB; ++sp) {
            if (s0 + sp < ns) {
                den = __fadd_rn(den, wl[sp]);
                num = fmaf(w[sp], w[sp] > 0.f ? v[sp] : 0.f, num);   // what an empty range left there is not a number to use
            }
        }
    }
    hs[i * ldh + hj * a.dim + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);   // no keys: a padding row
}

// NCH: 32-column chunks of the CTA's K-slice (2, 4 or 8: the weights of a warp's tile are 4 * NCH registers)
template <int MT, int NCH>
__global__ void __launch_bounds__(THREADS) merge_proj_kernel(const MergeProjArgs a) {
    CISR_TRACE_SCOPE(TRACE_MERGE_PROJ);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, t = lane & 3;
    const int rank = (int)cluster_rank(), ranks = (int)cluster_size();
    const int slice = a.heads_per_cta * a.dim;                     // K columns of this CTA
    const int head0 = rank * a.heads_per_cta;
    const int heads = max(0, min(a.heads_per_cta, a.hq - head0));  // the last CTA may hold fewer
    const int cols = heads * a.dim;
    const int k = a.hq * a.dim, col0 = head0 * a.dim;
    const int ldh = slice + 8, mw = MT * 8, ns = a.n_splits, nsp = (ns + 3) & ~3;    // nsp: ranges padded to whole float4
    bf16* hs = reinterpret_cast<bf16*>(smem_raw);                  // [mw][ldh] merged rows, this CTA's columns
    float* part = reinterpret_cast<float*>(hs + mw * ldh);         // [ranks][per][mw] every CTA's partial products of this CTA's features
    float* raw = part + (FT + 16) * mw;                                   // [pairs][2 * nsp] the ranges' maxima, then their denominators
    float* wsm = raw + (size_t)a.n_dec * a.heads_per_cta * 2 * nsp; // [pairs][2 * nsp] merge weights, then weights * denominators
    const int chunks = (cols + 31) / 32;

    // weights of this warp's 16 features over the CTA's K-slice: nothing here depends on an earlier kernel
    const bool tile_warp = warp < FT / 16;                          // the warps that own a 16-feature tile
    const int f0 = blockIdx.x * FT + warp * 16;
    const bool ok_lo = tile_warp && f0 + r < a.n, ok_hi = tile_warp && f0 + r + 8 < a.n;
    const bf16* row_lo = a.w + (size_t)(ok_lo ? f0 + r : 0) * k + col0 + 8 * t;
    const bf16* row_hi = a.w + (size_t)(ok_hi ? f0 + r + 8 : 0) * k + col0 + 8 * t;
    uint4 wl[NCH], wh[NCH];
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const bool in_k = i < chunks && i * 32 + 8 * t < cols;
        wl[i] = make_uint4(0, 0, 0, 0); wh[i] = make_uint4(0, 0, 0, 0);
        if (in_k && ok_lo) wl[i] = load_weights(row_lo + i * 32);
        if (in_k && ok_hi) wh[i] = load_weights(row_hi + i * 32);
    }
    pdl_trigger();
    pdl_wait();
    CISR_TRACE_WAITED();

    // ---- merge.  One trip to memory deep: a thread first requests the partial sums of its first elements (the first
    // sixteen ranges of each), then the statistics are fetched and turned into weights, and by then the sums are there.
    // (One element per thread is requested ahead and the code stays short: a kernel this brief pays for every
    // instruction-cache line it touches.)
    const int pairs = a.n_dec * heads, total = pairs * a.dim;
    // adding into `out` (the residual stream): what the thread's first output element holds now is requested with them
    const int per_out = (FT + ranks - 1) / ranks;
    float* first_out = nullptr;
    float there = 0.f;
    if (a.accumulate && tid < per_out * a.n_dec) {
        const int fr = tid / a.n_dec, i = tid - fr * a.n_dec, row = rank * per_out + fr, f = blockIdx.x * FT + row;
        if (row < FT && f < a.n) { first_out = a.out + (size_t)a.q_start[a.dec_req[i]] * a.n + f; there = *first_out; }
    }
    float pre[SB];
    {
        const int e = tid;
        const int p = e / a.dim, d = e - p * a.dim, i = p / max(heads, 1);
        const size_t base = ((size_t)i * a.hq + head0 + (p - i * heads)) * ns;
#pragma unroll
        for (int sp = 0; sp < SB; ++sp) pre[sp] = (e < total && sp < ns) ? a.partial[(base + sp) * a.dim + d] : 0.f;
    }
    // rows beyond the step's tokens, and columns beyond this CTA's heads, are zero
    for (int e = tid; e < mw * (ldh / 8); e += THREADS) {
        const int row = e / (ldh / 8), c = (e - row * (ldh / 8)) * 8;
        if (row >= a.n_dec || c >= cols) *reinterpret_cast<uint4*>(hs + row * ldh + c) = make_uint4(0, 0, 0, 0);
    }
    if (a.dim % 32 == 0 && ns <= 32 && total <= THREADS) {
        // The usual case, without shared memory or a barrier: the 32 elements of a warp belong to one (request, head),
        // lane s fetches range s's statistics and computes its weight, and the lanes pass the weights round.
        const int e = tid;
        const bool live = e < total;                               // the same for a whole warp
        const int p = e / a.dim, d = e - p * a.dim, i = p / max(heads, 1), hj = p - i * heads;
        const size_t base = ((size_t)i * a.hq + head0 + hj) * ns;
        float2 ml = make_float2(-INFINITY, 0.f);
        if (live && lane < ns) ml = reinterpret_cast<const float2*>(a.stats)[base + lane];
        const float m = warp_max(ml.y > 0.f ? ml.x : -INFINITY);
        const float w = ml.y > 0.f ? expf(ml.x - m) : 0.f;          // a range without keys weighs nothing
        const float wl_ = ml.y > 0.f ? __fmul_rn(w, ml.y) : 0.f;
        float den = 0.f, num = 0.f;                                 // both sums in the order of the ranges, as in the merge kernel
#pragma unroll
        for (int sp = 0; sp < SB; ++sp) {
            const float ws = __shfl_sync(0xffffffffu, w, sp), wls = __shfl_sync(0xffffffffu, wl_, sp);
            if (sp < ns) {
                den = __fadd_rn(den, wls);
                num = fmaf(ws, ws > 0.f ? pre[sp] : 0.f, num);
            }
        }
        if (ns > SB) {                                              // contexts beyond sixteen ranges: one more trip
            float v[SB];
#pragma unroll
            for (int sp = 0; sp < SB; ++sp) v[sp] = (live && SB + sp < ns) ? a.partial[(base + SB + sp) * a.dim + d] : 0.f;
#pragma unroll
            for (int sp = 0; sp < SB; ++sp) {
                const float ws = __shfl_sync(0xffffffffu, w, SB + sp), wls = __shfl_sync(0xffffffffu, wl_, SB + sp);
                if (SB + sp < ns) {
                    den = __fadd_rn(den, wls);
                    num = fmaf(ws, ws > 0.f ? v[sp] : 0.f, num);
                }
            }
        }
        if (live) hs[i * ldh + hj * a.dim + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);   // no keys: a padding row
        CISR_TRACE_MARK(0);
    } else {
    for (int x = tid; x < pairs * nsp; x += THREADS) {
        const int p = x / nsp, sp = x - p * nsp, i = p / heads;
        float2 ml = make_float2(-INFINITY, 0.f);                    // the padding behaves like a range without keys
        if (sp < ns) ml = reinterpret_cast<const float2*>(a.stats)[((size_t)i * a.hq + head0 + (p - i * heads)) * ns + sp];
        raw[(size_t)p * 2 * nsp + sp] = ml.x; raw[(size_t)p * 2 * nsp + nsp + sp] = ml.y;
    }
    __syncthreads();
    for (int x = tid; x < pairs * nsp; x += THREADS) {
        const int p = x / nsp, sp = x - p * nsp;
        const float4* mx = reinterpret_cast<const float4*>(raw + (size_t)p * 2 * nsp);
        const float4* lx = mx + nsp / 4;
        float m = -INFINITY;
#pragma unroll 4
        for (int q = 0; q < nsp / 4; ++q) {                         // the loads do not depend on one another
            const float4 mv = mx[q], lv = lx[q];
            m = fmaxf(m, fmaxf(fmaxf(lv.x > 0.f ? mv.x : -INFINITY, lv.y > 0.f ? mv.y : -INFINITY),
                               fmaxf(lv.z > 0.f ? mv.z : -INFINITY, lv.w > 0.f ? mv.w : -INFINITY)));
        }
        const float l = raw[(size_t)p * 2 * nsp + nsp + sp];
        const float w = l > 0.f ? expf(raw[(size_t)p * 2 * nsp + sp] - m) : 0.f;    // a range without keys weighs nothing
        wsm[(size_t)p * 2 * nsp + sp] = w;
        wsm[(size_t)p * 2 * nsp + nsp + sp] = l > 0.f ? __fmul_rn(w, l) : 0.f;
    }
    __syncthreads();
    CISR_TRACE_MARK(0);
    // the first element from the registers requested above; those beyond it (more tokens, wider slices) load as they go
    if (tid < total) merge_element<true>(a, tid, heads, head0, ns, nsp, ldh, wsm, hs, pre);
#pragma unroll 1
    for (int e = THREADS + tid; e < total; e += THREADS) merge_element<false>(a, e, heads, head0, ns, nsp, ldh, wsm, hs, pre);
    }
    __syncthreads();
    CISR_TRACE_MARK(1);

    // ---- this CTA's K-slice of the product
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) { acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f; }
    // Every lane runs every mma (a warp-wide instruction never sits under a lane-dependent condition); lanes whose
    // columns lie beyond the slice feed zeros on both sides.
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        if (i < chunks && tile_warp) {                              // the same for the whole warp
            const int kb = i * 32 + 8 * t;
            const bool in_k = kb < cols;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint4 b = make_uint4(0, 0, 0, 0);
                if (in_k) b = *reinterpret_cast<const uint4*>(hs + (mt * 8 + r) * ldh + kb);
                mma_bf16(acc[mt], wl[i].x, wh[i].x, wl[i].y, wh[i].y, b.x, b.y);
                mma_bf16(acc[mt], wl[i].z, wh[i].z, wl[i].w, wh[i].w, b.z, b.w);
            }
        }
    }
    // ---- the K-slices meet in the CTA that finishes the feature: CTA `rank` owns `per` features of the tile and
    // receives every CTA's partial products for them, [sender][feature][token], straight from the senders' registers.
    const int per = (FT + ranks - 1) / ranks;
    if (tile_warp) {
        const uint32_t here = smem_u32_of(part) + (uint32_t)(rank * per * mw * sizeof(float));   // this sender's block, in any receiver
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = warp * 16 + r + 8 * half, owner = row / per, fr = row - owner * per;
            const uint32_t there = shared_of_rank(here, (uint32_t)owner) + (uint32_t)(fr * mw * sizeof(float));
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                store_cluster(there + (uint32_t)((mt * 8 + 2 * t) * sizeof(float)), acc[mt][2 * half]);
                store_cluster(there + (uint32_t)((mt * 8 + 2 * t + 1) * sizeof(float)), acc[mt][2 * half + 1]);
            }
        }
    }
    cluster_barrier();                          // every CTA's partial products have arrived; nothing remote is touched after this
    CISR_TRACE_MARK(2);
    for (int e = tid; e < per * a.n_dec; e += THREADS) {
        const int fr = e / a.n_dec, i = e - fr * a.n_dec;
        const int row = rank * per + fr, f = blockIdx.x * FT + row;
        if (row >= FT || f >= a.n) continue;
        float sum = 0.f;
        for (int c = 0; c < ranks; ++c) sum += part[((size_t)c * per + fr) * mw + i];       // in the order of the CTAs
        float* dst = a.out + (size_t)a.q_start[a.dec_req[i]] * a.n + f;
        if (a.accumulate) sum += dst == first_out ? there : *dst;
        *dst = sum;
    }
}

size_t smem_bytes(const MergeProjArgs& a, int mt) {
    const int slice = a.heads_per_cta * a.dim, mw = mt * 8;
    return sizeof(bf16) * (size_t)mw * (slice + 8) + sizeof(float) * (size_t)(FT + 16) * mw +       // ranks * ceil(FT / ranks) <= FT + 16
           sizeof(float) * 4 * (size_t)a.n_dec * a.heads_per_cta * ((a.n_splits + 3) & ~3);
}

template <int MT, int NCH>
int launch_chunks(const MergeProjArgs& a, int ranks, cudaStream_t s) {
    const size_t smem = smem_bytes(a, MT);
    if (smem > 200 * 1024) return -2;
    static size_t configured = 48 * 1024;
    static bool non_portable = false;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(merge_proj_kernel<MT, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    if (ranks > 8 && !non_portable) {
        cudaError_t e = cudaFuncSetAttribute(merge_proj_kernel<MT, NCH>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) { cudaGetLastError(); return -2; }
        non_portable = true;
    }
    static int resident[17] = {};             // per cluster size: 0 unknown, 1 such clusters fit the device, -1 they do not
    if (!resident[ranks]) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(1, 1, ranks); config.blockDim = dim3(THREADS); config.dynamicSmemBytes = configured;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)ranks;
        config.attrs = attr; config.numAttrs = 1;
        int n = 0;
        const cudaError_t e = ranks > 1 ? cudaOccupancyMaxActiveClusters(&n, merge_proj_kernel<MT, NCH>, &config) : cudaSuccess;
        cudaGetLastError();
        resident[ranks] = (ranks == 1 || (e == cudaSuccess && n >= 1)) ? 1 : -1;
    }
    if (resident[ranks] < 0) return -2;
    return launch_kernel_cluster(merge_proj_kernel<MT, NCH>, dim3((a.n + FT - 1) / FT, 1, ranks), dim3(THREADS), smem, s, g_pdl, ranks, a);
}
template <int MT>
int launch(const MergeProjArgs& a, int ranks, cudaStream_t s) {
    const int slice = a.heads_per_cta * a.dim;
    if (slice <= 64) return launch_chunks<MT, 2>(a, ranks, s);
    if (slice <= 128) return launch_chunks<MT, 4>(a, ranks, s);
    return launch_chunks<MT, 8>(a, ranks, s);
}
}  // namespace

CISR_EXPORT void cisr_merge_proj_set_pdl(int on) { g_pdl = on != 0; }

// How the query heads are dealt to the CTAs of a cluster: heads per CTA (0 when this kernel does not take the shape).
CISR_EXPORT int cisr_merge_proj_heads_per_cta(int n_dec, int hq, int dim, int k) {
    if (n_dec <= 0 || n_dec > 16 || hq <= 0 || dim <= 0 || dim % 8 || k != hq * dim) return 0;
    const int per = (hq + 15) / 16;
    return per * dim <= MAX_SLICE ? per : 0;
}

// out[q_start[dec_req[i]], :] (float [tokens, n]) = merge over the key ranges of request i's partial sums, times w^T.
// Returns -2 for shapes it does not take (the caller then runs the merge kernel and the product apart).
CISR_EXPORT int cisr_merge_proj(const float* partial, const float* stats, int n_splits, const int* dec_req, const int* q_start,
                                int n_dec, int hq, int dim, const void* w, int n, int k, float* out, int accumulate, void* stream) {
    const int per = cisr_merge_proj_heads_per_cta(n_dec, hq, dim, k);
    if (!per || n <= 0 || n_splits <= 0 || (((uintptr_t)w) & 15) || (k % 8)) return -2;
    MergeProjArgs a;
    a.partial = partial; a.stats = stats; a.n_splits = n_splits; a.dec_req = dec_req; a.q_start = q_start; a.n_dec = n_dec;
    a.hq = hq; a.dim = dim; a.heads_per_cta = per; a.w = (const bf16*)w; a.n = n; a.out = out; a.accumulate = accumulate != 0;
    const int ranks = (hq + per - 1) / per;
    cudaStream_t s = (cudaStream_t)stream;
    return n_dec <= 8 ? launch<1>(a, ranks, s) : launch<2>(a, ranks, s);
}
