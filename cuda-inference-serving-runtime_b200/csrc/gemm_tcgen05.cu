// Matrix product on the 5th-generation tensor cores: out[M, N] (float) = a[M, K] * w[N, K]^T, bfloat16
// operands, float accumulation in tensor memory.  Used for steps with more tokens than the weight-streaming
// kernels take (prompt portions, large decode batches).
//
//   * persistent CTAs, each walking output tiles of 128 x BN (BN = 256, 128 or 64, chosen from the number of
//     tiles: see the launchers), with two accumulators of BN columns in tensor memory so that the epilogue of
//     one tile runs under the products of the next
//   * warp 0: one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the A tile
//     [128 rows x 64 k] and the B tile [BN rows x 64 k] into a STAGES-deep ring of shared memory (3 to 8
//     stages), each load completing on the stage's "full" mbarrier
//   * warp 1: allocates 2 * BN columns of tensor memory; one thread issues tcgen05.mma (kind::f16, M = 128,
//     N = BN, K = 16, four per 64-wide k block) on shared-memory descriptors and commits each stage to its
//     "empty" mbarrier, and each finished tile to its "accumulator ready" mbarrier
//   * warps 2..5: read the accumulator with tcgen05.ld (32 lanes x 32 columns per warp and step) and run the
//     epilogue: PLAIN writes float rows of `out` (or adds them to it: the residual form); SWIGLU (the B tile is
//     gate rows and the up rows of the same features) writes silu(gate) * up as bfloat16; ROPE (the tile is
//     whole heads of the stacked q/k/v projection) rotates q and k heads and writes q rows and the k, v cache
//     pages as bfloat16
//
// Rows and columns beyond M, N or K are zero-filled by TMA on the way in and skipped on the way out, so any
// M and N work; K must be a multiple of 8 (16-byte rows for the tensor map).  Every wait on an mbarrier
// gives up after a bounded number of polls: the kernel then sets `*error`, skips the rest of its work,
// frees its tensor memory and returns, and the host reports the failure.
//
// Parity: this is the product runtime/blas.py:41-56 of the reference hands to cuBLAS (C^T = W * X^T).
#include "tcgen05.cuh"

namespace {
typedef __nv_bfloat16 bf16;
enum : int { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_ROPE = 2 };
constexpr int BK = 64, UMMA_K = 16;     // BM = 128 (tcgen05.cuh)

struct Epilogue {                       // what the epilogue variants need beyond the accumulator
    float* out_f32; bf16* out_bf16; int inter;
    int accumulate;                     // PLAIN: out += product (the residual stream, in place) instead of out = product
    const float* cos_t; const float* sin_t; bf16* q_out; bf16* k_cache; bf16* v_cache; const int* positions;
    const int* token_req; const int* req_slot; const int* block_table; int table_width; int page_size; int hq; int hkv; int dim;
};
// 32 floats -> 32 bfloat16 (64 bytes) at dst; `count` of them are valid
__device__ __forceinline__ void store_bf16x32(bf16* dst, const float (&v)[32], int count) {
    if (count >= 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            uint4 p;
            __nv_bfloat162 a = __floats2bfloat162_rn(v[j], v[j + 1]), b = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
            __nv_bfloat162 c = __floats2bfloat162_rn(v[j + 4], v[j + 5]), d = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
            p.x = *reinterpret_cast<uint32_t*>(&a); p.y = *reinterpret_cast<uint32_t*>(&b);
            p.z = *reinterpret_cast<uint32_t*>(&c); p.w = *reinterpret_cast<uint32_t*>(&d);
            *reinterpret_cast<uint4*>(dst + j) = p;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < count) dst[j] = __float2bfloat16_rn(v[j]);
    }
}

// Columns of tensor memory for two accumulators of `bn` columns: allocations are powers of two.
__host__ __device__ constexpr int tmem_columns(int bn) { return 2 * bn <= 32 ? 32 : 2 * bn <= 64 ? 64 : 2 * bn <= 128 ? 128 : 2 * bn <= 256 ? 256 : 512; }

template <int BN, int STAGES>
struct Smem {
    static constexpr size_t A_BYTES = (size_t)BM * BK * sizeof(bf16);
    static constexpr size_t B_BYTES = (size_t)BN * BK * sizeof(bf16);
    static constexpr size_t TILES = STAGES * (A_BYTES + B_BYTES);
    static constexpr size_t TOTAL = TILES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// The epilogue of one output tile for one thread: `row` is the thread's output row, `lane_base` the tensor-memory
// address of its lane in the tile's accumulator, n0 the tile's first column (feature).
template <int BN, int EPI>
// `pos`, `page` (ROPE): the row's position and the cache page it is written to, looked up by the caller while the tile
// was still being accumulated (-1: a padding row, or a row beyond the step).
__device__ __forceinline__ void epilogue_tile(const Epilogue& ep, uint32_t lane_base, int row, int m, int n, int n0, int pos, int page) {
    if (EPI == EPI_PLAIN) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
            uint32_t v[32];
            tmem_load32(lane_base + (uint32_t)c, v);
            if (row < m) {
                float* dst = ep.out_f32 + (size_t)row * n + n0 + c;
                if (n0 + c + 32 <= n && (n & 3) == 0) {
                    if (ep.accumulate) {
                        // The add is done where the element lives (a reduction in L2), so the epilogue does not wait for
                        // a load: every element belongs to this thread alone, and one float add in round-to-nearest is
                        // the same sum wherever it is made.
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(__uint_as_float(v[j])),
                                         "f"(__uint_as_float(v[j + 1])), "f"(__uint_as_float(v[j + 2])), "f"(__uint_as_float(v[j + 3])) : "memory");
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                              __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + c + j < n) dst[j] = ep.accumulate ? dst[j] + __uint_as_float(v[j]) : __uint_as_float(v[j]);
                }
            }
        }
    } else if (EPI == EPI_SWIGLU) {
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
            uint32_t g[32], u[32];
            tmem_load32(lane_base + (uint32_t)c, g);
            tmem_load32(lane_base + (uint32_t)(BN / 2 + c), u);
            float act[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float gv = __uint_as_float(g[j]);
                act[j] = gv / (1.f + expf(-gv)) * __uint_as_float(u[j]);
            }
            if (row < m && n0 + c < ep.inter)
                store_bf16x32(ep.out_bf16 + (size_t)row * ep.inter + n0 + c, act, ep.inter - (n0 + c));
        }
    } else {
        // whole heads of the stacked q, k, v projection: BN / dim heads per tile, rotation pairs (i, i + dim / 2)
        const int dim = ep.dim, half = dim / 2;
#pragma unroll 1
        for (int h0 = 0; h0 < BN; h0 += dim) {
            const int hh = (n0 + h0) / dim;                        // head index in the stacked projection
            if (hh >= ep.hq + 2 * ep.hkv) break;
            const bool is_q = hh < ep.hq, is_k = !is_q && hh < ep.hq + ep.hkv;
            bf16* dst = nullptr;
            if (row < m) {
                if (is_q) dst = ep.q_out + ((size_t)row * ep.hq + hh) * dim;
                else if (page >= 0) {                               // a missing page entry: a padding row, nothing to write
                    const int kvh = is_k ? hh - ep.hq : hh - ep.hq - ep.hkv;
                    dst = (is_k ? ep.k_cache : ep.v_cache) +
                          (((size_t)page * ep.hkv + kvh) * ep.page_size + pos % ep.page_size) * dim;
                }
            }
#pragma unroll 1
            for (int c = 0; c < half; c += 32) {
                uint32_t lo[32], hi[32];
                tmem_load32(lane_base + (uint32_t)(h0 + c), lo);
                tmem_load32(lane_base + (uint32_t)(h0 + half + c), hi);
                float first[32], second[32];
                if ((is_q || is_k) && row < m) {
                    const float4* cs = reinterpret_cast<const float4*>(ep.cos_t + (size_t)row * half + c);   // half is a multiple of 32
                    const float4* sn = reinterpret_cast<const float4*>(ep.sin_t + (size_t)row * half + c);
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 cv = cs[j >> 2], sv = sn[j >> 2];
                        const float cc[4] = {cv.x, cv.y, cv.z, cv.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float a = __uint_as_float(lo[j + u]), b = __uint_as_float(hi[j + u]);
                            first[j + u] = a * cc[u] - b * ss[u];
                            second[j + u] = b * cc[u] + a * ss[u];
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) { first[j] = __uint_as_float(lo[j]); second[j] = __uint_as_float(hi[j]); }
                }
                if (dst) {
                    store_bf16x32(dst + c, first, 32);
                    store_bf16x32(dst + half + c, second, 32);
                }
            }
        }
    }
}

// Persistent: a CTA walks output tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the accumulator is double-buffered in
// tensor memory, so the MMA thread fills one buffer while the epilogue warps drain the other.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(192)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const Epilogue ep, int m, int n, int k, int tiles_m, int tiles_n, int* __restrict__ error) {
    CISR_TRACE_SCOPE(TRACE_GEMM_TCGEN05);
    extern __shared__ unsigned char smem_raw[];
    typedef Smem<BN, STAGES> S;
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1024-byte aligned
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + S::TILES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;       // [2]: the MMAs of a tile are done
    uint64_t* acc_empty = acc_full + 2;            // [2]: the epilogue has read the buffer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (k + BK - 1) / BK;
    const int total_tiles = tiles_m * tiles_n;
    constexpr int TILE_N = EPI == EPI_SWIGLU ? BN / 2 : BN;   // SWIGLU: 128 accumulator columns are 64 gate + 64 up features

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
        mbar_init_fence();
    }
    if (warp == 1) {    // one warp allocates two accumulators' columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_columns(BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    pdl_trigger();      // under programmatic dependent launch the next kernel may begin its own set-up now

    if (warp == 0) {
        if (lane == 0) {
            auto load_b = [&](int s, int kb, int n0) {
                unsigned char* b_tile = tiles + s * (S::A_BYTES + S::B_BYTES) + S::A_BYTES;
                if (EPI == EPI_SWIGLU) {      // two boxes of BN/2 rows: gate rows n0.., up rows inter + n0..
                    tma_load_2d(b_tile, &map_w, kb * BK, n0, full_bar + s);
                    tma_load_2d(b_tile + S::B_BYTES / 2, &map_w, kb * BK, ep.inter + n0, full_bar + s);
                } else {
                    tma_load_2d(b_tile, &map_w, kb * BK, n0, full_bar + s);
                }
            };
            // The weights do not come from the kernel before this one: the first stages' weight tiles are requested
            // before the wait on that kernel, the activation tiles after it.
            const int early = k_blocks < STAGES ? k_blocks : STAGES;
            if ((int)blockIdx.x < total_tiles) {
                const int n0 = ((int)blockIdx.x / tiles_m) * TILE_N;
                for (int kb = 0; kb < early; ++kb) {
                    mbar_expect_tx(full_bar + kb, (uint32_t)(S::A_BYTES + S::B_BYTES));
                    load_b(kb, kb, n0);
                }
            }
            pdl_wait();
            CISR_TRACE_WAITED();
            int kbg = 0;                                                      // k blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * TILE_N;   // neighbours share the weight tile
                for (int kb = 0; kb < k_blocks; ++kb, ++kbg) {
                    const int s = kbg % STAGES;
                    if (kbg < early) {        // this stage's barrier is armed and its weight tile on the way already
                        tma_load_2d(tiles + s * (S::A_BYTES + S::B_BYTES), &map_a, kb * BK, m0, full_bar + s);
                        continue;
                    }
                    ok = mbar_wait(empty_bar + s, ((kbg / STAGES) & 1) ^ 1);  // the MMAs that read this stage are done
                    if (!ok) break;
                    mbar_expect_tx(full_bar + s, (uint32_t)(S::A_BYTES + S::B_BYTES));
                    tma_load_2d(tiles + s * (S::A_BYTES + S::B_BYTES), &map_a, kb * BK, m0, full_bar + s);
                    load_b(s, kb, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            int kbg = 0, it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                ok = mbar_wait(acc_empty + acc, ((it >> 1) & 1) ^ 1);          // the epilogue has drained this buffer
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++kbg) {
                    const int s = kbg % STAGES;
                    ok = mbar_wait(full_bar + s, (kbg / STAGES) & 1);          // both tiles of this stage have landed
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint64_t desc_a = umma_desc(tiles + s * (S::A_BYTES + S::B_BYTES));
                    const uint64_t desc_b = umma_desc(tiles + s * (S::A_BYTES + S::B_BYTES) + S::A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)                    // 32 bytes further along K per step
                        umma_bf16(tmem_acc, desc_a + 2 * kk, desc_b + 2 * kk, idesc, (kb | kk) != 0);
                    umma_commit(empty_bar + s);                                // frees the stage when these MMAs finish
                }
                if (ok) umma_commit(acc_full + acc);                           // the whole tile is accumulated
            }
        }
    } else {
        const int quarter = warp & 3;                                          // the 32 lanes this warp may read
        int it = 0;
        pdl_wait();      // outputs may alias what the kernel before still reads; step metadata is older than that kernel
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * TILE_N;
            const int row = m0 + quarter * 32 + lane;
            // ROPE: where the row's key and value go hangs on four dependent loads of step metadata; they run while
            // the tile is still being accumulated instead of after it
            int pos = 0, page = -1;
            if (EPI == EPI_ROPE && row < m) {
                pos = ep.positions[row];
                page = ep.block_table[(size_t)ep.req_slot[ep.token_req[row]] * ep.table_width + pos / ep.page_size];
            }
            ok = mbar_wait(acc_full + acc, (it >> 1) & 1);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t lane_base = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
            epilogue_tile<BN, EPI>(ep, lane_base, row, m, n, n0, pos, page);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(acc_empty + acc)) : "memory");
        }
    }
    if (!ok && lane == 0) atomicExch(error, 1);
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_columns(BN)) : "memory");
}

// ---------------------------------------------------------------- host side
bool g_pdl = false;
int* g_error = nullptr;          // device flag, owned by the caller (see cisr_gemm_tcgen05_init)

template <int BN, int STAGES, int EPI>
int launch(const void* a, const void* w, const Epilogue& ep, int m, int n, int k, int tiles_n, cudaStream_t s) {
    CUtensorMap map_a, map_w;
    int status = cached_map(&map_a, a, m, k, BM);
    if (status) return status;
    if ((status = cached_map(&map_w, w, n, k, EPI == EPI_SWIGLU ? BN / 2 : BN))) return status;
    typedef Smem<BN, STAGES> S;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    static int slots = 0;                        // CTAs that fit on the device at once
    if (!slots) {
        int device = 0, sms = 0, per_sm = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_tcgen05_kernel<BN, STAGES, EPI>, 192, S::TOTAL);
        per_sm = per_sm < 1 ? 1 : per_sm;
        if (per_sm * tmem_columns(BN) > 512) per_sm = 512 / tmem_columns(BN);      // tensor memory: 512 columns per SM
        slots = sms * per_sm;
    }
    const int tiles_m = (m + BM - 1) / BM, total = tiles_m * tiles_n;
    return launch_kernel(gemm_tcgen05_kernel<BN, STAGES, EPI>, dim3(total < slots ? total : slots), dim3(192), S::TOTAL, s, g_pdl,
                         map_a, map_w, ep, m, n, k, tiles_m, tiles_n, g_error);
}

// 128 x 256 tiles read a third less from L2 per flop than 128 x 128; worth it once there are enough of them to
// occupy most of the device (one CTA per SM at that size).
bool wide_tiles(int m, int tiles_n256) { return (long long)((m + BM - 1) / BM) * tiles_n256 >= 120; }

// Fewer 128 x 128 tiles than SMs: every CTA runs one tile, alone on its SM, and the time is the ring's round trips to
// L2 (a stage is asked for again only after its product), not the tensor pipe.  A deeper ring with the whole SM's
// shared memory hides them, and while 128 x 64 tiles still fit the device at one per SM, twice as many CTAs share
// the weights.  Returns 64 or 128 for the tile width of the deep ring, 0 for the ordinary choice (also with
// CISR_GEMM_DEEP=0).  `cols`: output columns a 128-wide tile covers (64 features for the gated product).
int few_tiles(int m, int n, int cols) {
    static int sms = 0, on = -1;
    if (!sms) { int device = 0; cudaGetDevice(&device); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device); }
    if (on < 0) { const char* e = getenv("CISR_GEMM_DEEP"); on = !(e && e[0] == '0'); }
    if (!on) return 0;
    const long long tiles_m = (m + BM - 1) / BM;
    if (tiles_m * ((n + cols / 2 - 1) / (cols / 2)) <= sms) return 64;
    if (tiles_m * ((n + cols - 1) / cols) <= sms) return 128;
    return 0;
}

bool operands_ok(const void* a, const void* w, int k) {
    return g_encode && g_error && k > 0 && k % 8 == 0 && !(((uintptr_t)a | (uintptr_t)w) & 15);
}
}  // namespace

// `error_flag`: one zeroed int in device memory that a kernel sets when one of its waits ran out.
CISR_EXPORT int cisr_gemm_tcgen05_init(int* error_flag) {
    if (int status = tma_load_encoder()) return status;
    g_error = error_flag;
    return 0;
}

CISR_EXPORT void cisr_gemm_tcgen05_set_pdl(int on) { g_pdl = on != 0; }

// How many tensor maps the library remembers before it empties its cache (tests lower it to force evictions).
CISR_EXPORT void cisr_gemm_tcgen05_set_map_cache_limit(int entries) { g_map_cache_limit = entries < 1 ? 1 : (size_t)entries; }

// Three pipeline stages keep a CTA near 100 KB of shared memory, so two CTAs share an SM and one's epilogue overlaps
// the other's main loop.
// accumulate != 0: out += a w^T (each output element is read, added to in float and written by the one thread that
// owns it: what the residual add of a layer does, without a pass of its own).
CISR_EXPORT int cisr_gemm_tcgen05(const void* a, const void* w, float* out, int m, int n, int k, int accumulate, void* stream) {
    if (m <= 0 || n <= 0) return 0;
    if (!g_encode || !g_error) return -13;
    if (!operands_ok(a, w, k) || ((uintptr_t)out & 15)) return -2;
    Epilogue ep = {};
    ep.out_f32 = out; ep.accumulate = accumulate != 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (n <= 64) return launch<64, 8, EPI_PLAIN>(a, w, ep, m, n, k, (n + 63) / 64, s);
    if (wide_tiles(m, (n + 255) / 256)) return launch<256, 4, EPI_PLAIN>(a, w, ep, m, n, k, (n + 255) / 256, s);
    const int deep = few_tiles(m, n, 128);
    if (deep == 64) return launch<64, 8, EPI_PLAIN>(a, w, ep, m, n, k, (n + 63) / 64, s);
    if (deep == 128) return launch<128, 6, EPI_PLAIN>(a, w, ep, m, n, k, (n + 127) / 128, s);
    return launch<128, 3, EPI_PLAIN>(a, w, ep, m, n, k, (n + 127) / 128, s);
}

// w stacks gate rows [0, inter) over up rows [inter, 2 * inter); out (bfloat16 [m, inter]) = silu(a gate^T) * (a up^T).
CISR_EXPORT int cisr_gemm_tcgen05_swiglu(const void* a, const void* w, void* out, int m, int inter, int k, void* stream) {
    if (m <= 0 || inter <= 0) return 0;
    if (!g_encode || !g_error) return -13;
    if (!operands_ok(a, w, k)) return -2;
    Epilogue ep = {};
    ep.out_bf16 = (bf16*)out; ep.inter = inter;
    if (wide_tiles(m, (inter + 127) / 128)) {
        // 128 x 256 tiles, or 128 x 192 where their last round would be much emptier: 192 tiles of 256 columns on 148 SMs
        // are two rounds for 1.3 rounds of work, 256 tiles of 192 columns are two rounds of three quarters the length
        static int sms = 0;
        if (!sms) { int device = 0; cudaGetDevice(&device); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device); if (sms <= 0) sms = 148; }
        const long long tiles_m = (m + BM - 1) / BM;
        const long long rounds256 = (tiles_m * ((inter + 127) / 128) + sms - 1) / sms, rounds192 = (tiles_m * ((inter + 95) / 96) + sms - 1) / sms;
        if (rounds192 * 192 * 10 <= rounds256 * 256 * 9)
            return launch<192, 4, EPI_SWIGLU>(a, w, ep, m, 2 * inter, k, (inter + 95) / 96, (cudaStream_t)stream);
        return launch<256, 4, EPI_SWIGLU>(a, w, ep, m, 2 * inter, k, (inter + 127) / 128, (cudaStream_t)stream);
    }
    const int deep = few_tiles(m, inter, 64);
    if (deep == 64) return launch<64, 8, EPI_SWIGLU>(a, w, ep, m, 2 * inter, k, (inter + 31) / 32, (cudaStream_t)stream);
    if (deep == 128) return launch<128, 6, EPI_SWIGLU>(a, w, ep, m, 2 * inter, k, (inter + 63) / 64, (cudaStream_t)stream);
    return launch<128, 3, EPI_SWIGLU>(a, w, ep, m, 2 * inter, k, (inter + 63) / 64, (cudaStream_t)stream);
}

// w stacks the q, k and v heads; q and k heads are rotated (pairs (i, i + dim / 2), cos/sin [m, dim / 2]); q goes to
// q_out [m, hq, dim], k and v to their cache pages.  Takes dim 64 or 128 (whole heads per 128-column tile and 32-column
// halves of the rotation); other head sizes use the plain product and the separate rotation kernel.
CISR_EXPORT int cisr_gemm_tcgen05_rope(const void* a, const void* w, int m, int k, const float* cos_t, const float* sin_t,
                                       void* q_out, void* k_cache, void* v_cache, const int* positions,
                                       const int* token_req, const int* req_slot, const int* block_table,
                                       int table_width, int page_size, int hq, int hkv, int dim, void* stream) {
    if (m <= 0) return 0;
    if (!g_encode || !g_error) return -13;
    if (!operands_ok(a, w, k) || (dim != 64 && dim != 128)) return -2;
    Epilogue ep = {};
    ep.cos_t = cos_t; ep.sin_t = sin_t; ep.q_out = (bf16*)q_out; ep.k_cache = (bf16*)k_cache; ep.v_cache = (bf16*)v_cache;
    ep.positions = positions; ep.token_req = token_req; ep.req_slot = req_slot; ep.block_table = block_table;
    ep.table_width = table_width; ep.page_size = page_size; ep.hq = hq; ep.hkv = hkv; ep.dim = dim;
    const int n = (hq + 2 * hkv) * dim;
    if (wide_tiles(m, (n + 255) / 256)) return launch<256, 4, EPI_ROPE>(a, w, ep, m, n, k, (n + 255) / 256, (cudaStream_t)stream);
    const int deep = few_tiles(m, n, 128);
    if (deep == 64 && dim == 64) return launch<64, 8, EPI_ROPE>(a, w, ep, m, n, k, (n + 63) / 64, (cudaStream_t)stream);   // a whole head per tile
    if (deep) return launch<128, 6, EPI_ROPE>(a, w, ep, m, n, k, (n + 127) / 128, (cudaStream_t)stream);
    return launch<128, 3, EPI_ROPE>(a, w, ep, m, n, k, (n + 127) / 128, (cudaStream_t)stream);
}
