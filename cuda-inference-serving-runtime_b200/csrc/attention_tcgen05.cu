// Causal grouped-query attention of prompt portions on the 5th-generation tensor cores, for head sizes 64 and 128
// (bfloat16 cache).  One CTA per (128-query tile, query head); scores and the output accumulate in tensor memory.
//
//   warps 0, 2  producers: warp 0 the query tile once and then the key tiles, warp 2 the value tiles (128 keys each),
//               into rings of their own (four stages each at head size 64; three key and two value stages at 128),
//               by tensor-map copies (cp.async.bulk.tensor.2d, 128-byte swizzle), one box per page and 64 columns;
//               page ids come straight from the block table.  A key tile is free again when its score product is
//               done, a value tile after the output product, one softmax later
//   warp 1      one thread issues the products: S = Q K^T (tcgen05.mma kind::f16, M = 128, N = 128, K = 16 steps,
//               Q and K both K-major) into one of two score buffers in tensor memory, and, for each half of a
//               tile's keys, O_g += P_g V (N = head size, P read from tensor memory as the A operand, V as the
//               MN-major B operand straight from its [key][dim] tile).  The scores run two tiles ahead of the
//               output products
//   warps 3..10 softmax, two groups of four warps, each a stream of its own: thread (group g, r) has keys
//               [64 g, 64 g + 64) of every tile for query row r (tensor-memory lane r), its own running max and sum
//               in float and its own output accumulator O_g, so one group's exponentials run while the other waits,
//               loads or stores.  Once a row has a max in use, the exponentials of a tile are taken against it in
//               the same pass that finds the tile's own max; only when that turns out more than 8 above the max in
//               use (a stale max is exact arithmetic as long as 2^(s - m) stays small) is the row of O_g rescaled
//               and the tile done again from the scores.  P = 2^(s - m) goes back to tensor memory as bfloat16
//               pairs (tcgen05.st) over the first half of the thread's own scores.  At the end the two streams of
//               a row are merged with their maxima and sums.
//
// Exactness: scores are scaled by scale * log2(e) in float after the product, exponentials are base 2 (ex2.approx),
// the sums and the maxima are float, P is rounded to bfloat16 once.  The keys a query sees, their split into the two
// streams and their order do not depend on the batch: tiles start at multiples of 128 in absolute positions.
//
// Every wait on an mbarrier is bounded; a role whose wait ran out raises the CTA's abort flag and the device flag
// (5), the other roles leave at their next wait, tensor memory is freed, and the host reports the failure.
//
// Parity: the online softmax of runtime/reference.py:18-27 and kernels/ops.cu:88-123 of the reference, tiled.
// Cache layout: [pages, kv_heads, page_size, HEAD_DIM]; page sizes: multiples of 8 that divide 128 or are multiples of it.
#include "tcgen05.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=64 or 128"
#endif
#if HEAD_DIM != 64 && HEAD_DIM != 128
#error "the tcgen05 attention takes head sizes 64 and 128"
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int D = HEAD_DIM;
constexpr int NSUB = D / 64;                  // 64-column sub-tiles of Q, K and V rows
constexpr int BN = 128;                       // keys per tile
constexpr int SUB_BYTES = 128 * 128;          // one 128-row x 64-column sub-tile (queries, probabilities)
constexpr int KV_SUB = BN * 128;              // one BN-key x 64-column sub-tile (keys, values)
constexpr int Q_BYTES = NSUB * SUB_BYTES;
constexpr int KV_BYTES = NSUB * KV_SUB;       // a K tile, or a V tile
// tensor memory: two score buffers [0, 2 BN), then the two groups' output accumulators [256, 256 + 2 D)
// Key tiles and value tiles have rings of their own: a key tile is free again when its score product is done, a value
// tile only after the output product, one softmax later.  A tile is 16 KB at head size 64 and 32 KB at 128.
constexpr int K_STAGES = D == 64 ? 4 : 3;
constexpr int V_STAGES = D == 64 ? 4 : 2;
constexpr size_t SMEM_FIXED = 1024 + Q_BYTES + (K_STAGES + V_STAGES) * KV_BYTES + 256 + 4 * 128 * sizeof(float);
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;           // the max may lag by this much (base-2 exponent) before O is rescaled
constexpr int SOFTMAX_THREADS = 256;          // two groups of four warps: each thread has half of a query row's columns
constexpr int FIRST_SOFTMAX_WARP = 3;         // warps 0 to 2: key producer, issuing thread, value producer
constexpr int THREADS = 32 * FIRST_SOFTMAX_WARP + SOFTMAX_THREADS;
constexpr int HALF = BN / 2;                  // score columns per softmax thread and tile
bool g_pdl = false;
int* g_error = nullptr;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int cache_rows,
                            const int* __restrict__ req_slot, const int* __restrict__ block_table, int table_width,
                            const int* __restrict__ tile_req, const int* __restrict__ tile_q0,
                            const int* __restrict__ q_start, const int* __restrict__ q_len,
                            const int* __restrict__ ctx_len, int hq, int hkv, int page_size, float scale, int window,
                            int* __restrict__ error) {
    CISR_TRACE_SCOPE(TRACE_ATTN_PREFILL);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = base;                                   // [NSUB][128 queries][128 B]
    unsigned char* Kring = Qs + Q_BYTES;                        // [K_STAGES] key tiles, each [NSUB][BN keys][128 B]
    unsigned char* Vring = Kring + K_STAGES * KV_BYTES;         // [V_STAGES] value tiles, the same layout
    uint64_t* bars = reinterpret_cast<uint64_t*>(Vring + V_STAGES * KV_BYTES);
    uint64_t* q_full = bars;                                    // the query tile has landed
    uint64_t* k_full = bars + 1;                                // [K_STAGES] a key tile has landed
    uint64_t* k_empty = k_full + K_STAGES;                      // [K_STAGES] the score product that read it is done
    uint64_t* v_full = k_empty + K_STAGES;                      // [V_STAGES] a value tile has landed
    uint64_t* v_empty = v_full + V_STAGES;                      // [V_STAGES] the output product that read it is done
    uint64_t* s_full = v_empty + V_STAGES;                      // [2] a score buffer is complete
    // [2 groups][2 score buffers] a group's P of a tile is in tensor memory (and its O rescaled).  One barrier per score
    // buffer: a group may finish tile j + 1 before the issuing thread has looked at its tile j, and a barrier tells
    // only the last phase from the one before
    uint64_t* p_full = s_full + 2;
    uint64_t* pv_done = p_full + 4;                             // [2] a group's output product of a tile is done
    static_assert(1 + 2 * (K_STAGES + V_STAGES) + 8 <= 31, "the barriers and the two words behind them fit 256 bytes");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 31);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
    float* exchange = reinterpret_cast<float*>(bars + 32);      // [2 sets][2 groups][128 rows]: the groups' maxima of a tile, then their sums

    pdl_trigger();
    const int tile = blockIdx.x, head = blockIdx.y;
    const int req = tile_req[tile], q0 = tile_q0[tile];
    const int rows = min(BM, q_len[req] - q0);
    const int tok0 = q_start[req] + q0;
    const int ctx = ctx_len[req];
    const int qpos0 = ctx - q_len[req] + q0;
    const int kvh = head / (hq / hkv);
    const int* table = block_table + (size_t)req_slot[req] * table_width;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int k_end = qpos0 + rows;                                                       // the last row sees keys up to its own position
    const int k_begin = ((window > 0 ? max(0, qpos0 - window + 1) : 0) / BN) * BN;
    const int n_tiles = (k_end - k_begin + BN - 1) / BN;
    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < K_STAGES; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); }
        for (int s = 0; s < V_STAGES; ++s) { mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(s_full + s, 1);
            mbar_init(p_full + 2 * s, SOFTMAX_THREADS / 64);   // one arrival per warp of the group, by its first lane after the warp has met
            mbar_init(p_full + 2 * s + 1, SOFTMAX_THREADS / 64);
            mbar_init(pv_done + s, 1);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {    // two score buffers of 128 columns and the output: 512 columns, all of this SM's tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;
    pdl_wait();          // the queries, and this step's keys and values, come from the kernel before
    CISR_TRACE_WAITED();

    auto gave_up = [&]() {
        atomicExch(error, 5);
        *(volatile int*)abort_flag = 1;
    };
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {     // false: leave (this or another role gave up)
        if (mbar_test(bar, parity)) return true;                  // the usual case: the phase is over already
        if (*(volatile int*)abort_flag) return false;
        if (mbar_wait(bar, parity)) return true;
        gave_up();
        return false;
    };

    if (warp == 0 || warp == 2) {
        // ------------------------------------------------------------ producers: warp 0 the queries and the keys, warp 2 the values
        const bool values = warp == 2;
        const int stages = values ? V_STAGES : K_STAGES;
        uint64_t* full = values ? v_full : k_full;
        uint64_t* empty = values ? v_empty : k_empty;
        unsigned char* ring = values ? Vring : Kring;
        const CUtensorMap* map = values ? &map_v : &map_k;
        if (!values && lane == 0) {
            mbar_expect_tx(q_full, (uint32_t)Q_BYTES);
            for (int sub = 0; sub < NSUB; ++sub) tma_load_2d(Qs + sub * SUB_BYTES, &map_q, head * D + sub * 64, tok0, q_full);
        }
        const int box_rows = min(page_size, BN), boxes = BN / box_rows;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j % stages;
            bool ok = true;
            if (j >= stages) ok = wait(empty + s, ((j / stages) & 1) ^ 1);
            if (!__all_sync(0xffffffffu, ok)) break;
            if (lane == 0) mbar_expect_tx(full + s, (uint32_t)KV_BYTES);
            __syncwarp();
            for (int b = lane; b < NSUB * boxes; b += 32) {       // lane b: box b (64-column half, run of box_rows keys)
                const int i = b % boxes, sub = b / boxes;
                const int kpos = k_begin + j * BN + i * box_rows;
                const int page = kpos < k_end ? __ldg(table + kpos / page_size) : -1;     // the table is older than the kernel before
                const int row = page < 0 ? cache_rows : (page * hkv + kvh) * page_size + kpos % page_size;   // beyond the cache: zeros
                tma_load_2d(ring + s * KV_BYTES + sub * KV_SUB + i * box_rows * 128, map, sub * 64, row, full + s);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ products
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(BN);
            constexpr uint32_t idesc_o = umma_idesc(D) | UMMA_B_MN_MAJOR;
            auto score_product = [&](int j) -> bool {             // S(j) = Q K(j)^T into score buffer j & 1
                if (!wait(k_full + j % K_STAGES, (j / K_STAGES) & 1)) return false;
                tcgen05_fence_after();
                const unsigned char* Ks = Kring + (j % K_STAGES) * KV_BYTES;
#pragma unroll
                for (int kd = 0; kd < D / 16; ++kd) {             // 16 of the head's dimensions per step
                    const uint64_t desc_q = umma_desc(Qs + (kd >> 2) * SUB_BYTES) + 2 * (kd & 3);
                    const uint64_t desc_k = umma_desc(Ks + (kd >> 2) * KV_SUB) + 2 * (kd & 3);
                    umma_bf16(tmem_base + (uint32_t)((j & 1) * BN), desc_q, desc_k, idesc_s, kd != 0);
                }
                umma_commit(s_full + (j & 1));
                umma_commit(k_empty + j % K_STAGES);              // the key tile is free when these products are done
                return true;
            };
            // O_g += P_g(j) V(j)[keys 64 g ...]: half g of the tile's keys, with the P that group g left over the first
            // 32 columns of its own scores
            auto output_product = [&](int j, int g) {
                const unsigned char* Vs = Vring + (j % V_STAGES) * KV_BYTES;
                const uint32_t tmem_p = tmem_base + (uint32_t)((j & 1) * BN + g * HALF);
#pragma unroll
                for (int ks = 0; ks < HALF / 16; ++ks) {          // 16 keys per step: 8 columns of P, V two 8-row groups down
                    const uint64_t desc_v = umma_desc_mn_major(Vs + (g * HALF + ks * 16) * 128, KV_SUB);
                    umma_bf16_ts(tmem_o + (uint32_t)(g * D), tmem_p + 8 * ks, desc_v, idesc_o, (j | ks) != 0);
                }
                umma_commit(pv_done + g);
            };
            // Both score buffers are filled at the start.  Then, tile by tile: each half's output product as soon as its
            // P has arrived, and after both the scores of the tile two on, into the buffer that these output products
            // read P from: products run in the order they are issued, so the buffer is overwritten after it was read.
            bool ok = wait(q_full, 0) && score_product(0);
            if (ok && n_tiles > 1) ok = score_product(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = wait(v_full + j % V_STAGES, (j / V_STAGES) & 1);
                for (int g = 0; g < 2 && ok; ++g) {
                    ok = wait(p_full + 2 * g + (j & 1), (j >> 1) & 1);
                    if (!ok) break;
                    tcgen05_fence_after();
                    output_product(j, g);
                }
                if (!ok) break;
                umma_commit(v_empty + j % V_STAGES);
                if (j + 2 < n_tiles) ok = score_product(j + 2);
            }
        }
    } else {
        // ------------------------------------------------------------ softmax and output
        // Two groups of four warps, each a stream of its own: thread (group, r) has the keys [64 * group, 64 * group + 64)
        // of every tile for query row r, with its own running max and sum and its own output accumulator; nothing is
        // exchanged between the groups until the end, so one group's exponentials run while the other waits or stores.
        const int quarter = warp & 3;                              // the 32 tensor-memory lanes this warp may touch
        const int group = (warp - FIRST_SOFTMAX_WARP) >> 2;
        const int row = quarter * 32 + lane;
        const int qpos = qpos0 + row;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t tmem_own = tmem_o + lane_base + (uint32_t)(group * D);     // this thread's row of its group's accumulator
        const float scale2 = scale * LOG2E;
        auto softmax_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS) : "memory"); };
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        uint32_t raw[HALF];
        auto step = [&](int j) {
            if (ok) ok = __all_sync(0xffffffffu, wait(s_full + (j & 1), (j >> 1) & 1));
            if (!ok) return;
            const int kt = k_begin + j * BN;                       // the tile's first key
            const int k0 = kt + group * HALF;                     // this thread's first key
            // tiles on the diagonal, at the window's start and at the end of the keys need the per-element mask
            const bool edge = kt + BN - 1 > qpos0 || kt + BN > k_end || (window > 0 && kt <= qpos0 + BM - 1 - window);
            auto masked = [&](int kpos) { return kpos > qpos || kpos >= k_end || (window > 0 && kpos <= qpos - window); };
            const uint32_t s_addr = tmem_base + lane_base + (uint32_t)((j & 1) * BN + group * HALF);
            auto fetch = [&]() {
#pragma unroll
                for (int c0 = 0; c0 < HALF; c0 += 32) tmem_load32_nowait(s_addr + c0, raw + c0);
                tmem_load_wait();
                if (edge) {
#pragma unroll
                    for (int c = 0; c < HALF; ++c)
                        if (masked(k0 + c)) raw[c] = __float_as_uint(-INFINITY);
                }
            };
            uint32_t* packed = raw;                               // pair c / 2 takes the place of scores already used
            // P = 2^(s - m), rounded to bfloat16 for the product; the sum keeps the unrounded values; also the max of the scores
            auto exponentials = [&](float m_ref, float& mx_out) -> float {
                float sums[4] = {0.f, 0.f, 0.f, 0.f}, mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < HALF; c += 2) {
                    const float a = __uint_as_float(raw[c]), b = __uint_as_float(raw[c + 1]);
                    mx[0] = fmaxf(mx[0], a); mx[1] = fmaxf(mx[1], b);
                    const float p0 = fast_exp2(fmaf(a, scale2, -m_ref));       // -inf (masked) gives 0
                    const float p1 = fast_exp2(fmaf(b, scale2, -m_ref));
                    sums[(c >> 1) & 3] += p0 + p1;
                    __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
                    packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
                }
                mx_out = fmaxf(mx[0], mx[1]);
                return (sums[0] + sums[1]) + (sums[2] + sums[3]);
            };
            // One pass when the row already has a max in use: the exponentials are taken against it while the tile's own
            // max is found, and only a tile whose max turns out more than RESCALE_STEP above it is done again (from the
            // scores, which stay in tensor memory until P is written over them).  A warp with a row that has no max
            // yet (the first tile, or only masked keys so far) finds the max first.
            tcgen05_fence_after();
            fetch();
            const bool ahead = __all_sync(0xffffffffu, m_used != -INFINITY);
            float mx = -INFINITY, sum = 0.f;
            if (ahead) {
                sum = exponentials(m_used, mx);
            } else {
#pragma unroll
                for (int c = 0; c < HALF; ++c) mx = fmaxf(mx, __uint_as_float(raw[c]));
            }
            const float m_tile = mx * scale2;                     // the scale is positive: the max of the raw scores, scaled
            // the max in use moves only when it lags by more than RESCALE_STEP; the first finite max is taken as it is
            float alpha = 1.f;
            const bool moved = m_tile > m_used + RESCALE_STEP || (m_used == -INFINITY && m_tile > -INFINITY);
            if (moved) {
                alpha = m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_tile);
                m_used = m_tile;
            }
            const float m_ref = m_used == -INFINITY ? 0.f : m_used;
            if (!ahead) {
                float unused;
                sum = exponentials(m_ref, unused);
            } else if (__any_sync(0xffffffffu, moved)) {          // tensor-memory access is warp-wide: every lane does its row again
                fetch();
                float unused;
                sum = exponentials(m_ref, unused);
            }
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // the group's accumulator may be touched once its output product of the tile before is done; all lanes
                // go, most with alpha 1
                ok = __all_sync(0xffffffffu, wait(pv_done + group, (j - 1) & 1));
                if (!ok) return;
                tcgen05_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t acc[32];
                    tmem_load32(tmem_own + c0, acc);
#pragma unroll
                    for (int c = 0; c < 32; ++c) acc[c] = __float_as_uint(__uint_as_float(acc[c]) * alpha);
                    tmem_store32(tmem_own + c0, acc);
                }
            }
            l = l * alpha + sum;
            // the thread's P goes over the first half of its own scores, where the output product reads it as its A operand
#pragma unroll
            for (int c0 = 0; c0 < HALF / 2; c0 += 16) tmem_store16_nowait(s_addr + c0, packed + c0);
            tmem_store_wait();
            tcgen05_fence_before();
            if (kt + BN > k_end) {
                // Value rows beyond the last key were never written, or are left over from another request: they must
                // not meet the zero probabilities of those keys (0 * NaN).  Once the tile has landed, each group zeroes
                // those among the rows that its own output product reads.
                ok = __all_sync(0xffffffffu, wait(v_full + j % V_STAGES, (j / V_STAGES) & 1));
                if (!ok) return;
                unsigned char* Vs = Vring + (j % V_STAGES) * KV_BYTES;
                for (int e = (warp - FIRST_SOFTMAX_WARP - 4 * group) * 32 + lane; e < HALF * NSUB * 8; e += SOFTMAX_THREADS / 2) {
                    const int r = group * HALF + e / (NSUB * 8), c = e % (NSUB * 8);
                    if (kt + r >= k_end)
                        *reinterpret_cast<uint4*>(Vs + (c >> 3) * KV_SUB + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeroed rows before the tensor core reads them
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 2 * group + (j & 1));
        };
        for (int j = 0; j < n_tiles; ++j) step(j);
        if (ok) ok = wait(pv_done, (n_tiles - 1) & 1) && wait(pv_done + 1, (n_tiles - 1) & 1);
        const bool all_ok = __all_sync(0xffffffffu, ok);
        if (!all_ok) *(volatile int*)abort_flag = 1;
        // The two streams of a row meet: with m the larger of their maxima, out = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) /
        // (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)); each group writes half of the output columns.
        exchange[group * BM + row] = m_used;
        exchange[(2 + group) * BM + row] = l;
        softmax_sync();
        if (all_ok && !*(volatile int*)abort_flag) {
            tcgen05_fence_after();
            const float m0 = exchange[row], m1 = exchange[BM + row], m = fmaxf(m0, m1);
            const float w0 = m0 == -INFINITY ? 0.f : fast_exp2(m0 - m), w1 = m1 == -INFINITY ? 0.f : fast_exp2(m1 - m);
            const float total = exchange[2 * BM + row] * w0 + exchange[3 * BM + row] * w1;
            const float inv = total > 0.f ? 1.f / total : 0.f;
            const float f0 = w0 * inv, f1 = w1 * inv;
            bf16* dst = out + ((size_t)(tok0 + row) * hq + head) * D;
#pragma unroll 1
            for (int c0 = group * (D / 2); c0 < (group + 1) * (D / 2); c0 += 32) {
                uint32_t a0[32], a1[32];
                tmem_load32_nowait(tmem_o + lane_base + c0, a0);            // warp-wide, also for rows beyond the portion
                tmem_load32_nowait(tmem_o + lane_base + D + c0, a1);
                tmem_load_wait();
                if (row < rows) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 8 * q + 2 * e;
                            // a stream without keys for this row weighs nothing, whatever its accumulator holds
                            const float x0 = (w0 > 0.f ? __uint_as_float(a0[c]) * f0 : 0.f) + (w1 > 0.f ? __uint_as_float(a1[c]) * f1 : 0.f);
                            const float x1 = (w0 > 0.f ? __uint_as_float(a0[c + 1]) * f0 : 0.f) + (w1 > 0.f ? __uint_as_float(a1[c + 1]) * f1 : 0.f);
                            __nv_bfloat162 pair = __floats2bfloat162_rn(x0, x1);
                            w[e] = *reinterpret_cast<uint32_t*>(&pair);
                        }
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}
}  // namespace

CISR_EXPORT int cisr_attn_tcgen05_head_dim() { return D; }
CISR_EXPORT int cisr_attn_tcgen05_tile() { return BM; }
CISR_EXPORT void cisr_attn_tcgen05_set_pdl(int on) { g_pdl = on != 0; }

// `error_flag`: one zeroed int in device memory that the kernel sets (to 5) when one of its waits ran out.
CISR_EXPORT int cisr_attn_tcgen05_init(int* error_flag) {
    if (int status = tma_load_encoder()) return status;
    g_error = error_flag;
    return 0;
}

// 1 when the kernel takes this page size.
CISR_EXPORT int cisr_attn_tcgen05_ok(int page_size) {
    return page_size > 0 && page_size % 8 == 0 && (BN % page_size == 0 || page_size % BN == 0);
}

// Attention of portions: q, out [n_tokens, hq, D]; tiles of 128 queries given as (request, first query) pairs.
CISR_EXPORT int cisr_attn_prefill_tcgen05(const void* q, void* out, int n_tokens, const void* k_cache, const void* v_cache,
                                          int n_pages, const int* req_slot, const int* block_table, int table_width,
                                          const int* tile_req, const int* tile_q0, int n_tiles, const int* q_start,
                                          const int* q_len, const int* ctx_len, int hq, int hkv, int page_size, float scale,
                                          int window, void* stream) {
    if (n_tiles <= 0) return 0;
    if (!g_encode || !g_error) return -13;
    if (hq % hkv || !cisr_attn_tcgen05_ok(page_size)) return -2;
    const long long cache_rows = (long long)n_pages * hkv * page_size;
    if (cache_rows <= 0 || cache_rows >= (1ll << 31) || (((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q | (uintptr_t)out) & 15)) return -2;
    const int box_rows = page_size < BN ? page_size : BN;
    CUtensorMap map_q, map_k, map_v;
    int status = cached_map(&map_q, q, n_tokens, hq * D, BM, 64);
    if (status) return status;
    if ((status = cached_map(&map_k, k_cache, cache_rows, D, box_rows, 64))) return status;
    if ((status = cached_map(&map_v, v_cache, cache_rows, D, box_rows, 64))) return status;
    const size_t smem = SMEM_FIXED;
    static_assert(SMEM_FIXED <= 227 * 1024, "a CTA has 227 KB of shared memory");
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    return launch_kernel(attn_prefill_tcgen05_kernel, dim3(n_tiles, hq), dim3(THREADS), smem, (cudaStream_t)stream, g_pdl, map_q,
                         map_k, map_v, (bf16*)out, (int)cache_rows, req_slot, block_table, table_width, tile_req, tile_q0,
                         q_start, q_len, ctx_len, hq, hkv, page_size, scale, window, g_error);
}
