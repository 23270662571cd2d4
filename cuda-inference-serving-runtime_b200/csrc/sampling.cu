// Token selection on the device: greedy argmax (lowest index on ties) and
// temperature sampling by inverse CDF with a counter-based uniform.
//
// Parity: the reference selects greedily only (runtime/engine.py:99, an argmax on
// the device followed by a copy to the host).  Temperature sampling is this engine's
// own: p = softmax(logits / T) in float, u = uniform(seed, counter), token = first
// index whose running sum of p exceeds u * sum(p).  The uniform depends only on the
// request's seed and on how many tokens it has sampled, never on the batch.
#include "common.cuh"

__host__ __device__ inline float cisr_uniform(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);  // 24 random bits: [0, 1)
}

constexpr int SAMPLE_THREADS = 256;     // threads that take part in the inverse CDF (one contiguous segment each)
constexpr int ARGMAX_THREADS = 1024;    // threads of the block; all of them scan for the largest logit
constexpr int MAX_PARTS = 8;            // CTAs that share a row, as one thread-block cluster
constexpr int PART_LOGITS = 16384;      // logits per CTA: one batch of 16-byte loads per thread, one trip to memory
static bool g_pdl = false;

__device__ __forceinline__ void take(float v, int i, float& best, int& best_i) {
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
}
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t shared_of_rank(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void store_cluster(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void store_cluster(uint32_t addr, int v) { asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
// Every thread of every CTA of the cluster arrives (no thread leaves the kernel before the last of these).
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One row per cluster of gridDim.z CTAs; CTA c scans logits [c * part, (c + 1) * part) (`part` a multiple of 4).  The
// CTAs tell one another their largest logit (and, when sampling, their sum of exponentials) through distributed
// shared memory, so every CTA knows the row's maximum and where its own share of the cumulative distribution begins;
// the CTA whose share holds the target picks the token.  How a row is cut depends on the vocabulary alone, never on
// the batch, so a request draws the same token whatever else is in the step.
__global__ void __launch_bounds__(ARGMAX_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, int part, const float* __restrict__ temperature,
              const long long* __restrict__ seed, const int* __restrict__ counter, int* __restrict__ out) {
    CISR_TRACE_SCOPE(TRACE_SAMPLE);
    __shared__ float s_val[SAMPLE_THREADS];
    __shared__ int s_idx[SAMPLE_THREADS];
    __shared__ float s_pre[SAMPLE_THREADS + 1];
    __shared__ float c_val[MAX_PARTS];            // every CTA's largest logit ...
    __shared__ int c_idx[MAX_PARTS];              // ... and where it is
    __shared__ float c_tot[MAX_PARTS];            // every CTA's sum of exponentials
    const int row = blockIdx.x, tid = threadIdx.x;
    const int rank = (int)cluster_rank(), ranks = (int)cluster_size();
    const float* x = logits + (size_t)row * vocab;
    const int lo = min(rank * part, vocab), hi = min(lo + part, vocab), n = hi - lo;
    pdl_trigger();
    pdl_wait();                      // the logits come from the kernel before
    CISR_TRACE_WAITED();

    // argmax of the CTA's share, lowest index on ties; also the softmax shift.  Rows that start on a 16-byte boundary
    // are read four logits at a time, several loads in flight per thread; the few logits behind the last whole four
    // singly.
    float best = -INFINITY; int best_i = 0x7fffffff;
    const float* xs = x + lo;
    const int quads = ((uintptr_t)xs & 15) ? 0 : n / 4;
    const float4* x4 = reinterpret_cast<const float4*>(xs);
    for (int q0 = tid; q0 < quads; q0 += 4 * ARGMAX_THREADS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = q0 + u * ARGMAX_THREADS;
            v[u] = q < quads ? x4[q] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = lo + 4 * (q0 + u * ARGMAX_THREADS);
            take(v[u].x, i, best, best_i); take(v[u].y, i + 1, best, best_i);
            take(v[u].z, i + 2, best, best_i); take(v[u].w, i + 3, best, best_i);
        }
    }
    for (int i = lo + 4 * quads + tid; i < hi; i += ARGMAX_THREADS) take(x[i], i, best, best_i);
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, best, o);
        const int i = __shfl_xor_sync(0xffffffffu, best_i, o);
        take(v, i, best, best_i);
    }
    if ((tid & 31) == 0) { s_val[tid >> 5] = best; s_idx[tid >> 5] = best_i; }
    __syncthreads();
    if (tid < 32) {
        best = tid < ARGMAX_THREADS / 32 ? s_val[tid] : -INFINITY;
        best_i = tid < ARGMAX_THREADS / 32 ? s_idx[tid] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float v = __shfl_xor_sync(0xffffffffu, best, o);
            const int i = __shfl_xor_sync(0xffffffffu, best_i, o);
            take(v, i, best, best_i);
        }
        if (tid < ranks) {           // lane c tells CTA c
            store_cluster(shared_of_rank(c_val + rank, (uint32_t)tid), best);
            store_cluster(shared_of_rank(c_idx + rank, (uint32_t)tid), best_i);
        }
    }
    cluster_barrier();               // every CTA's entry has arrived in every CTA
    float mx = -INFINITY; int arg = 0x7fffffff;
    for (int c = 0; c < ranks; ++c) take(c_val[c], c_idx[c], mx, arg);
    if (arg == 0x7fffffff) arg = 0;
    const float temp = temperature ? temperature[row] : 0.f;
    if (!(temp > 0.f)) {             // the same for every CTA of the row: nothing of another CTA is touched after this
        if (rank == 0 && tid == 0) out[row] = arg;
        return;
    }

    // each of SAMPLE_THREADS threads owns one contiguous segment of the CTA's share, summed left to right
    const int seg = (n + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = lo + min(tid * seg, n), end = min(begin + seg, hi);
    const float inv_t = 1.f / temp;
    if (tid < SAMPLE_THREADS) {
        float sum = 0.f;
        for (int i = begin; i < end; ++i) sum += expf((x[i] - mx) * inv_t);
        s_val[tid] = sum;
    }
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) { s_pre[i] = run; run += s_val[i]; }
        s_pre[SAMPLE_THREADS] = run;
    }
    __syncthreads();
    if (tid < ranks) store_cluster(shared_of_rank(c_tot + rank, (uint32_t)tid), s_pre[SAMPLE_THREADS]);
    cluster_barrier();               // the last access to another CTA's memory; every thread is still here
    float offset = 0.f, grand = 0.f;                 // the same running sum in every CTA: the shares tile [0, grand)
    for (int c = 0; c < ranks; ++c) { if (c == rank) offset = grand; grand += c_tot[c]; }
    const float target = cisr_uniform((unsigned long long)seed[row], (unsigned long long)counter[row]) * grand;
    // the CTA whose share holds the target; the last one with logits if rounding put the target past the end
    const int last_cta = (vocab - 1) / part;
    const bool cta_mine = n > 0 && offset <= target && (target < offset + c_tot[rank] || rank == last_cta);
    if (!cta_mine || tid >= SAMPLE_THREADS) return;
    const float local = target - offset;
    // the segment whose running range holds the target; the last non-empty one if rounding put the target past the end
    const bool mine = (begin < end) && (s_pre[tid] <= local) &&
                      (local < s_pre[tid + 1] || tid == SAMPLE_THREADS - 1 || min((tid + 1) * seg, n) >= n);
    if (mine) {
        float run = s_pre[tid];
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            run += expf((x[i] - mx) * inv_t);
            if (run > local) { pick = i; break; }
        }
        out[row] = pick;
    }
}

CISR_EXPORT int cisr_sample(const float* logits, int rows, int vocab, const float* temperature,
                            const long long* seed, const int* counter, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return -2;
    int parts = (vocab + PART_LOGITS - 1) / PART_LOGITS;
    if (parts > MAX_PARTS) parts = MAX_PARTS;
    const int part = ((vocab + parts - 1) / parts + 3) & ~3;          // whole groups of four, so every share starts aligned
    return launch_kernel_cluster(sample_kernel, dim3(rows, 1, parts), dim3(ARGMAX_THREADS), 0, (cudaStream_t)stream, g_pdl, parts, logits,
                                 vocab, part, temperature, seed, counter, out);
}

// After a decode step whose tokens were chosen on the device: feed each live row's token back as its next
// input and move its position, context length and sample counter on by one, so the next step can run without
// the host.  Rows with live == 0 (padding) stay as they are.
// With `ring` ([ring_slots][rows + 1] ints) the sampled tokens of all rows and, behind them, *status_in (the kernels'
// "gave up on a wait" flag) are also written to slot (*step_index % ring_slots), and *step_index moves on by one: the
// host copies a slot out while later steps, which write other slots, already run.  One block; any number of rows.
__global__ void decode_advance_kernel(int* token_ids, int* positions, int* ctx_len, int* counter,
                                      const int* __restrict__ sampled, const int* __restrict__ live, int rows,
                                      const int* status_in, int* ring, int ring_slots, int* step_index) {
    CISR_TRACE_SCOPE(TRACE_DECODE_ADVANCE);
    pdl_trigger();
    pdl_wait();                                    // the sampled tokens come from the kernel before
    int* slot = nullptr;
    if (ring) {
        slot = ring + (size_t)(*step_index % ring_slots) * (rows + 1);
        __syncthreads();                           // every thread has read the index before thread 0 moves it on
        if (threadIdx.x == 0) { *step_index += 1; slot[rows] = status_in ? *status_in : 0; }
    }
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        if (slot) slot[i] = sampled[i];
        if (!live[i]) continue;
        token_ids[i] = sampled[i];
        positions[i] += 1;
        ctx_len[i] += 1;
        counter[i] += 1;
    }
}

CISR_EXPORT int cisr_decode_advance(int* token_ids, int* positions, int* ctx_len, int* counter, const int* sampled,
                                    const int* live, int rows, const int* status_in, int* ring, int ring_slots,
                                    int* step_index, void* stream) {
    if (rows <= 0) return 0;
    if (ring && (ring_slots <= 0 || !step_index)) return -2;
    return launch_kernel(decode_advance_kernel, dim3(1), dim3(128), 0, (cudaStream_t)stream, g_pdl, token_ids, positions, ctx_len,
                         counter, sampled, live, rows, status_in, ring, ring_slots, step_index);
}

CISR_EXPORT void cisr_sampling_set_pdl(int on) { g_pdl = on != 0; }

CISR_EXPORT float cisr_uniform_host(long long seed, long long counter) {
    return cisr_uniform((unsigned long long)seed, (unsigned long long)counter);
}
