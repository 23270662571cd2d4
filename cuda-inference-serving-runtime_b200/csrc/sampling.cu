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
static bool g_pdl = false;

__device__ __forceinline__ void take(float v, int i, float& best, int& best_i) {
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
}

__global__ void __launch_bounds__(ARGMAX_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const long long* __restrict__ seed, const int* __restrict__ counter, int* __restrict__ out) {
    CISR_TRACE_SCOPE(TRACE_SAMPLE);
    __shared__ float s_val[SAMPLE_THREADS];
    __shared__ int s_idx[SAMPLE_THREADS];
    __shared__ float s_pre[SAMPLE_THREADS + 1];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * vocab;
    pdl_trigger();
    pdl_wait();                      // the logits come from the kernel before
    CISR_TRACE_WAITED();

    // argmax, lowest index on ties; also the softmax shift.  Rows that start on a 16-byte boundary are read four
    // logits at a time, several loads in flight per thread; the few logits behind the last whole four singly.
    float best = -INFINITY; int best_i = 0x7fffffff;
    const int quads = ((uintptr_t)x & 15) ? 0 : vocab / 4;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int q0 = tid; q0 < quads; q0 += 4 * ARGMAX_THREADS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = q0 + u * ARGMAX_THREADS;
            v[u] = q < quads ? x4[q] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = 4 * (q0 + u * ARGMAX_THREADS);
            take(v[u].x, i, best, best_i); take(v[u].y, i + 1, best, best_i);
            take(v[u].z, i + 2, best, best_i); take(v[u].w, i + 3, best, best_i);
        }
    }
    for (int i = 4 * quads + tid; i < vocab; i += ARGMAX_THREADS) take(x[i], i, best, best_i);
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
    }
    __syncthreads();                 // every warp has read its entry before the result takes entry 0's place
    if (tid == 0) { s_val[0] = best; s_idx[0] = best_i; }
    __syncthreads();
    const float mx = s_val[0];
    const int arg = s_idx[0] == 0x7fffffff ? 0 : s_idx[0];
    const float temp = temperature ? temperature[row] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) out[row] = arg;
        return;
    }
    __syncthreads();
    if (tid >= SAMPLE_THREADS) return;           // the rest is SAMPLE_THREADS threads' work

    // each thread owns one contiguous segment, summed left to right
    const int seg = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(tid * seg, vocab), end = min(begin + seg, vocab);
    const float inv_t = 1.f / temp;
    float sum = 0.f;
    for (int i = begin; i < end; ++i) sum += expf((x[i] - mx) * inv_t);
    s_val[tid] = sum;
    asm volatile("bar.sync 1, %0;" ::"n"(SAMPLE_THREADS) : "memory");
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) { s_pre[i] = run; run += s_val[i]; }
        s_pre[SAMPLE_THREADS] = run;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(SAMPLE_THREADS) : "memory");
    const float target = cisr_uniform((unsigned long long)seed[row], (unsigned long long)counter[row]) * s_pre[SAMPLE_THREADS];
    // the segment whose running range holds the target; the last non-empty one if rounding put the target past the end
    const bool mine = (begin < end) && (s_pre[tid] <= target) &&
                      (target < s_pre[tid + 1] || tid == SAMPLE_THREADS - 1 || min((tid + 1) * seg, vocab) >= vocab);
    if (mine) {
        float run = s_pre[tid];
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            run += expf((x[i] - mx) * inv_t);
            if (run > target) { pick = i; break; }
        }
        out[row] = pick;
    }
}

CISR_EXPORT int cisr_sample(const float* logits, int rows, int vocab, const float* temperature,
                            const long long* seed, const int* counter, int* out, void* stream) {
    if (rows <= 0) return 0;
    return launch_kernel(sample_kernel, dim3(rows), dim3(ARGMAX_THREADS), 0, (cudaStream_t)stream, g_pdl, logits, vocab, temperature,
                         seed, counter, out);
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
