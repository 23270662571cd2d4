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

constexpr int SAMPLE_THREADS = 256;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const long long* __restrict__ seed, const int* __restrict__ counter, int* __restrict__ out) {
    CISR_TRACE_SCOPE(TRACE_SAMPLE);
    __shared__ float s_val[SAMPLE_THREADS];
    __shared__ int s_idx[SAMPLE_THREADS];
    __shared__ float s_pre[SAMPLE_THREADS + 1];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * vocab;

    // argmax, lowest index on ties; also the softmax shift
    float best = -INFINITY; int best_i = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = x[i];
        if (v > best) { best = v; best_i = i; }
    }
    s_val[tid] = best; s_idx[tid] = best_i;
    __syncthreads();
    for (int s = SAMPLE_THREADS / 2; s; s >>= 1) {
        if (tid < s) {
            const float v = s_val[tid + s]; const int i = s_idx[tid + s];
            if (v > s_val[tid] || (v == s_val[tid] && i < s_idx[tid])) { s_val[tid] = v; s_idx[tid] = i; }
        }
        __syncthreads();
    }
    const float mx = s_val[0];
    const int arg = s_idx[0] == 0x7fffffff ? 0 : s_idx[0];
    const float temp = temperature ? temperature[row] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) out[row] = arg;
        return;
    }
    __syncthreads();

    // each thread owns one contiguous segment, summed left to right
    const int seg = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(tid * seg, vocab), end = min(begin + seg, vocab);
    const float inv_t = 1.f / temp;
    float sum = 0.f;
    for (int i = begin; i < end; ++i) sum += expf((x[i] - mx) * inv_t);
    s_val[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) { s_pre[i] = run; run += s_val[i]; }
        s_pre[SAMPLE_THREADS] = run;
    }
    __syncthreads();
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
    sample_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, vocab, temperature, seed, counter, out);
    return launch_status();
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
    decode_advance_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(token_ids, positions, ctx_len, counter, sampled, live, rows,
                                                               status_in, ring, ring_slots, step_index);
    return launch_status();
}

CISR_EXPORT float cisr_uniform_host(long long seed, long long counter) {
    return cisr_uniform((unsigned long long)seed, (unsigned long long)counter);
}
