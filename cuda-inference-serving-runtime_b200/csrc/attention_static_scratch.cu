// Split decode attention with its scratch memory inside the library: see attention_static_scratch.h for
// who this is for and the rules of use.  The kernels are the engine's own (attention.cu is compiled into
// this library as well); only where the partial sums live differs.
#include <stdio.h>

#include "attention.cu"
#include "attention_static_scratch.h"

namespace {
// Partial sums and their (max, denominator) pairs of one call.  Device code could name this array
// directly; host code may not use the name as an address (it is a host-side stand-in), so the launcher
// asks the runtime for the device address once per device.
static __device__ __align__(256) float g_static_scratch[CISR_STATIC_SCRATCH_BYTES / sizeof(float)];

constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES] = {};

void explain(char* message, int message_len, const char* text) {
    if (message && message_len > 0) snprintf(message, (size_t)message_len, "%s", text);
}
}  // namespace

extern "C" __attribute__((visibility("default")))
int cisr_attn_decode_static(const void* q, void* out, const void* k_cache, const void* v_cache, const int* req_slot,
                            const int* block_table, int table_width, const int* dec_req, int n_dec,
                            const int* q_start, const int* ctx_len, int hq, int hkv, int page_size, float scale,
                            int window, int split_size, int n_splits, void* stream, char* message, int message_len) {
    if (n_dec <= 0) return 0;
    if (hq <= 0 || hkv <= 0 || hq % hkv || split_size <= 0 || n_splits <= 0 || page_size <= 0) {
        explain(message, message_len, "cisr_attn_decode_static: head counts, page size, split size and split count "
                                      "must be positive and hq a multiple of hkv");
        return CISR_STATIC_BAD_ARGUMENT;
    }
    const unsigned long long cells = (unsigned long long)n_dec * hq * n_splits;
    const unsigned long long need = cells * (D + 2);
    const unsigned long long limit = CISR_STATIC_SCRATCH_BYTES / sizeof(float);
    if (need > limit) {
        if (message && message_len > 0)
            snprintf(message, (size_t)message_len,
                     "cisr_attn_decode_static: %d requests x %d heads x %d key ranges need %llu floats of scratch, the "
                     "library holds %llu (%u bytes per GPU); use fewer key ranges or the entry point that takes "
                     "caller-owned scratch", n_dec, hq, n_splits, need, limit, CISR_STATIC_SCRATCH_BYTES);
        return CISR_STATIC_TOO_LARGE;
    }
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return (int)err;
    if (device < 0 || device >= MAX_DEVICES) {
        explain(message, message_len, "cisr_attn_decode_static: device ordinal beyond the 64 this library tracks");
        return CISR_STATIC_BAD_ARGUMENT;
    }
    if (!g_scratch_address[device]) {   // first call on this device: not inside a stream capture
        float* address = nullptr;
        err = cudaGetSymbolAddress((void**)&address, g_static_scratch);
        if (err != cudaSuccess) {
            explain(message, message_len, "cisr_attn_decode_static: cudaGetSymbolAddress failed for the scratch array");
            return (int)err;
        }
        g_scratch_address[device] = address;
    }
    float* partial = g_scratch_address[device];       // [n_dec, hq, n_splits, D]
    float* stats = partial + cells * D;                // [n_dec, hq, n_splits, 2]
    return cisr_attn_decode(q, out, k_cache, v_cache, req_slot, block_table, table_width, dec_req, n_dec, q_start,
                            ctx_len, partial, stats, hq, hkv, page_size, scale, window, split_size, n_splits, stream);
}
