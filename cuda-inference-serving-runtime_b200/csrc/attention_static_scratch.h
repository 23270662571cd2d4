// Split decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in nehanmohammed19/cuda-inference-serving-runtime; it is an
// addition of this engine.
//
// Who needs it.  The split decode attention writes one partial sum per (request, query head, key
// range) and merges them afterwards, so it needs scratch memory beyond its inputs and outputs.  The
// engine's own entry point (cisr_attn_decode) takes that scratch from the caller, who gets it from an
// allocator.  Some callers have no allocator to ask: code that runs inside another runtime's callback
// or plugin slot where cudaMalloc is forbidden (it synchronises the device and may fail late), code
// bound by a fixed memory budget that was handed out at start-up, and hosts that drive the kernels from
// a language binding without any tensor library.  For them the scratch lives inside this library, in a
// file-scope `static __device__` array of CISR_STATIC_SCRATCH_BYTES bytes.  Every GPU on which the
// library is loaded holds that array from load until the process exits, whether or not it is used.
//
// What the caller still passes: queries, the output, the key and value caches, block tables and the
// per-request arrays, exactly as for cisr_attn_decode.  What it no longer passes: `partial` and `stats`.
//
// Rules.
//  * The call allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and remembers it for that device.  Make this first call before any stream capture.
//    The remembered addresses are filled in without a lock: two host threads that make the first call on
//    one device at the same moment both look the address up and both store the same value, which is
//    harmless; nothing else about the entry point is shared between host threads but the array itself.
//  * Sizes whose partial sums do not fit are refused: the call returns CISR_STATIC_TOO_LARGE and, if
//    `message` is given, writes a sentence there that names the need and the limit.
//        need = n_dec * hq * n_splits * (head_dim + 2) floats  <=  CISR_STATIC_SCRATCH_BYTES / 4
//  * All calls share the one array, which keeps whatever the last call left.  Nothing in it has to start
//    at zero: every cell the merge reads is written by the same call first (an empty key range writes a
//    zero denominator, which the merge skips).  Two calls that overlap on the GPU (different streams, or
//    graphs replayed concurrently) race on the array and give wrong results: keep calls on one device in
//    stream order.
//
// The library is built per head size and storage type like the engine's attention library
// (-DHEAD_DIM=<multiple of 16 up to 256> -DSTORAGE_BF16=<0|1>); q, out and the caches have that type.
#pragma once

#define CISR_STATIC_SCRATCH_BYTES (8u << 20)   // 8 MiB per GPU
#define CISR_STATIC_TOO_LARGE (-4)
#define CISR_STATIC_BAD_ARGUMENT (-2)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, CISR_STATIC_BAD_ARGUMENT, CISR_STATIC_TOO_LARGE, or a positive cudaError_t.
// `message` (may be null) receives a zero-terminated explanation of a refusal, at most message_len bytes.
int cisr_attn_decode_static(const void* q, void* out, const void* k_cache, const void* v_cache, const int* req_slot,
                            const int* block_table, int table_width, const int* dec_req, int n_dec,
                            const int* q_start, const int* ctx_len, int hq, int hkv, int page_size, float scale,
                            int window, int split_size, int n_splits, void* stream, char* message, int message_len);

#ifdef __cplusplus
}
#endif
