/* Decode attention without any allocation — an entry point for hosts that may not call cudaMalloc.
 *
 * This entry point has no counterpart in the reference (1483795887/qwen3_from_scratch); it exists for
 * users of this library whose process cannot allocate device memory when the call is made:
 * a serving loop that has handed all of the GPU's memory to its cache pool and weights at start-up,
 * a plug-in that runs inside another program's memory budget and must not grow it, or code that
 * runs where an allocation would synchronise the device or fail the real-time deadline of the step.
 * The ordinary entry point, q3_attn_decode, needs a float32 scratch buffer from its caller for the
 * partial results of the key ranges ("splits"); here that scratch is a fixed array inside the
 * library image instead.
 *
 *   - The array holds q3_attn_decode_noalloc_capacity() floats (4 Mi floats = 16 MiB).  Every GPU on
 *     which the library is loaded carries these 16 MiB from load until the process exits, whether or
 *     not this function is ever called.
 *   - A call needs B * Hq * num_splits * (D + 2) floats when num_splits > 1, none when it is 1.
 *     A call that needs more than the capacity is refused with -4 and launches nothing; use fewer
 *     splits or the ordinary entry point.
 *   - The first call on a device asks the CUDA runtime for the array's device address
 *     (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call on each
 *     device before any stream capture begins, and from one thread.  The address is kept for the life
 *     of the process: after cudaDeviceReset (or anything else that tears the device's context down) it
 *     is stale, and this entry point must not be called on that device again.
 *   - All calls share the one array, and it keeps whatever the last call left in it.  Nothing has to
 *     be zero at the start: every split writes its whole record (output, maximum, denominator) before
 *     the merging kernel reads it.  Two calls whose kernels can overlap on the GPU (different
 *     streams, or one stream and a graph that is replayed beside it) race on the array; keep calls
 *     that use it in one stream order.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, by this function or by
 *     anything it calls.
 *
 * Arguments, results and refusals are those of q3_attn_decode (attn_decode.cu) without `partial`:
 *   q, out      bfloat16 [T, Hq, D]; the token of sequence b is row q_start[b]
 *   k_pages,
 *   v_pages     bfloat16 [num_pages, Hkv, page_size, D]
 *   q_start     int32 [B] (one token per sequence), kv_len int32 [B], block_table int32 [B, table_stride]
 *   status      int32 device word that kernels OR error bits into
 * Returns 0, a cudaError_t, or a negative refusal (-2 size, -3 alignment, -4 scratch too small).
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long q3_attn_decode_noalloc_capacity(void);

int q3_attn_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, void* out, const int* q_start,
                           const int* kv_len, const int* block_table, int table_stride, int page_size,
                           int num_pages, int B, int Hq, int Hkv, int D, float scale, int window, int num_splits,
                           int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
