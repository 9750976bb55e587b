/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference; it exists for two kinds of callers of
 * this library:
 *   - programs that hand all device memory to an arena of their own when they start, so that a
 *     later cudaMalloc by a library would simply fail;
 *   - latency-critical loops that must not call cudaMalloc or cudaFree while they run, because
 *     those calls may synchronise the whole device and take an unbounded time.
 * The ordinary entry point, ts_flash_decode, asks such a caller for a scratch buffer of a size
 * that depends on the batch; this one brings its own.
 *
 * ts_flash_decode_static computes exactly what ts_flash_decode computes (paged attention of one
 * query token per request over the request's keys, cut into num_splits parts along the keys, for
 * bfloat16 and head sizes 64 and 128), with the same arguments except the scratch pointer.
 * Inputs and outputs are still the caller's.  The partial results of the splits are kept in an
 * array that is part of the library's device image:
 *
 *   capacity  1,048,576 floats (4 MiB), see ts_flash_decode_static_capacity_floats().  Every GPU on
 *             which this library is loaded holds these 4 MiB until the process exits, whether or
 *             not this entry point is ever called.
 *   need      num_tokens * num_heads * num_splits * (head_dim + 2) floats when num_splits > 1,
 *             nothing when num_splits == 1.  Examples that fit: 8 tokens x 28 heads x 32 splits
 *             at head_dim 128; 64 tokens x 28 heads x 4 splits.
 *   too big   the call launches nothing and returns -5.
 *
 * Return value: 0 on success; -5 if the call needs more scratch than the array holds; another
 * negative code if an argument is refused (same codes as ts_flash_decode: -2 size, -3 alignment,
 * -4 argument); a positive cudaError_t if a CUDA call fails.
 *
 * It calls no cudaMalloc, cudaFree or any routine that allocates.  The first call on a device
 * (with that device current) looks up the array's device address with cudaGetSymbolAddress and
 * remembers it; make that first call during start-up, before any stream capture begins.
 * The CUDA runtime itself may load a kernel's code the first time that kernel is launched (lazy
 * module loading), which can take device memory outside this library's control: a caller for
 * whom that matters warms up each head size it will use with one call with num_splits > 1 at
 * start-up (that launches both kernels), or runs with CUDA_MODULE_LOADING=EAGER.
 *
 * All calls on a device share the one array and the array keeps what the last call left in it.
 * Nothing in it has to be cleared between calls: every slot the joining kernel reads is written
 * by the same call first.  Two calls whose kernels can overlap on the GPU (different streams, or
 * graph branches) race on the array; run them in one stream or order them yourself.
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long ts_flash_decode_static_capacity_floats(void);

int ts_flash_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                           const void* k_pages, const void* v_pages, const int* block_table,
                           int table_stride, const int* seq_of_token, const int* positions,
                           int num_tokens, int page_size, int num_heads, int num_kv_heads,
                           int head_dim, int window, float scale, int num_splits,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
