/* Entry points of libti_sm100 that never allocate. They have no counterpart in the reference
 * project (tinyInfer allocates its FlashDecoding partials on every call, tinyinfer/csrc/bind.cpp:195-211).
 *
 * For callers that may not allocate device memory: a plugin running inside another runtime's
 * capture region or callback, an engine that has given all free memory to its cache, a host with a
 * no-allocation rule after start-up. The call issues kernel launches and nothing else: no
 * cudaMalloc, no cudaFree, no allocating library routine.
 *
 * Limit: the partial results live in an 8 MB array built into the library (one copy on every GPU
 * that loads it, held until exit), so
 *     ti_attention_decode_scratch_floats(num_rows, hq, hkv, d, max_context, window)
 *         <=  ti_attention_decode_noalloc_capacity()
 * must hold (about (1.75 * SMs + num_rows * hkv) * (hq / hkv) * (d + 2) floats: 471 requests with
 * Qwen3-8B's 32 query and 8 kv heads of size 128); larger calls are refused with a message (return value
 * != 0, text from ti_last_error()).
 * The first call on a device does set-up work that later calls do not: it resolves the array's device
 * address, may make the driver load this library's code and its 8 MB array onto that device, and
 * raises the kernel's shared-memory limit there. Make that call at start-up, before any stream
 * capture and before the region in which allocation is forbidden begins. Calls on one device share
 * the array: order them on one stream, or they race.
 */
#ifndef TINYINFER_B200_NOALLOC_H
#define TINYINFER_B200_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Floats of built-in scratch (2 Mi). */
long long ti_attention_decode_noalloc_capacity(void);
/* Floats of scratch a call with these arguments needs. */
long long ti_attention_decode_scratch_floats(int num_rows, int hq, int hkv, int d, int max_context, int window);

/* Paged attention for single decoded tokens, bfloat16, head_dim 64 or 128.
 * out [T, Hq * D] and q [T, Hq, D] are the step's flat token rows; only the rows listed in
 * `rows` (num_rows of them, each the one new token of its request) are read and written.
 * kv_cache [2, num_pages, Hkv, page_size, D]; block_table int32 [requests, max_blocks] (-1: no page);
 * positions / token_seq int32 [T]: position of each row in its request, and its request's row in
 * block_table. max_context: an upper bound of the rows' contexts (it sizes the launch only). rows,
 * positions, token_seq, block_table and the keys and values of all positions before each row's own are
 * read before the kernels wait for the work ahead of them in the stream: they must be complete when the
 * call is made (the kernels launched just before may write q and the keys and values at the rows' own
 * positions). status: optional device int set on a bounded wait that ran out. Same results as
 * ti_attention_decode_bf16. */
int ti_attention_decode_bf16_noalloc(void* out, const void* q, const void* kv_cache, const int* rows,
                                     int num_rows, const int* positions, const int* token_seq,
                                     const int* block_table, int max_blocks, int hq, int hkv, int d,
                                     int page_size, int num_pages, float scale, int window, int max_context,
                                     int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
