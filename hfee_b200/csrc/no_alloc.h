/* Entry point of the kernel library for callers that must not allocate GPU memory.
 *
 * This entry point has no counterpart in hostfog/hfee (a CPU program); it exists for users of
 * this library only.
 *
 * Who needs it: code that runs where cudaMalloc is forbidden or unsafe - a host that is in the
 * middle of capturing other work and cannot afford an allocation's implicit synchronisation, a
 * plug-in living inside somebody else's memory pool with a fixed budget, a real-time loop that
 * may not block on the driver.  The regular split-key decode attention
 * (hfee_attention_mma with num_splits > 1) needs a scratch buffer for its partial results that
 * such a caller has no means to provide.  Here the scratch is a fixed array inside the library.
 *
 * hfee_attention_decode_noalloc computes the same thing as hfee_attention_mma with
 * num_splits > 1: causal grouped-query attention over the paged cache for a batch in which no
 * request brings more new tokens than fit one query tile (in decoding: one each), the keys of
 * each request divided among `num_splits` CTAs and merged.  The caller passes inputs and the
 * output exactly as for hfee_attention_mma; the partial results live in a file-scope
 * `static __device__` array of HFEE_NOALLOC_SCRATCH_FLOATS floats (4 MiB), which every GPU that
 * loads the library holds until the process ends.
 *
 * Limits and rules
 *  - n_tokens * heads * num_splits * (head_dim + 2) must not exceed
 *    HFEE_NOALLOC_SCRATCH_FLOATS; larger requests are refused with HFEE_ERR_ARG and a message
 *    (hfee_last_error()).  Nothing is launched in that case.
 *  - The function calls no cudaMalloc, cudaFree or other allocating routine.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and remembers it per device.  Make that first call before any stream
 *    capture begins.
 *  - All calls share the one array, and it keeps what the last call left in it.  Nothing in it
 *    has to start at zero: every (token, head, split) cell a call later reads is first written
 *    by that call, empty key ranges included.  Two calls whose kernels overlap on the GPU (other
 *    streams, other threads) race on the array; run them one after the other on one stream.
 */
#pragma once

#include <cuda_runtime.h>

#define HFEE_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

/* Returns 0, or a negative HfeeError (see common.cuh).  Arguments as hfee_attention_mma, without
 * the scratch pointer:
 *   q [n_tokens, ld_q], out [n_tokens, ld_o]: bfloat16; k_pool, v_pool: bfloat16 pages
 *   [num_pages, kv_heads, page_size, head_dim]; block_table [*, max_pages], cu_tokens
 *   [requests + 1], slots [requests], context_before [requests]: int32 on the device. */
int hfee_attention_decode_noalloc(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                  const int* block_table, int max_pages, int page_size, const int* cu_tokens,
                                  const int* slots, const int* context_before, void* out, int ld_o,
                                  int n_tokens, int requests, int max_new, int heads, int kv_heads, int head_dim,
                                  float scale, int window, int num_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
