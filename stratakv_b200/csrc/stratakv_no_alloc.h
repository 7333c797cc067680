/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference engine (Mourya05/StrataKV): it
 * exists for hosts that drive the kernels from a context in which cudaMalloc is off
 * limits, for example a plug-in that runs inside another program's memory budget, a
 * real-time loop that must not enter the allocator, or a process whose device memory
 * was all handed to one pool at start-up and that has no way to ask that pool for more.
 * Such a caller still owns the tensors it passes (queries, the paged key and value cache,
 * the block table, the lengths, the output), but the split form of decode attention also
 * needs room for each split's partial result.  Here that room is a fixed array inside the
 * library's device image, so the call allocates nothing: it calls neither cudaMalloc nor
 * cudaFree nor any library routine that could.
 *
 * What this costs and what to watch for:
 *   - Every GPU that loads the library holds the array (4.5 MiB) until the process ends.
 *   - A call needs n_seqs * num_heads * splits * (head_dim + 2) floats; the array holds
 *     skv_attention_decode_no_alloc_capacity() of them.  A larger request is refused with
 *     a message that names both numbers; nothing is launched then.
 *   - The first call on a device looks up the array's device address (it is not the
 *     address the name has in host code) and sets a kernel attribute.  Make that first
 *     call outside any CUDA stream capture, with the device current.
 *   - All calls share the one array and it keeps what the last call left there.  The kernels
 *     write every slot they later read, so stale contents do no harm, but two calls that
 *     overlap on the GPU (different streams, or graphs replayed side by side) race on it.
 *     Serialise them.  On the host side the entry point may be called from several threads:
 *     its per-device set-up is done under a lock.  That lock orders host threads only; it
 *     does nothing about two calls whose kernels overlap on the GPU.
 *
 * Arguments are those of skv_attention_decode without the two scratch pointers: bfloat16
 * q [n_seqs, num_heads * head_dim], the cache of one layer [blocks][kv_heads][block_size]
 * [head_dim], int32 block_table [n_seqs, table_width], int32 ctx_after [n_seqs] (keys
 * cached for each sequence, the query's own included), bfloat16 out like q.  Returns 0, or
 * non-zero after recording a message that skv_last_error() returns.  Only the bfloat16
 * build of the library implements it, for the head size that build was compiled for.
 */
#ifndef STRATAKV_NO_ALLOC_H
#define STRATAKV_NO_ALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long skv_attention_decode_no_alloc_capacity(void);

int skv_attention_decode_no_alloc(const void* q, const void* k_cache, const void* v_cache,
                                  const int* block_table, int table_width, const int* ctx_after, void* out,
                                  int n_seqs, int num_heads, int num_kv_heads, int head_dim, int block_size,
                                  float scale, int window, int splits, cudaStream_t stream);

const char* skv_last_error(void);

#ifdef __cplusplus
}
#endif

#endif
