/* Allocation-free decode attention.
 *
 * This entry point has no counterpart in umarhassan-cloud/kvforge: it exists for callers of
 * this library that are not in a position to allocate device memory.
 *
 * Who that is.  Some hosts hand a GPU library a fixed set of buffers and forbid it to ask the
 * driver for more: a plugin that runs inside another runtime's enqueue call, a serving
 * process whose whole device budget was carved up at start-up, a control loop that must not
 * hit the implicit device-wide synchronisation that cudaMalloc and cudaFree can bring.  The
 * regular split-KV decode attention of this library needs a float scratch area for the
 * partial results of its key ranges, which the regular caller allocates.  The function below
 * does the same computation but keeps that scratch in a fixed array that is part of the
 * library image itself, so the caller passes inputs and outputs and nothing else.
 *
 * What it costs.  The array is KVF_NOALLOC_SCRATCH_BYTES large and lives in every GPU context
 * that loads libkvforge_b200_noalloc.so, from load until the process exits.  A problem whose
 * partial results do not fit is refused (see below); nothing is ever allocated to make room.
 *
 * Rules of use.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and remembers it.  Make that first call outside any stream capture.
 *  - All calls share the one array, and it keeps whatever the last call left in it.  No part
 *    of it has to start at zero: a call writes every (maximum, sum) pair it later reads and
 *    never reads the weighted sums of a key range it found empty.  But two calls that are in
 *    flight on the GPU at the same time (different streams, or different host threads on
 *    streams that do not order them) would overwrite each other's partial results: keep calls
 *    on one device ordered.
 *  - It calls no cudaMalloc, cudaFree or allocating library routine.
 */
#ifndef KVFORGE_NOALLOC_H
#define KVFORGE_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Size of the built-in scratch array: 8 MiB. */
#define KVF_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)

/* Return codes beyond cudaError values. */
#define KVF_NOALLOC_TOO_LARGE (-2) /* the partial results would not fit in the built-in scratch */
#define KVF_NOALLOC_BAD_ARGUMENT (-3)

/* Paged grouped-query attention for one query token per sequence (decoding), bfloat16.
 *
 *   q            [B rows of q_stride elements]; the first nh*d of a row are the query heads
 *   out          [B rows of out_stride elements]
 *   kcache/vcache  [num_blocks][nkv][block_size][d]
 *   block_tables [B][bt_stride] page numbers; qsl [B+1] = 0,1,..,B; ctx_lens [B] keys per sequence
 *   d in {64, 128}; nh/nkv <= 16; split_size a multiple of 64; max_context >= every ctx_lens[b]
 *
 * Needs B * nh * ceil(max_context / split_size) * (d + 2) floats of scratch; returns
 * KVF_NOALLOC_TOO_LARGE if that exceeds KVF_NOALLOC_SCRATCH_BYTES.  Returns 0 on success, a
 * cudaError value if the launch failed.  kvf_noalloc_last_error() describes the last refusal
 * on the calling thread. */
int kvf_paged_attention_decode_noalloc_bf16(const void* q, void* out, const void* kcache, const void* vcache,
                                            const int* block_tables, const int* qsl, const int* ctx_lens, int B,
                                            int q_stride, int out_stride, int bt_stride, int nh, int nkv, int d,
                                            int block_size, float scale, int window, int split_size,
                                            int max_context, cudaStream_t stream);

const char* kvf_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
