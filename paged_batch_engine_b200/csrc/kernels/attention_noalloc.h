/* Paged attention with key splits for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference engine (Destination2020/
 * Paged-Batch-Engine); it is an addition of this library.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a plugin inside a host
 * application that owns the whole device heap and forbids further allocation, a
 * latency-critical loop that must not take the allocator's lock, a process whose memory
 * budget was fixed at start-up.  The regular entry points (pbe_attn_simple followed by
 * pbe_attn_merge) expect the caller to bring two scratch buffers for the partial results
 * of split key ranges; such a caller has nowhere to get them from.  Here the scratch is a
 * fixed array inside the library itself.
 *
 * Contract
 *  - The caller passes the same arguments as to pbe_attn_simple and pbe_attn_merge; the
 *    part_o / part_ml pointers inside them are ignored and replaced by the library's own
 *    scratch.  Inputs and outputs stay the caller's.
 *  - Limit: split_rows * num_heads * max_splits * (head_dim + 2) floats must not exceed
 *    PBE_NOALLOC_SCRATCH_FLOATS (2 Mi floats = 8 MiB).  Larger requests are refused with
 *    cudaErrorInvalidValue and a message on stderr; nothing is launched.
 *  - The array is part of the library image: every GPU on which the library is loaded
 *    holds these 8 MiB until the process exits.
 *  - The first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress) with that device current and keeps it; make that first call
 *    outside any stream capture.  Later calls only launch kernels.
 *  - No cudaMalloc, cudaFree or allocating library routine is called, on any call.
 *  - All calls share the one array, and it keeps what the last call wrote.  Nothing in it
 *    has to start at zero: every partial that the merge reads was written by the attention
 *    kernel of the same call.  Two calls whose kernels overlap on the GPU (different
 *    streams, or several host threads) race on the array; serialise them.
 *  - Returns 0 or a cudaError_t value.
 */
#pragma once
#include <cuda_runtime.h>

#include "attention_params.cuh"

#define PBE_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif
int pbe_attn_simple_noalloc(const AttnParams* attn, int num_work, const AttnMergeParams* merge,
                            int split_rows, int dtype, cudaStream_t stream);
/* PBE_NOALLOC_SCRATCH_FLOATS as the loaded library was built with. */
long long pbe_attn_noalloc_scratch_floats(void);
#ifdef __cplusplus
}
#endif
