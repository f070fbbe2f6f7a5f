/* A decode-attention entry point for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference (integemjack/sglang.c): it exists for
 * users of this library who run where cudaMalloc is not an option, for example inside a
 * plug-in or a real-time loop whose host forbids allocation after start-up, under a memory
 * budget that was fixed before this library was loaded, or from a thread that must not take
 * the allocator's locks.  Such callers still own their inputs and outputs; what they cannot
 * provide is the scratch memory the split-key attention kernel needs to merge its key
 * ranges.  Here that scratch is a fixed array inside the library itself.
 *
 * What to know before calling it:
 *   - The scratch is a file-scope device array of SGLC_NOALLOC_SCRATCH_BYTES (4,260,096 bytes).
 *     Every GPU on which the library is loaded holds it until the process exits.
 *   - Sizes must fit: T*H*n_splits*(D+2) floats <= SGLC_NOALLOC_MAX_WS_FLOATS and
 *     T*H <= SGLC_NOALLOC_MAX_COUNTERS; otherwise the call returns
 *     SGLC_NOALLOC_ERR_TOO_LARGE and launches nothing.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress).  Make that first call before any stream capture begins.
 *   - All calls share the one array, and it keeps what the last call left.  The part that
 *     must start at zero (the arrival counters) is cleared on the caller's stream at the
 *     start of every call.  Two calls that overlap on the GPU (different streams, or two
 *     host threads) race on the scratch and give wrong results: serialise them.
 *   - max_keys must cover every token: positions[t] + 1 <= max_keys.  The launch sizes its
 *     shared memory from it; a token beyond it is not computed: its output rows are zeros and
 *     a status word inside the scratch is set.  sglc_attention_decode_noalloc_check(stream)
 *     waits for the stream, returns SGLC_NOALLOC_ERR_POSITION if the word was set since the
 *     last check (and clears it), 0 otherwise; it allocates nothing either.
 *   - The table of looked-up addresses is filled without a lock; two host threads making a
 *     device's first call at the same moment both store the same value, which is harmless.
 *   - It calls no cudaMalloc, cudaFree or other allocating routine.
 * Arguments are those of sglc_attention_decode without the scratch pointers:
 *   q, out: bfloat16 rows [T][stride], heads side by side; cache: one layer's bfloat16 pages
 *   [n_pages][2][Hkv][page_size][D]; block_table: int32 [n_requests][bt_stride];
 *   token_req[t]: the block-table row of token t; positions[t]: its position (the last key it
 *   sees); max_keys: the most keys any token sees; n_splits: key ranges per (token, head), 1..32.
 * Returns 0, a cudaError_t value, or one of the negative codes below;
 * sglc_attention_decode_noalloc_error() turns any of them into text.
 */
#ifndef SGLC_ATTENTION_DECODE_NOALLOC_H
#define SGLC_ATTENTION_DECODE_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SGLC_NOALLOC_MAX_WS_FLOATS (1 << 20)
#define SGLC_NOALLOC_MAX_COUNTERS (1 << 14)
#define SGLC_NOALLOC_SCRATCH_BYTES (SGLC_NOALLOC_MAX_WS_FLOATS * 4 + SGLC_NOALLOC_MAX_COUNTERS * 4 + 256)
#define SGLC_NOALLOC_ERR_TOO_LARGE (-10)
#define SGLC_NOALLOC_ERR_SETUP (-11)
#define SGLC_NOALLOC_ERR_POSITION (-12)

int sglc_attention_decode_noalloc(const void* q, int q_stride, const void* cache,
                                  const int* block_table, int bt_stride, const int* token_req,
                                  const int* positions, void* out, int o_stride, int T, int H,
                                  int Hkv, int D, int page_size, float scale, int window,
                                  int max_keys, int n_splits, cudaStream_t stream);

int sglc_attention_decode_noalloc_check(cudaStream_t stream);

const char* sglc_attention_decode_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
#endif
