/* Greedy token selection that never allocates: swb_argmax_static().
 *
 * This entry point has no counterpart in the reference project; it exists for callers that are not allowed to
 * allocate when they pick the next token: a decode loop recorded by someone else's runtime, a plugin called from
 * inside another framework's allocator lock, a real-time thread that must not reach the CUDA memory manager, or a
 * host without torch that has nowhere to keep a scratch tensor alive. swb_argmax() asks such callers for a scratch
 * buffer; this variant brings its own.
 *
 * What it does: out_ids[r] = index of the largest value in row r of `logits` (ties go to the lowest index, NaN never
 * wins, a row with no candidate gives 0); out_vals[r] (optional) = that value. `allow_mask` (optional, uint8 [V],
 * 1 = allowed) restricts the candidates. Every row is split into chunks reduced by separate thread blocks; the
 * last block to finish a row merges the chunk results, so one launch does the whole job.
 *
 * Memory: the chunk results and one arrival counter per row live in a fixed array inside the library image
 * (SWB_ARGMAX_STATIC_SCRATCH_BYTES = 397,312 bytes per device). The function calls no cudaMalloc / cudaFree /
 * cudaMallocAsync and no library routine that does, on any call. The caller owns logits, allow_mask, out_ids and
 * out_vals.
 *
 * Limits: 1 <= rows <= SWB_ARGMAX_STATIC_MAX_ROWS (1024) and 1 <= V; anything else returns
 * SWB_ARGMAX_STATIC_E_SIZE (and prints one line to stderr) without launching. rows == 0 returns 0.
 *
 * First call on a device: looks up the array's device address (cudaGetSymbolAddress, with that device current) and
 * remembers it; this may load the library's device code. Make that first call outside any stream capture; later
 * calls only launch one kernel on `stream`.
 *
 * Sharing: all calls on a device use the same array. Calls on one stream are ordered and safe. Calls that may
 * overlap (two streams, two threads without ordering) race on it and give wrong tokens. The array keeps whatever
 * the previous call left in its chunk slots; that is harmless because a call writes every slot before it reads it.
 * The arrival counters must be zero when a call starts: they are zero when the library is loaded and every call
 * puts them back to zero before it ends, so the caller never clears anything.
 *
 * After a failure: a launch that does not run to completion (a sticky device fault in this or an earlier kernel, the
 * context torn down under it) can leave arrival counters non-zero, and nothing in this interface clears them; the
 * device is then only usable again from a new process (a fresh load of the library image zeroes the array).
 * cudaDeviceReset() destroys the array whose address was remembered on the first call: after it, do not call this
 * function on that device again in the same process.
 *
 * V may be any value from 1 to INT_MAX (index arithmetic is 64-bit).
 */
#ifndef SWB_ARGMAX_STATIC_H_
#define SWB_ARGMAX_STATIC_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SWB_ARGMAX_STATIC_MAX_ROWS 1024
#define SWB_ARGMAX_STATIC_MAX_CHUNKS 32
/* counters (4 B per row) + chunk values (4 B) + chunk indices (8 B) per (row, chunk) */
#define SWB_ARGMAX_STATIC_SCRATCH_BYTES \
  (SWB_ARGMAX_STATIC_MAX_ROWS * 4 + SWB_ARGMAX_STATIC_MAX_ROWS * SWB_ARGMAX_STATIC_MAX_CHUNKS * 12)

#define SWB_ARGMAX_STATIC_E_SIZE (-20)   /* rows or V outside the limits above */
#define SWB_ARGMAX_STATIC_E_SETUP (-21)  /* the scratch array's address could not be obtained */
#define SWB_ARGMAX_STATIC_E_ARG (-22)    /* null logits / out_ids, or ld < V */

/* logits: [rows, V] bf16 (is_fp32 == 0) or fp32 (is_fp32 != 0), row stride `ld` elements; out_ids: int64 [rows];
 * out_vals: fp32 [rows] or null; stream: cudaStream_t. Returns 0, one of the codes above, or -cudaError of the
 * launch. */
int swb_argmax_static(const void* logits, int is_fp32, long long ld, int rows, int V, const void* allow_mask,
                      long long* out_ids, float* out_vals, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SWB_ARGMAX_STATIC_H_ */
