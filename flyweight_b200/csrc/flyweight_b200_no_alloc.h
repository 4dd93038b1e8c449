/* flyweight_b200: the one entry point of the library that allocates nothing.
 *
 * It has no counterpart in yairpatch/flyweight; it exists for callers of this library that
 * must not (or cannot) allocate device memory at the moment they need a result:
 *   - code that runs while a CUDA stream is being captured into a graph, where cudaMalloc and
 *     the allocators built on it are not permitted;
 *   - a host that hands this library a fixed memory budget up front (an embedding server
 *     process, a plugin inside another engine) and treats any later allocation as a fault;
 *   - latency-critical loops in which an allocator call (a lock, possibly a device
 *     synchronisation) is not acceptable.
 * Every other entry point of the library takes its scratch memory from the caller or, through
 * the Python layer, from torch's allocator.
 */
#ifndef FLYWEIGHT_B200_NO_ALLOC_H
#define FLYWEIGHT_B200_NO_ALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Largest problem the built-in scratch array serves. */
#define FWB_NO_ALLOC_MAX_ROWS 256      /* rows of logits in one call */
#define FWB_NO_ALLOC_MAX_VOCAB 1048576 /* entries per row */

/* Greedy sampling: out[r] = index of the largest value of logits[r][0..vocab), the lowest
 * index among equal values (-0 equals +0; NaN counts as smallest).  Same result as fwb_argmax.
 *
 *   logits  [rows][vocab] float32, device memory, row-major, contiguous
 *   out     [rows] int32, device memory
 *   stream  the stream the work is enqueued on; its device must be the current device of the
 *           calling thread (the scratch array is found for the current device), else -1
 *
 * The slices of a row are scanned by separate thread blocks; their partial results and a
 * per-row arrival counter live in a scratch array that is part of the library image
 * (about 130 KiB of device memory on every GPU that loads the library, until the process
 * exits).  No cudaMalloc, cudaFree or allocating library routine is called.
 *
 * First call on a device: the entry point looks the scratch array's device address up once
 * per device (with that device current) and keeps it.  Make that first call outside of any
 * stream capture; later calls only enqueue work on `stream`.
 *
 * All calls share the one scratch array per device, and it keeps what the last call left in
 * it.  The entry point clears the counters it needs at the start of every call, so a call
 * never depends on an earlier one -- but two calls whose GPU work may overlap (different
 * streams without an ordering between them, or two host threads) race on the array and give
 * wrong results.  Order them, or use fwb_argmax with scratch of your own.
 *
 * Returns 0 on success; -1 for a null pointer or non-positive size; -3 if rows or vocab
 * exceed the maxima above (nothing is launched); a positive cudaError_t if a CUDA call failed.
 * fwb_no_alloc_last_error() gives the reason of the calling thread's last failure as text.
 */
int fwb_argmax_no_alloc(const float* logits, int rows, int vocab, int* out, cudaStream_t stream);

const char* fwb_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
