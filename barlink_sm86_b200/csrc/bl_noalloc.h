/* SPDX-License-Identifier: MIT
 *
 * Arg max without any allocation.  This entry point has no counterpart in the
 * reference; it exists for callers of this library that are not allowed to
 * allocate device memory at the moment they call: code inside another
 * framework's allocator callback or memory-pool critical section, and
 * embedders that hand the library a fixed memory budget up front and forbid
 * cudaMalloc afterwards (cudaMalloc synchronises the device and can fail at an
 * unpredictable point).
 *
 * bl_argmax (bl_ops.h) needs a scratch buffer from its caller for the
 * per-slice partial results of its first kernel.  bl_argmax_noalloc runs the
 * same two kernels, but the partial results live in a file-scope device array
 * that is part of the library image.
 *
 *   - Limit: at most BL_ARGMAX_NOALLOC_MAX_ROWS rows per call (the array is
 *     BL_ARGMAX_NOALLOC_MAX_ROWS * 16 slices * 8 bytes = 512 KiB, held by
 *     every GPU that loads the library until the process exits).  More rows
 *     are rejected with an error message; nothing is launched.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress); later calls on that device do no set-up.
 *   - All calls share the one array.  Every slot a call reads is written by
 *     that same call first, so nothing has to be cleared between calls; but
 *     two calls that overlap in time on one GPU (different streams) race on
 *     it.  Keep calls on one stream, or order them yourself.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on any
 *     path, including the error paths.
 *
 * logits: bf16 [rows x n], row pitch ld elements.  idx: int32 [rows] (index of
 * the maximum, lowest index on ties, plus `offset`).  val: fp32 [rows] or
 * null.  stream: cudaStream_t.  Returns 0, or -1 with a message in err.
 */
#ifndef BARLINK_B200_NOALLOC_H
#define BARLINK_B200_NOALLOC_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BL_ARGMAX_NOALLOC_MAX_ROWS 4096

int bl_argmax_noalloc(const void* logits, int rows, int n, int ld, int offset, int* idx, float* val,
                      void* stream, char* err, size_t errlen);

#ifdef __cplusplus
}
#endif
#endif
