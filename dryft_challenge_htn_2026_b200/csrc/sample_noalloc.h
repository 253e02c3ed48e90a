/* dk_sample_noalloc: the token sampler for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference engine; it exists for users of this
 * library who call the sampler from a place where device memory cannot be requested: inside
 * somebody else's serving loop that owns all GPU memory up front, from a host thread that may not
 * block (cudaMalloc can synchronise the whole device), or from a plug-in that is handed raw
 * pointers and no allocator. The ordinary entry point (dk_sample in sampling.cu) needs the caller
 * to bring n_rows * chunks(V) floats and ints of scratch; this one keeps that scratch in a fixed
 * array inside the library, so the caller passes inputs and outputs only.
 *
 * What to know before using it:
 *  - The scratch is a file-scope device array of DK_NOALLOC_SCRATCH_BYTES (128 KiB). Every GPU that
 *    loads this library holds that much memory until the process exits.
 *  - Limit: n_rows * ceil(V / 4096) <= DK_NOALLOC_MAX_PARTIALS (16384), e.g. 64 rows of a
 *    1,000,000-entry vocabulary or 256 rows of 262,144. Larger requests are refused with
 *    DK_NOALLOC_TOO_LARGE and nothing is launched.
 *  - The first call on each device looks up the array's device address (a host-side set-up step,
 *    done once per device with that device current). Make that first call before any stream
 *    capture begins on that device.
 *  - All calls share the one array, and it keeps whatever the last call left there. Nothing has
 *    to be cleared: each call writes every element it later reads. But two calls whose kernels
 *    overlap on the GPU (different streams, no ordering between them) would overwrite each other's
 *    partial results: keep calls on one device ordered.
 *  - It calls no cudaMalloc, cudaFree or any other allocating routine.
 *  - logits may have any alignment; rows that start on 16-byte boundaries (a 16-byte aligned
 *    pointer and V a multiple of 4) are read with wider loads.
 *  - Calls may follow one another on a stream on the same positions with advance != 0, also under
 *    programmatic dependent launch: the position is read after the wait for the kernel before.
 *
 * Arguments are those of dk_sample without the two scratch pointers:
 *   logits [n_rows, V] float32, temperature [n_rows] float32 (0 = greedy), seeds [n_rows][2]
 *   uint32 (low, high word), pos int32 positions (looked up through rows when rows != NULL; the
 *   draw's counter is position + 1; negative = padding row), out_tok [n_rows] int32, advance != 0
 *   moves each used position on by one. All pointers are device pointers.
 * Returns 0, a cudaError_t (> 0), or one of the negative codes below;
 * dk_sample_noalloc_error(code) gives the text.
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define DK_NOALLOC_MAX_PARTIALS 16384
#define DK_NOALLOC_SCRATCH_BYTES (DK_NOALLOC_MAX_PARTIALS * 8)
#define DK_NOALLOC_TOO_LARGE (-1)
#define DK_NOALLOC_BAD_ARGUMENT (-2)

#ifdef __cplusplus
extern "C" {
#endif
int dk_sample_noalloc(const float* logits, int n_rows, int V, const float* temperature, const uint32_t* seeds,
                      int* pos, const int* rows, int* out_tok, int advance, cudaStream_t stream);
const char* dk_sample_noalloc_error(int code);
#ifdef __cplusplus
}
#endif
