/* fg_attention_decode_noalloc: decode attention for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference engine (lawnak/FastGGUF); it exists for
 * users of this library who call it from places where device memory cannot be allocated or
 * freed: inside a latency-critical serving loop that has handed all device memory to its own
 * pool, from a host thread that is not allowed to synchronise the device (cudaMalloc and
 * cudaFree may), or from a runtime that forbids allocation after start-up.
 *
 * It computes what fg_attention_decode computes on its scratch-memory path (the pages of each
 * sequence split over n_splits CTAs, partial results merged by a second kernel), but the
 * partial results go to a fixed array that is part of the library image instead of to buffers
 * the caller allocates.  The caller still passes every input and the output.
 *
 * Limits and rules
 *   - With n_splits > 1, B * H * n_splits * (head_dim + 2) must not exceed
 *     FG_NOALLOC_SCRATCH_FLOATS (1 Mi floats, 4 MiB); larger requests return
 *     FG_ERR_NOALLOC_TOO_LARGE and launch nothing.  A call with n_splits == 1 writes its output
 *     directly, uses none of the array and has no such limit.  Every GPU that loads the library
 *     holds these 4 MiB until the process exits.
 *   - The first call on a device looks up the array's device address (once per device, with
 *     that device current).  Make that first call outside any stream capture.
 *   - All calls share the one array, which keeps the last call's contents.  Every element a
 *     call reads is written by that call first, so nothing needs clearing; but two calls that
 *     overlap on the GPU (different streams, or concurrent graphs) race on it.  Issue them on
 *     one stream, or order them yourself.
 *   - It calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Arguments are those of fg_attention_decode without the two scratch pointers; n_splits may be
 * any value >= 1.  Returns 0 or an error code (a cudaError_t, or an FG_ERR_* value).
 */
#pragma once
#include <cuda_runtime.h>

#define FG_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define FG_ERR_NOALLOC_TOO_LARGE 10005

#ifdef __cplusplus
extern "C" {
#endif

int fg_attention_decode_noalloc(const void *q, int ldq, void *out, int ldo, const int *positions,
                                const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                                int B, int H, int KV, int hd, int page_size, float scale, int window, int n_splits,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
