/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference: it exists for hosts that embed this
 * library where cudaMalloc is off the table. Think of a caller that runs inside someone else's
 * memory budget (a plugin in a serving process whose allocator owns all of the device), of code
 * that must stay allocation-free because it runs between the begin and end of a stream capture
 * it does not control, or of a real-time loop where an allocation's latency and its implicit
 * synchronisation are not acceptable. Such callers still own their inputs and outputs and pass
 * them in; what they cannot provide is the scratch buffer that the sliced kernel needs for its
 * per-slice partial results (`r2_attention_decode` takes that buffer as an argument).
 *
 * Here the scratch lives in a file-scope `__device__` array inside the library:
 * R2_STATIC_SCRATCH_FLOATS floats (2 MiB). Every GPU on which the library is loaded holds that
 * array until the process exits. The call computes exactly what `r2_attention_decode` computes,
 * with the same arguments minus the scratch pointer and its size.
 *
 * Rules for the caller:
 *   - n_rows * n_heads * n_slices * (head_dim + 2) must not exceed R2_STATIC_SCRATCH_FLOATS;
 *     otherwise nothing is launched, the call returns R2_STATIC_SCRATCH_TOO_SMALL and
 *     `r2_attention_decode_static_error()` says how much was asked for and how much there is.
 *     With n_slices == 1 no scratch is used and any size passes.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current) and keeps it; make this first call before any stream capture begins.
 *   - The array is shared by every call and keeps the last call's contents. Each call overwrites
 *     every word it later reads, so nothing has to be cleared in between; but two calls that
 *     overlap on the GPU (different streams, or concurrent graph branches) race on it. Keep
 *     calls into this entry point ordered on one stream per device.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on any path.
 *   - Row t of `q` is entry t: `seq_lens[t]` is its context length (the new token included),
 *     `positions[t]` its position, row t of `block_tables` its pages. `row_entry` is not read (pass
 *     NULL); a batch whose rows are not its entries in order is not what this kernel computes.
 *   - The kernels of this entry point are launched in plain stream order, so every array may be
 *     produced by the caller's kernel just before the call in the same stream. (`r2_attention_decode`
 *     itself is launched with programmatic stream serialization when that is switched on, and reads
 *     positions, seq_lens and block_tables before it waits for its predecessor: its index arrays must
 *     be complete before the kernel ahead of it in the stream has started.)
 */
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define R2_STATIC_SCRATCH_FLOATS (512 * 1024)
#define R2_STATIC_SCRATCH_TOO_SMALL (-5)
#define R2_STATIC_SETUP_FAILED (-6)

int r2_attention_decode_static(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                               const void* v_cache, long long page_stride, int page_size, int n_pages,
                               const int32_t* block_tables, int table_width, const int32_t* row_entry,
                               const int32_t* positions, const int32_t* seq_lens, int n_rows, int n_heads,
                               int n_kv_heads, float scale, int window, int n_slices, cudaStream_t stream);

/* The message of the last refused call on this thread ("" if none). */
const char* r2_attention_decode_static_error(void);

#ifdef __cplusplus
}
#endif
