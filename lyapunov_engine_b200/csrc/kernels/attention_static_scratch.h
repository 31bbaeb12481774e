/* Split-key decode attention for callers that must not allocate.
 *
 * This entry point has no counterpart in IanConery/lyapunov-engine; it exists
 * for users of this library only.
 *
 * le_attention_decode_bf16 needs scratch memory for its partial results and
 * expects the caller to bring it.  Some callers have no way to get device
 * memory at the moment of the call: a plugin that runs inside a host
 * application's execution callback, where the application owns every byte of
 * device memory and forbids cudaMalloc; a serving loop that has handed all
 * free memory to its page pool and whose allocator would fail or fragment; a
 * latency-critical loop that cannot afford the device-wide synchronisation an
 * allocation may imply.  For them this variant keeps the scratch inside the
 * library itself, in a fixed array in device memory.
 *
 * What to know before using it:
 *   - The array holds LE_STATIC_SCRATCH_FLOATS floats (4 MiB).  The attention
 *     kernels are built as one library per head size, and each of them has
 *     an array of its own: every GPU on which such a library is loaded keeps
 *     4 MiB for it until the process exits.
 *   - Libraries for head sizes above 128 have no split-key kernel; there the
 *     symbol exists and refuses every call with LE_INVALID.
 *   - A call whose partial results do not fit is refused with LE_INVALID
 *     (le_last_error() names the size asked for and the limit); nothing is
 *     launched.  The size needed is
 *     le_attention_decode_scratch_floats(num_requests, num_heads, num_splits).
 *   - The first call on each device looks the array's address up (with that
 *     device current).  Make that first call outside any stream capture.
 *     The driver may also load the library's kernels and place the array on
 *     the device at that first call (it loads modules lazily unless
 *     CUDA_MODULE_LOADING=EAGER is set), which takes device memory once: a
 *     caller with a window in which nothing may be allocated makes one call
 *     before that window opens.
 *   - The address is remembered per device ordinal.  After cudaDeviceReset
 *     (or anything else that destroys the device's primary context) it is
 *     stale; this entry point is not for processes that reset a device and
 *     carry on.
 *   - All calls on a device share the one array and it keeps what the last
 *     call left.  The kernels write every slot they later read, so nothing
 *     needs clearing, but two calls that overlap on the GPU (different
 *     streams, or the same call from two threads) race on it: order them.
 *   - Apart from that first call, neither this function nor anything it
 *     calls allocates or frees memory.
 *   - As in le_attention_decode_bf16, the pool's last page (num_pages - 1) is
 *     the page that nobody owns: a request at position 0 whose block table
 *     starts with it is taken for padding and gets a row of zeros.
 *
 * Arguments and result are those of le_attention_decode_bf16 without the
 * scratch pointer.
 */
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LE_STATIC_SCRATCH_FLOATS (1 << 20)

int le_attention_decode_bf16_static(void *out, int64_t out_stride, const void *q, int64_t q_stride,
                                    const void *k_cache, const void *v_cache, const int32_t *block_table,
                                    int max_blocks, const int32_t *cu_q, const int32_t *ctx_before,
                                    const int32_t *requests, int num_requests, int num_heads, int num_kv_heads,
                                    int page_size, int num_pages, int window, float scale, int num_splits,
                                    int *status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
