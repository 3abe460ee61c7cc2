/* Allocation-free entry point of the expert router.
 *
 * This entry point has no counterpart in the reference: there every buffer a kernel touches is
 * allocated by the Python block objects before the first launch.
 *
 * Who it is for: callers that must not (or cannot) create device memory at the moment they need a
 * routing decision - a host thread running inside another framework's stream capture, a plugin
 * that was handed a stream and pointers but no allocator, a signal-safe or real-time path where a
 * cudaMalloc (which may synchronise the device and take a driver lock) is unacceptable.  The
 * regular entry point (nexrt_moe_router in api.h) expects the caller to bring three pieces of
 * scratch: the per-k-quarter partial logits, the summed logits and the ticket word.  Here that
 * scratch lives in one file-scope device array inside the library, so the caller passes only
 * inputs and outputs.
 *
 * Limits and rules:
 *   - at most NEXRT_ROUTER_NOALLOC_MAX_ROWS token rows, router weights padded to at most
 *     NEXRT_ROUTER_NOALLOC_MAX_EXPERT_ROWS rows (a multiple of 16), H a multiple of 1024 and at most
 *     4096; anything larger is rejected with cudaErrorInvalidValue and nothing is launched;
 *   - the array (21 184 floats, 84.7 KB) is held by every GPU that loads the library until the process exits;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call outside of any stream capture.  The per-device address cache is a table of atomics, so host
 *     threads may make their first calls concurrently (they store the same value);
 *   - every call shares the one array and leaves its logits in it: the ticket word is cleared on
 *     the caller's stream before each launch, and two calls that overlap on the GPU (different
 *     streams, no dependency) race - serialise them;
 *   - no cudaMalloc, cudaFree or allocating library routine is called.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define NEXRT_ROUTER_NOALLOC_MAX_ROWS 8
#define NEXRT_ROUTER_NOALLOC_MAX_EXPERT_ROWS 528

/* x [M][H] bf16, post_ln [H] fp32 (1 + w), w [rows_pad][H] bf16 (rows E+1.. zero),
 * ids [M][topk+1] int32 and wts [M][topk+1] fp32 outputs (last entry: shared expert, sigmoid gate).
 * Returns a cudaError_t as int. */
int nexrt_moe_router_noalloc(const void* x, const void* post_ln, const void* w, void* ids, void* wts, int rows_pad, int H, int E, int topk,
                             int M, float eps, void* stream);

#ifdef __cplusplus
}
#endif
