// llm_attention_mma_static_scratch: paged attention for callers that must not allocate.
//
// This entry point has no counterpart in cuongvng/bare-cuda-4gib; it exists for users of this
// library whose code cannot call cudaMalloc at the point where attention runs:
//   * a host program that has already handed all of the GPU's memory to an allocator of its own
//     (an arena sized at start-up, another framework's pool): a cudaMalloc there fails or
//     fragments what the program planned, and the program has no way to lend this library a
//     buffer through its own interfaces;
//   * a latency-critical loop: cudaMalloc and cudaFree may synchronise the whole device, which
//     stalls every stream the program has in flight.
// llm_attention_mma (the ordinary entry point) needs scratch memory whenever a tile's keys are
// split over several thread blocks (n_splits > 1: the decode shape), and the caller has to
// allocate it.  Here the scratch is a fixed array that lives inside the library instead.
//
// What it costs and what it limits
//   * The array holds LLM_ATTENTION_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on which the
//     library is loaded keeps that much memory until the process exits, used or not, and each
//     head-size build of the library has an array of its own.
//   * A call needs 4096 + n_tiles * kv_heads * n_splits * rows_per_tile * (head_dim + 1) words
//     (llm_attention_scratch_floats).  If that is more than the array holds, the call launches
//     nothing and returns LLM_ERR_STATIC_SCRATCH_TOO_SMALL: use fewer splits, or the ordinary
//     entry point.  With n_splits == 1 no scratch is used and any size is accepted.
//   * All calls share the one array.  Two calls whose kernels can overlap on the GPU (different
//     streams, or several host threads) race on it and give wrong results: keep calls that use
//     it on one stream, or order them yourself.  The array keeps whatever the last call wrote.
//     Only its first 4096 words have to be zero when a call starts: they count, per tile, the
//     splits that have finished.  They are zero when the library is loaded, and the thread block
//     that merges a tile sets that tile's counter back to zero, so a call that ran to its end
//     leaves them zero for the next one.  Everything else a call reads was written by the same
//     call before (each split writes its whole partial output and its log-sum-exp before it counts
//     itself done).
//
//   * After a call that did not run to its end (a CUDA error in its stream, a launch that was
//     aborted) those counters may be left non-zero, and every later split call would then merge a
//     tile too early.  After any CUDA error, clear the first 4096 words yourself before the next
//     split call: cudaMemsetAsync on the address that llm_attention_static_scratch_address()
//     returns (it is known once one call on this device has succeeded; a call with n_splits == 1
//     is enough).
//
// Set-up.  The first call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and remembers it; this makes the first call
// slower and is ordinary host-side CUDA runtime work, so make that first call before any stream
// capture begins.  The address is looked up for the device that is CURRENT on the calling thread
// (cudaGetDevice), so `stream` must be a stream of that device: a stream of another device would
// hand the kernel an address that means nothing there (where the runtime can tell which device a
// stream belongs to, such a call is refused with LLM_ERR_STATIC_SCRATCH_WRONG_DEVICE and nothing
// is launched).  The remembered addresses are plain host variables: if several host threads may
// make the first call on a device at the same time, make one call on that device first from one
// thread (the look-up itself is idempotent, but the C++ memory model promises nothing for the race).
//
// The function never calls cudaMalloc, cudaFree or any allocating library routine;
// inputs, outputs and the step's index arrays are the caller's, exactly as for llm_attention_mma.
//
// Arguments and return value are those of llm_attention_mma without the `scratch` pointer:
// 0 on success, a small positive code for refused arguments, 1000 + cudaError_t for a CUDA error.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define LLM_ATTENTION_STATIC_SCRATCH_FLOATS (1 << 20)
#define LLM_ERR_STATIC_SCRATCH_TOO_SMALL 4
#define LLM_ERR_STATIC_SCRATCH_WRONG_DEVICE 5

#ifdef __cplusplus
extern "C" {
#endif

int llm_attention_mma_static_scratch(const void* q, void* out, void* k_base, void* v_base,
                                     const int32_t* block_table, long long page_stride, int table_stride,
                                     int page_tokens, int kv_heads, int head_dim, const int32_t* seq_q_start,
                                     const int32_t* seq_q_len, const int32_t* seq_kv_len, const int32_t* tile_seq,
                                     const int32_t* tile_index, int n_tiles, int rows_per_tile, int n_splits,
                                     int q_heads, float scale, int window, cudaStream_t stream);

// The array's address on the current device (null before the first call on it, or on an error):
// only for clearing the counters after a failed call, as described above.
float* llm_attention_static_scratch_address(void);

#ifdef __cplusplus
}
#endif
