// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for
// embedders of this library. Some hosts cannot call cudaMalloc at the moment
// they need attention: code running inside a CUDA stream capture or another
// region where allocation is forbidden, a runtime whose memory is handed out
// once at start-up by a supervisor and then locked, or a plugin that is only
// allowed to touch buffers its host gives it. The ordinary entry point
// (stride_paged_decode_attention) asks such a caller for a scratch buffer it has
// no way to obtain. This one brings its own: the partial results of the key
// splits live in a fixed array inside the library's device image.
//
// Limits and rules
//   * The array holds STRIDE_DECODE_STATIC_SCRATCH_FLOATS float32 values (8 MiB).
//     Every GPU that loads this library carries that array until the process
//     exits, whether the entry point is ever called or not.
//   * A call whose sizes need more than that is refused with
//     STRIDE_STATIC_SCRATCH_TOO_SMALL and launches nothing. Ask
//     stride_paged_decode_attention_static_floats() beforehand if in doubt.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) and raises the kernel's shared-memory limit. Make
//     that first call outside any stream capture; later calls only launch.
//   * All calls on a device share the one array, and it keeps whatever the last
//     call left in it. Only the ticket counters at its start (one per token and
//     key head, by which the last split of a group finds out that it is the
//     last) have to be zero when a call begins: they are zero when the library
//     is loaded, and the CTA that draws the last ticket of a group sets it back
//     to zero, so every completed call leaves them cleared for the next one.
//     Everything else a call reads was written earlier in the same call. Two
//     calls that overlap on the GPU (different streams, or one device driven
//     from two threads) overwrite each other's partial results and tickets:
//     run them one after the other.
//   * max_context must exceed every token's position. A row whose position does
//     not lie below it gets zeros instead of attention and draws no ticket, so
//     the array stays clean for the next call (there is no way to reset it
//     short of unloading the library, so nothing may leave a ticket behind).
//   * The key and value tiles are copied with cp.async. The ordinary entry
//     point can also copy them by TMA, for which it needs the size of the cache
//     and a status word that this signature does not have; the arithmetic and
//     the order of every sum are the same, so both give the same bits.
//   * No cudaMalloc, cudaFree or allocating library routine is called.
//
// Inputs and outputs are the caller's, with the meanings of
// stride_paged_decode_attention: q [tokens, q_stride] bfloat16 with head h of
// token t at q[t * q_stride + h * hd]; out [tokens, nq * hd] bfloat16; pages
// [num_pages, nkv, page_size, hd] bfloat16; block_table [seqs, table_width],
// seq_of_token [tokens] (-1 marks padding), positions [tokens] int32;
// max_context bounds position + 1 over the tokens. Returns 0, a negative code
// below, or a positive cudaError_t.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define STRIDE_DECODE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define STRIDE_STATIC_SCRATCH_TOO_SMALL (-3)

#ifdef __cplusplus
extern "C" {
#endif

int stride_paged_decode_attention_static(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                         const int32_t* block_table, int table_width, const int32_t* seq_of_token,
                                         const int32_t* positions, int tokens, int nq, int nkv, int hd, int page_size,
                                         float scale, int window, int max_context, cudaStream_t stream);

// float32 values of the static array that a call with these sizes would use.
long long stride_paged_decode_attention_static_floats(int tokens, int nq, int nkv, int hd, int max_context);

#ifdef __cplusplus
}
#endif
