// rl_attn_decode_noalloc: decode attention over the paged cache for callers that cannot
// allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for users of
// this library only.
//
// Who needs it: code that runs where cudaMalloc is off limits, for instance a plug-in
// inside a host process that hands out a fixed memory budget up front and forbids any
// later allocation, a real-time loop that must not take the allocator's locks or its
// unbounded latency, or a caller that has already given all device memory to its own pools.
// The ordinary entry point, rl_attn_decode, asks such a caller for three scratch buffers
// (per-partition outputs, their softmax statistics, arrival counters) that it would have
// to allocate.  Here the scratch lives in a fixed array inside the library instead, so
// the caller passes inputs and outputs only.
//
// What to know before calling:
//   * The array is RL_ATTN_NOALLOC_SCRATCH_BYTES (8 MiB) per loaded copy of the library
//     (one per head size) on every GPU that loads it, and stays until the process exits.
//   * The scratch a call needs, with rows = nitems * hq * max_parts, is
//         round_up(nitems * hkv * 4, 256)  +  round_up(rows * 8, 256)  +  rows * head_dim * 4
//     bytes (arrival counters, softmax statistics, partition outputs; the first two are each
//     rounded up to 256 bytes).  A call that needs more than the array holds is refused: the function
//     returns RL_ATTN_NOALLOC_TOO_LARGE, writes a message that names both numbers into
//     errbuf (if given) and launches nothing.
//   * The first call on each device looks up the array's device address (with that
//     device current), sets the kernels' shared-memory limits there, and remembers both.
//     Make that first call outside any stream capture.  First calls from several threads
//     at once are safe: the look-up is under a lock, and the limits are the same values
//     whoever sets them first.
//   * All calls share the one array, and it keeps what the last call left.  The part that
//     must start at zero (the arrival counters) is cleared on the caller's stream at the
//     start of every call; nothing else needs clearing.  Two calls whose work overlaps on
//     the GPU (different streams, or the same stream on different threads without
//     ordering) would write the same scratch and race: order them.
//   * The function calls no cudaMalloc, cudaFree or other allocating routine.
//
// Arguments are those of rl_attn_decode without part_o, part_ml and counters (see
// attention.cu).  Returns 0, a cudaError_t value, or RL_ATTN_NOALLOC_TOO_LARGE.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define RL_ATTN_NOALLOC_SCRATCH_BYTES (8u << 20)
#define RL_ATTN_NOALLOC_TOO_LARGE (-1)

#ifdef __cplusplus
extern "C" {
#endif

int rl_attn_decode_noalloc(int dtype, const void* q, int q_stride, const void* kcache, const void* vcache,
                           const int32_t* block_table, int max_blocks, const int32_t* items, int max_parts,
                           void* out, int out_stride, int nitems, int hq, int hkv, int page_size, int window,
                           float scale, cudaStream_t stream, char* errbuf, int errbuf_len);

#ifdef __cplusplus
}
#endif
