// Allocation-free decode attention.
//
// This entry point has no counterpart in the reference project; it exists for hosts that must
// not allocate device memory while they serve.
//
// Who needs it: a program that embeds this library next to its own memory plan, for example a
// serving process that has given all device memory to its own arena at start-up, or a plain C
// host without a caching allocator.  For such a caller a cudaMalloc in the middle of a decode
// step is not acceptable: it may fail once memory is fragmented or spoken for, and it
// serialises with everything else running on the device.  sprout_attention_decode asks its caller
// for scratch memory for the partial results of its key splits; this variant brings its own, a
// fixed array that lives in the library's device image.
//
//   * Inputs and outputs are passed exactly as to sprout_attention_decode (minus `scratch`).
//   * The scratch array holds SPROUT_STATIC_SCRATCH_FLOATS float32 values (8 MiB).  Every GPU
//     whose context loads the library keeps that much resident until the process ends.
//   * A call whose splits need more (requests * heads * splits * (head_dim + 2) floats) is
//     refused with an error; nothing is launched.
//   * The first call on a device looks up the array's device address (once per device, with that
//     device current).  Make that first call before any stream capture begins.
//   * The call performs no cudaMalloc, no cudaFree and no allocating library routine.
//   * All calls share the one array and it keeps the previous call's contents.  Nothing has to be
//     cleared: a call reads only the slots that the same call has written.  Two calls that run on
//     the GPU at the same time (different streams) would overwrite each other's partial results:
//     keep calls on one device in stream order.
#pragma once

#include <cuda_runtime.h>

#define SPROUT_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

extern "C" int sprout_attention_decode_static(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                              const int* block_table, int table_stride, const int* context_lens,
                                              void* out, int out_stride, int requests, int heads, int kv_heads,
                                              int head_dim, int page_tokens, int num_pages, int split_keys,
                                              int splits, int* status, cudaStream_t stream);
