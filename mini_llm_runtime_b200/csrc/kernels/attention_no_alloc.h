// Split-KV decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in lilong555/mini-llm-runtime; it is an addition
// of this engine.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a host
// program that embeds the library and whose own memory manager holds all of the device
// memory already; a real-time loop that must not call into the allocator because its
// latency is unbounded; a plugin that is handed a stream and buffers by its host and
// is forbidden from creating more.  The normal entry point
// (mlr_attention_decode_bf16) asks its caller for a scratch buffer in which the
// partial results of the key splits are kept until they are merged.  A caller of the
// kind above has nowhere to get that buffer from.  This variant brings its own: a
// fixed array that lives in the library's device image.
//
// What it costs: MLR_ATTENTION_STATIC_SCRATCH_FLOATS floats (4 MiB) of device memory
// on every GPU that loads this library, from load until the process exits, whether or
// not the entry point is ever called.
//
// Limits and rules:
//  * The scratch a call needs is items * kv_heads * max_splits * 16 * (head_dim + 2)
//    floats (mlr_attention_decode_scratch_floats).  A call that needs more than the
//    fixed array holds is refused with an error; nothing is launched.
//  * The first call on a device looks up the array's device address (with that device
//    current) and remembers it.  Make that first call outside any stream capture.
//  * All calls share the one array.  Calls whose kernels may overlap on the GPU (other
//    streams, other host threads) would overwrite each other's partial results: run
//    them one after the other on one stream.
//  * The array keeps what the last call left in it.  That is harmless here: every
//    element a merge reads was written by the same call's split blocks before, so
//    nothing of it has to start at zero and nothing is cleared.  A small counter array
//    beside it (one int per request and kv head, MLR_ATTENTION_STATIC_COUNTERS of
//    them; a call with more is refused) does have to be zero: it is when the library
//    is loaded, and the block that merges the splits sets its counter back to zero.
//  * Inputs and outputs are still the caller's: q, out, the cache, the block table and
//    the segment table are passed exactly as to mlr_attention_decode_bf16.
//
// Returns 0 on success; otherwise mlr_last_error() of this library says why.
#pragma once

#include <cuda_runtime.h>

#define MLR_ATTENTION_STATIC_SCRATCH_FLOATS (1 << 20)
#define MLR_ATTENTION_STATIC_COUNTERS 4096      // requests x kv heads of one call

extern "C" int mlr_attention_decode_bf16_no_alloc(const void* q, int ldq, void* out, int ldo, const void* cache,
                                                  int num_pages, const int* items, int n_items,
                                                  const int* segment_info, const int* block_table,
                                                  int table_stride, int page_size, int q_heads, int kv_heads,
                                                  int head_dim, int window, float scale, int chunk, int max_splits,
                                                  int* status, cudaStream_t stream);
