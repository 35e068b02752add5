// tie_attention_split_noalloc: split attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this
// library. Some of them cannot call cudaMalloc where they call attention: code that runs inside
// a memory budget fixed at start-up, plugins that are handed their buffers by a host
// application and may not grow the device heap, and callers on a path where an allocation
// (which may synchronize the device) is not acceptable. tie_attention_split asks such a caller
// for a scratch buffer it has no way to provide. This variant needs none: the partial results
// of the splits live in an array that is part of the library's own device image.
//
// Same arguments and same results as tie_attention_split (attention_simt.cu) without the
// `scratch` argument. What to know:
//   * The array holds TIE_NOALLOC_SCRATCH_FLOATS floats (4 MiB). Every GPU that loads the library
//     keeps that much memory for it until the process exits. A call that needs more
//     (n_list * q_heads * max_splits * (head_dim + 2) floats) is refused with a message; nothing
//     is launched.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) and remembers it. Make that first call outside of any stream
//     capture; later calls on that device only launch kernels.
//   * A sequence is cut into at most max_splits splits of split_keys keys; if its context is longer than
//     max_splits * split_keys the last split takes the rest (slower, still right). Size max_splits as
//     ceil(longest context / split_keys) to keep the splits even.
//   * It calls no cudaMalloc, cudaFree or any allocating routine, on any call.
//   * All calls share the one array and it keeps what the last call left. Nothing in it has to
//     start at zero: the split kernel writes every entry that the merge kernel reads. But two
//     calls whose kernels overlap on the GPU (different streams, or different host threads on
//     one device) race on it. Serialize them, e.g. by using one stream.
#pragma once

#include <cuda_runtime.h>

#define TIE_NOALLOC_SCRATCH_FLOATS (1 << 20)

extern "C" int tie_attention_split_noalloc(int dtype, const void* q, long long q_stride, const void* k_cache,
                                           const void* v_cache, void* out, const int* query_start,
                                           const int* context_lens, const int* block_tables, int max_blocks, int seqs,
                                           int q_heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                           const int* seq_list, int n_list, int split_keys, int max_splits,
                                           cudaStream_t stream);
