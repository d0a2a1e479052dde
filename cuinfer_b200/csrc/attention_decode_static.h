// Declaration of the one entry point of this library that allocates no memory.
//
// This entry point has no counterpart in the reference, whose attention kernel needs no scratch memory
// (csrc/ops/paged_attention.cu walks all keys of a request in one CTA).
//
// Who it is for.  `cib_paged_attention_decode` splits the keys of a request over several CTAs and needs a
// scratch buffer for their partial results; its caller has to allocate that buffer.  Some callers cannot:
// an embedding host that has handed every free byte of device memory to the cache pool (a later cudaMalloc
// would fail or would have to shrink the pool), or a serving loop written in C that must never call into the
// CUDA allocator between steps because cudaMalloc and cudaFree synchronise the whole device and stall every
// stream.  For them the scratch lives inside the library, in a fixed `__device__` array.
//
// What the caller has to know.
//   * The array has a fixed size: kStaticScratchFloats floats (8 MiB) of partial results plus
//     kStaticCounters counters.  Every GPU that loads this library holds that memory until the process exits.
//     A call whose num_requests * nq * splits * (head_dim + 2) exceeds kStaticScratchFloats, or whose
//     num_requests * nkv exceeds kStaticCounters, is refused with an error message; nothing is launched.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and keeps it.
//     Make that first call during set-up, before any stream capture is begun on that device.
//   * All calls share the one array, and it keeps what the last call left there.  The entry point clears the
//     counters on the given stream before every launch; the partial results need no clearing because every
//     split is written before it is read.  Two calls that overlap on the GPU (different streams, or the same
//     call replayed concurrently) race on the array and give wrong results: keep calls in stream order.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine, of CUDA or of torch.
//
// Arguments are those of `cib_paged_attention_decode` without `scratch` and `counters`.  Returns 0, or a
// negative code after recording a message for `cib_last_error()`.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { kStaticScratchFloats = 2 * 1024 * 1024, kStaticCounters = 4096 };

int cib_paged_attention_decode_static(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                      int num_pages, int page_size, const int* block_table, int table_stride,
                                      const int* seq_lens, int num_requests, int nq, int nkv, int head_dim,
                                      float scale, int window, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
