// Allocation-free entry point of the paged-KV decode attention.
//
// This entry point has no counterpart in the reference project: it exists for
// callers of this library that are not allowed to allocate device memory at
// all.  Examples are a host that embeds the kernels inside a process whose
// memory is owned by another runtime (a fixed arena handed out at start-up, no
// cudaMalloc afterwards), or code that runs while an allocator is frozen, for
// instance around a checkpoint of the device state.  Such a caller still owns
// and passes every input and output tensor; what it cannot provide is the
// temporary buffer in which the split-KV kernel parks its partial results.
//
// Here that buffer is a fixed array that lives inside the library image.  Every
// GPU that loads the library holds US_NOALLOC_SCRATCH_BYTES of it until the
// process exits, whether or not this entry point is ever called.
//
// Contract
//   * Same arguments and results as us_paged_decode_attention, minus `scratch`.
//   * The call never calls cudaMalloc, cudaFree or any allocating library
//     routine.  The first call on a device looks up the device address of the
//     array (cudaGetSymbolAddress, with that device current) and remembers it;
//     make that first call before starting any stream capture.
//   * Needs B * Hq * splits * (D + 1) * 4 bytes; a call that needs more than
//     US_NOALLOC_SCRATCH_BYTES is rejected with US_ERR_LIMIT and a message in
//     us_last_error().  splits == 1 needs none.
//   * All calls on a device share the one array.  The kernel overwrites every
//     word it later reads, so nothing has to be cleared between calls, but two
//     calls that can overlap on the GPU (different streams without an ordering
//     between them) race on it: order them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define US_NOALLOC_SCRATCH_BYTES (8u << 20)

int us_paged_decode_attention_noalloc(const void* q, const void* kcache, const void* vcache,
                                      const int* page_table, const int* seq_lens, void* out,
                                      int B, int Hq, int Hkv, int D, int max_pages, int page_size,
                                      int splits, int window, float scale, long long ldq,
                                      long long ldo, void* stream);

#ifdef __cplusplus
}
#endif
