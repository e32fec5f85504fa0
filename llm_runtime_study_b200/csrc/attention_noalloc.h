// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference runtime (which allocates freely
// through PyTorch); it exists for embedders of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Typical cases are a
// real-time or safety-certified host loop that fixes its memory map at start-up, a plugin
// living inside another framework's memory pool (a second allocator would fragment or
// exceed the pool the host budgeted), and code executing while a CUDA stream capture is
// open on another thread, where an allocation can invalidate the capture.  Such callers
// own their input and output buffers already; the only thing the split-sequence decode
// kernel needs beyond those is a place to park the per-part (max, sum, output) triples
// before they are merged.  Here that place is a fixed array inside the library image.
//
// Contract
//   * Same arguments and result as b200_attention_decode_bf16, minus the scratch pointer
//     and its size.  Inputs and outputs are still the caller's.
//   * The scratch array holds B200_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  It is part of
//     the library image, so every GPU on which the library is used keeps that much memory
//     until the process exits.  A call needs requests * query_heads * num_splits *
//     (head_size + 2) floats; a call that needs more is refused with
//     B200_ERR_NOALLOC_TOO_LARGE and nothing is launched.  With num_splits == 1 no scratch
//     is needed and any size passes.
//   * No cudaMalloc, cudaFree, or allocating library routine is called, on any path.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and remembers it.  Make that first call outside any stream
//     capture; later calls only launch kernels.
//   * All calls share the one array.  Its contents survive from call to call, but nothing
//     has to be cleared: every slot the merge step reads is written earlier in the same
//     call.  Two calls whose kernels can be in flight at the same time (different streams,
//     or different threads) race on the array and give wrong results; serialise them.
//
// Returns 0 on success, a cudaError_t value if the runtime reports one, or one of the
// B200_ERR_* codes below.
#pragma once

#include <cuda_runtime.h>

#define B200_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define B200_ERR_NOALLOC_TOO_LARGE 10010
#define B200_ERR_NOALLOC_SETUP 10011

#ifdef __cplusplus
extern "C" {
#endif

int b200_attention_decode_bf16_noalloc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                       const int* kv_len, const int* block_table, int table_stride,
                                       int page_size, int requests, int nq, int nkv, float scale, int window,
                                       int num_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
