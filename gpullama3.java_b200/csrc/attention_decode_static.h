// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project (AskMyu/GPULlama3.java): it is an
// addition of this library for host programs that drive the kernels through the C symbols and have
// no allocator to offer at the moment of the call -- a serving loop that must not pay for
// cudaMalloc (which synchronises the whole device), a process whose device memory has already been
// handed over in full to some other pool, or code that runs where allocation is simply forbidden
// (a plugin's enqueue hook, a host callback).
//
// The regular entry point, b200_attention_decode, needs scratch memory for the partial results of
// the spans a sequence's keys are cut into, and expects the caller to bring it.  This variant
// brings its own: one array of fixed size that lives in the library's device image
// (b200_attention_decode_static_capacity() floats; 2 Mi floats = 8 MiB).  Every GPU that loads
// the library holds that array until the process exits, whether or not this function is called.
//
// What a caller has to know:
//  * Inputs and outputs are the caller's, exactly as for b200_attention_decode.  q, k_pool and v_pool
//    must be 16-byte aligned (and q_row_stride a multiple of 8 elements); a call that
//    is not is refused with 10002 and nothing is launched.
//  * The kernel starts when everything before it on the stream has finished, so kv_lens and
//    page_table may be written by the kernel right before the call.  (Inside the engine the regular
//    entry point is allowed to start early, because there those two arrays are copied in ahead of
//    the step's first kernel; this entry point does not assume that.)
//  * A call whose partials do not fit (n_seqs * n_heads * n_splits * (head_dim + 2) floats more
//    than the capacity) is refused with error 10004 and nothing is launched.  n_splits = 1 needs
//    no scratch at all and always fits.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current) and remembers it.  Make that first call outside of any stream
//    capture.
//  * All calls share the one array and it keeps whatever the last call left in it.  Nothing in it
//    has to start at zero: a call writes every partial before its merge step reads it.  But two
//    calls that overlap on the GPU (different streams, no ordering between them) race on it; order
//    them.
//  * It calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Floats the built-in scratch array holds.
long long b200_attention_decode_static_capacity(void);

// Same arguments and meaning as b200_attention_decode without the scratch pair.  Returns 0, a
// cudaError_t, one of the library's argument errors, or 10004 when the call needs more scratch
// than the built-in array holds.
int b200_attention_decode_static(const void* q, int q_row_stride, void* out, const int* kv_lens,
                                 const int* page_table, int table_stride, const void* k_pool, const void* v_pool,
                                 int n_seqs, int n_heads, int n_kv_heads, int head_dim, int window, int n_splits,
                                 cudaStream_t stream);

#ifdef __cplusplus
}
#endif
