// Decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference (bigmah/llmoxide): it
// exists for hosts of this library, not for parity.
//
// Who needs it.  llmx_attention_decode() splits the key range over CTAs and
// merges the pieces through a float32 workspace that the caller allocates and
// passes in.  Some callers cannot do that at the moment of the call: a
// serving process that handed all device memory to its own pool at start-up
// and forbids driver allocations afterwards, or a latency-critical decode loop
// in which cudaMalloc is unacceptable because it synchronises the whole
// device.  For them the workspace lives inside the library: a file-scope
// __device__ array of LLMX_NOALLOC_WS_FLOATS floats (16 MiB) and one of
// LLMX_NOALLOC_COUNTERS arrival counters, which every GPU that loads the
// library holds from load until the process exits.
//
// What it does.  Exactly what llmx_attention_decode() does, with that array as
// the workspace.  The caller still passes the inputs (q, caches, block table,
// positions) and the output.  It calls no cudaMalloc, no cudaFree and no
// allocating library routine.
//
// Limits and rules.
//  * With more than 8 shares per sequence (n_chunks > 8), B * H * n_chunks *
//    (D + 4) must not exceed LLMX_NOALLOC_WS_FLOATS, and B * G * ceil((H/G)/8)
//    must not exceed LLMX_NOALLOC_COUNTERS; a larger request is refused with
//    LLMX_NOALLOC_TOO_LARGE and nothing is launched.  With up to 8 shares the
//    pieces are merged inside a thread-block cluster, neither array is
//    touched, and no size limit applies.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it; make
//    that first call outside any stream capture.
//  * All calls share the arrays, and they keep what the last call left.
//    The partials need no initial value: every one that the merge reads is
//    written earlier in the same call.  The counters start at zero, as every
//    device array without an initialiser does, and each call leaves them at
//    zero.  Two calls whose kernels overlap on the GPU (different streams, no
//    ordering between them) race on the arrays; order them.
#pragma once

#include <cuda_runtime.h>

#define LLMX_NOALLOC_WS_FLOATS (4u * 1024u * 1024u)
#define LLMX_NOALLOC_COUNTERS 4096u
#define LLMX_NOALLOC_TOO_LARGE (-5)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as llmx_attention_decode(), without the workspace and counter pointers.
// Returns 0, a negative refusal code, or the positive cudaError_t of a failed call.
int llmx_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                  long long n_pages, const int* block_table, int table_width, const int* seq_past, int B, int H,
                                  int G, int D, int window, float scale, int n_chunks, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
