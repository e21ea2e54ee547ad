// kvad_attention_decode_noalloc: the split-key decode attention for callers that may not allocate.
//
// This entry point has no counterpart in bisand/kvad.  It exists for hosts that use the compiled
// kernel library directly, through its C symbols, and have no allocator to offer: a C or C++
// program that links nothing but this library, a plug-in inside an application that has already
// handed the whole device memory to a pool of its own, or a latency-critical loop that must not
// meet the implicit device synchronisation and the system call behind cudaMalloc / cudaFree.
// The ordinary entry point, kvad_attention_decode, needs scratch memory from its caller when the
// keys are split over several CTAs; this one brings its own.
//
// The scratch is a file-scope device array of KVAD_DECODE_NOALLOC_SCRATCH_FLOATS 32-bit floats
// (4 MiB).  Every GPU that loads the library holds it until the process ends.  A call needs
// n_rows * n_heads * n_splits * (head_dim + 2) floats of it (nothing when n_splits == 1) and is
// refused with a message, before anything is launched, when that is more than the array holds.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress) with that
// device current and keeps it; make that first call before any stream capture begins.  The call
// itself allocates nothing: no cudaMalloc, no cudaFree, no library routine that allocates.
// The address is kept in a plain per-device table without a lock: two host threads that make
// their first call on one device at once both look it up and both store the same value, which
// is harmless; no other state is shared between host threads.
//
// All calls share the one array, and it keeps what the last call left in it.  Nothing in it has to
// start at zero - each call writes every word it later reads - but two calls that overlap on the
// GPU (different streams, or concurrent graph branches) race on it: keep calls in one stream order.
//
// Arguments, results and numerics are those of kvad_attention_decode (see attention_decode.cu); the
// output is the same to the bit for the same n_splits.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define KVAD_DECODE_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// 0 on success; a negative code otherwise, with the message in kvad_last_error().
int kvad_attention_decode_noalloc(int dtype, const void* q, int64_t ld_q, void* out, int64_t ld_out,
                                  const int* row_seq, const int* row_pos, const int* page_table, int table_width,
                                  const void* k_pages, const void* v_pages, int n_rows, int n_heads, int n_kv_heads,
                                  int head_dim, int page_size, int n_splits, float scale, int window,
                                  cudaStream_t stream);

// How many floats of the built-in scratch a call with these sizes would use.
int64_t kvad_attention_decode_noalloc_need(int n_rows, int n_heads, int head_dim, int n_splits);

#ifdef __cplusplus
}
#endif
