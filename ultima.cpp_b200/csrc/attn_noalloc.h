// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (tattooinmtl/Ultima.cpp); it is an
// addition of this library.
//
// Who it is for: a host program that owns all device memory itself and forbids any further
// allocation once it is running (an embedding runtime with fixed pools, a process whose
// memory was sized to the last byte for the cache, a latency-critical loop in which an
// allocation would stall every stream of the device).  The ordinary entry point, ub_attn_mma,
// leaves the scratch for its split-key partial results to the caller, who in this package
// takes it from a torch buffer; a caller of the kind above has nowhere to take it from.
//
// What it does: the same decode attention as ub_attn_mma in mode 1 (one new token for every
// sequence, keys cut into ``n_slices`` slices, partial results merged by a second kernel),
// with the partial results kept in an array that is part of the library's own device image:
// UB_NOALLOC_SCRATCH_BYTES (4 MiB + 64 KiB) on every GPU that loads the library, held until
// the process exits.  It calls no cudaMalloc, cudaFree or other allocating routine.
//
// Limits and rules:
//   * n_seqs * n_heads * n_slices * HEAD_DIM floats must fit 4 MiB and n_seqs * n_heads *
//     n_slices * 2 floats must fit 64 KiB; otherwise nothing is launched and
//     UB_ERR_NOALLOC_TOO_LARGE (-3) comes back.
//   * The first call on a device looks up the array's device address (once a device, with that
//     device current).  Make that first call before any stream capture begins.
//   * All calls share the one array and it keeps what the last call wrote.  Nothing in it has
//     to start at zero: every slice writes its whole partial result before the merge reads it.
//     Two calls that overlap on the GPU (different streams, no ordering between them) race on
//     the array; order them.
//   * Inputs and outputs are the caller's, exactly as for ub_attn_mma.
#pragma once
#include <cuda_runtime.h>

#define UB_NOALLOC_SCRATCH_O_FLOATS (1 << 20)
#define UB_NOALLOC_SCRATCH_ML_FLOATS (1 << 14)
#define UB_NOALLOC_SCRATCH_BYTES ((UB_NOALLOC_SCRATCH_O_FLOATS + UB_NOALLOC_SCRATCH_ML_FLOATS) * 4)
#define UB_ERR_NOALLOC_TOO_LARGE (-3)

extern "C" __attribute__((visibility("default")))
int ub_attn_decode_noalloc(const void* q, long long q_stride, void* out, long long o_stride, const void* kcache,
                           const void* vcache, const int* seq_start, const int* seq_before, const int* table,
                           int pages_per_seq, int ring, int page, int n_seqs, int nh, int nkv, int window,
                           float scale, int n_slices, cudaStream_t st);
