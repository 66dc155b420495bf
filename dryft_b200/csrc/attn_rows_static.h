// dryft_attn_rows_static_scratch — row-wise attention over the paged cache for callers that cannot
// allocate device memory.
//
// This entry point has no counterpart in hari495/dryft (its decode attention,
// engine/dryft_qwen3/kernels/attn_decode.py:152-176, allocates its split partials with torch.empty on
// every call).  It exists for hosts of this library that must not, or cannot, call cudaMalloc: code
// running under a fixed memory budget fixed at start-up, plug-ins that are handed device pointers by
// an application owning the allocator, and any caller between the begin and the end of a stream
// capture, where an allocation would break the capture.
//
// It is dryft_attn_rows (attn_rows.cu) with one difference: the scratch for the split partials
// (un-normalised outputs, running maxima and sums) is not passed in.  It is a file-scope device array
// of DRYFT_ATTN_ROWS_STATIC_FLOATS floats (4 MiB) inside the library, which every GPU that loads the
// library holds until the process exits.  Inputs and outputs are still the caller's.
//
// Contract
//   * Sizes: with n_splits > 1,  rows * heads * n_splits * (head_dim + 2)  floats must fit in the
//     array; otherwise the call returns DRYFT_ERR_SCRATCH_TOO_SMALL (-3) and launches nothing.  With
//     n_splits == 1 no scratch is used and any size passes.
//   * Set-up: the first call on a device asks the runtime for the array's device address
//     (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call outside any
//     stream capture.
//   * The call allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//   * All calls on a device share the one array, and it keeps the last call's contents.  Nothing in it
//     has to start at zero (every partial is written before it is read), but two calls that overlap on
//     the GPU — different streams, or graphs replayed side by side — race on it.  Order them.
//   * Return value: 0, a cudaError_t, DRYFT_ERR_UNSUPPORTED (-2) or DRYFT_ERR_SCRATCH_TOO_SMALL (-3).
#pragma once

#include <cuda_runtime.h>

#define DRYFT_ATTN_ROWS_STATIC_FLOATS (1u << 20)
#define DRYFT_ERR_SCRATCH_TOO_SMALL (-3)

#ifdef __cplusplus
extern "C" {
#endif

int dryft_attn_rows_static_scratch(int is_bf16, const void* q, const void* k_pages, const void* v_pages,
                                   const int* page_table, int max_pages, const int* tok_slot, const int* tok_pos,
                                   void* out, int n_rows, int nKV, int n_splits, float scale, int window,
                                   cudaStream_t stream);

// Capacity of the built-in scratch, in floats.
long long dryft_attn_rows_static_scratch_floats(void);

#ifdef __cplusplus
}
#endif
