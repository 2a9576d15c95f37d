// Paged attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (RishDevs/mercury has no native
// code at all); it exists for users of this library who embed the attention kernel in a
// host program where cudaMalloc is off limits: a program whose memory is wholly owned by
// another runtime's pool, a real-time loop that may not take the allocator's lock, or a
// plug-in that is handed device buffers and must not create its own.
//
// `mb_paged_attention_static` computes exactly what `mb_paged_attention_simt` computes
// with num_splits > 1, but takes no scratch pointer: the per-split partial results live in
// a file-scope `__device__` array inside the library.
//
// What the caller has to know:
//   * Size limit, for num_splits > 1: tokens * n_q * num_splits * (head_dim + 2) floats
//     must not exceed MB_STATIC_SCRATCH_FLOATS (4 Mi floats = 16 MiB). Larger problems are
//     refused with MB_ERR_SCRATCH (5) and nothing is launched. With num_splits <= 1 the
//     array is not used and no limit applies. Every GPU on which the library is loaded
//     holds these 16 MiB until the process exits.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it. Make that first
//     call outside any stream capture. Later calls only launch kernels. The address is
//     kept per device in a plain table: two threads that make their first call on a device
//     at the same moment both look it up and store the same value, which is harmless.
//     The device is the one that is current at the call, which must be the stream's.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine; inputs and outputs
//     are the caller's.
//   * All calls share the one array, which keeps whatever the last call left in it. Nothing
//     in it has to start at zero: every value the merge step reads was written by the same
//     call just before. But two calls that overlap on the GPU (different streams, or
//     different threads launching at once) race on it; run them one after the other.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define MB_STATIC_SCRATCH_FLOATS (4ll * 1024 * 1024)

// Arguments as for mb_paged_attention_simt, without `scratch` and `scratch_floats`.
// Returns 0, or an MB_ERR_* code (5 when the problem is larger than the built-in scratch).
int mb_paged_attention_static(const void* qkv, int q_row_stride, const void* k_pages,
                              const void* v_pages, const int* table, int max_pages,
                              const int* q_start, const int* kv_len, const int* seq_of_token,
                              void* out, int tokens, int num_seqs, int max_q_len, int n_q,
                              int n_kv, int d, int page_size, float scale, int window,
                              int num_splits, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
