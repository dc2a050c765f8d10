// Paged decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in fankh/zllm: it is an addition of this engine.
//
// Who needs it.  The regular entry point (zllm_attention_decode_bf16) takes two scratch
// buffers for the per-split partial results, which its caller allocates.  Some callers cannot
// do that: code that runs inside a CUDA stream capture or under a memory pool that forbids
// new allocations, a plug-in handed only its input and output tensors by a host framework, a
// real-time loop that must not touch the allocator (cudaMalloc can synchronise the device and
// take milliseconds).  For them the scratch lives inside the library, in a fixed array in
// device memory of ZLLM_NOALLOC_SCRATCH_FLOATS floats (16 MiB) that every GPU which loads
// the library holds until the process exits.
//
// What to know before calling it:
//  * Sizes are limited: rows * nq * n_splits * (hd + 2) must not exceed
//    ZLLM_NOALLOC_SCRATCH_FLOATS; larger calls are refused with ZLLM_NOALLOC_TOO_LARGE and a
//    message, nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current).  Make that first call outside any stream capture.
//  * The entry point and everything it calls allocate nothing: no cudaMalloc, no cudaFree, no
//    library routine that allocates.
//  * All calls on a device share the one array, which keeps whatever the last call left in
//    it.  The kernels write every partial they later read, so nothing needs clearing; but two
//    calls that overlap on the GPU (different streams, or a graph replayed concurrently)
//    race on it.  Keep calls on one device ordered.
//  * n_splits must cover the longest row: ceil(keys of the row / 256).  The host cannot check
//    it (positions live on the device); a row that needs more splits than were passed is
//    merged from the splits that were computed only, i.e. its oldest n_splits * 256 keys.
//  * The kernels are launched with programmatic dependent launch and read rows, positions,
//    row_slot, table and every key and value older than a row's own position BEFORE they wait
//    for the kernel launched just before them on the stream.  That kernel may write qkv, out
//    and the keys and values at the rows' own positions, nothing else of the operands.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ZLLM_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define ZLLM_NOALLOC_TOO_LARGE 10002

// Same operands and meaning as zllm_attention_decode_bf16 without the two scratch pointers:
//   qkv [T, (nq + 2 nkv) * hd] bf16; out [T, nq * hd] bf16; rows[n_rows] the decoded rows;
//   positions[T], row_slot[T]; k_pages / v_pages [pages, nkv, bs, hd] bf16;
//   table [slots, max_blocks] int32; scale > 0; window 0 = all keys;
//   n_splits >= splits of the longest row (256 keys per split).
// err / err_len: optional buffer for a message when the return value is not 0.
// Returns 0, a cudaError_t, 10001 (sizes the kernel does not take) or ZLLM_NOALLOC_TOO_LARGE.
int zllm_attention_decode_bf16_noalloc(const void* qkv, void* out, const int* rows, int n_rows, const int* positions,
                                       const int* row_slot, const void* k_pages, const void* v_pages, const int* table,
                                       int max_blocks, int bs, int nq, int nkv, int hd, float scale, int window,
                                       int n_splits, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
