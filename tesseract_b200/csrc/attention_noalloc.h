// Split decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (Leikoe/tesseract), whose attention
// keeps no partial results at all; it exists because this package's split decode kernel does.
//
// Who needs it.  The ordinary path (tb_attention_mma, driven from Python) takes the buffers for
// the per-split partial results from the caller, who gets them from an allocator.  Some callers
// have no allocator to ask: a host program that hands the GPU's whole memory to its own pool at
// start-up and treats any later cudaMalloc as a fault; a latency-bound loop where an allocation
// (which may synchronise the whole device) is forbidden once serving has begun; a plug-in that
// is handed raw pointers through a C interface and owns nothing.  For them the partial results
// live in an array that is part of the library image itself.
//
// The limit.  The array holds TB_NOALLOC_SCRATCH_FLOATS 32-bit floats (16 MiB).  Every GPU on
// which this library is loaded carries that array from load until the process exits, whether the
// entry point is ever called or not.  A call with at most 8 splits needs none of it (its splits meet
// inside a thread-block cluster), so no limit applies to it, however many rows it has.  A call with
// more than 8 splits needs
//     splits * num_seqs * num_kv_heads * 16 * (padded_head_dim + 2) floats (+ up to 63 of padding),
// where padded_head_dim is head_dim rounded up to 32, 64, 128 or 256: sixteen folded rows for every
// (split, sequence, kv head), whatever the number of rows.  Such a call that needs more, or that has more
// than TB_NOALLOC_COUNTERS (sequence, kv head) pairs (a second, 64 KiB static array counts the splits that
// have finished for each pair), is refused with TB_NOALLOC_TOO_LARGE and nothing is launched.
//
// Rules of use.
//  * The first call with more than 8 splits on each device looks the array's device address up (once,
//    with that device current).  Make that first call outside of any stream capture.  Two host threads
//    that make it at the same moment both look the address up and both store the same value, which is
//    the only reason the unguarded cache is safe.
//  * All calls share the arrays, and they keep whatever the last call left in them.  Nothing in the
//    float array has to start at zero: every slot the merge step reads is written earlier in the same
//    call.  The counters must be zero when a call starts; they are zero at load, and the split that
//    merges puts its counter back to zero, so a call that ran to completion leaves them ready.
//  * Because the array is shared, two calls whose kernels can overlap on the GPU (different
//    streams, or different host threads) race on it.  Keep calls on one device in stream order.
//  * Only sequences with at most 16 folded rows (new tokens * num_heads / num_kv_heads) are
//    computed, exactly as tb_attention_mma does with run_tiles = 0, run_decode = 1.
//  * It never calls cudaMalloc, cudaFree, or any routine that allocates.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define TB_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define TB_NOALLOC_COUNTERS 16384
#define TB_NOALLOC_TOO_LARGE (-5)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, a negative refusal code (see tb_attention_noalloc_strerror) or a positive cudaError_t.
// Arguments are those of tb_attention_mma without the scratch pointers and the kernel selection.
int tb_attention_decode_noalloc(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                                const int* row_start, const int* seq_begin, const int* block_table, int bt_stride,
                                int num_seqs, int total_rows, int max_rows_per_seq, int num_heads, int num_kv_heads,
                                int head_dim, int page_size, int window, float scale, int splits,
                                cudaStream_t stream);

// How many floats of the array a call with these sizes needs: 0 up to 8 splits (negative: the sizes
// themselves are refused).
int64_t tb_attention_noalloc_floats_needed(int splits, int num_seqs, int num_kv_heads, int head_dim);

// A sentence for a return code of tb_attention_decode_noalloc.
const char* tb_attention_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
