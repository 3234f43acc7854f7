// Single-token paged attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in mlx-lm; it exists for users of this
// library alone.
//
// Who needs it.  mlxb_attention_decode() (attention.cu) cuts each row's keys
// into chunks and needs scratch memory for the per-chunk partial results; its
// caller allocates that scratch.  Some callers cannot: code that runs inside a
// region where the CUDA allocator must not be entered (a host callback, a
// real-time loop with a no-allocation rule, a process whose memory is handed out
// once at start-up by another owner), or a thin foreign-language binding that
// has no allocator of its own to ask.  For them this variant keeps the scratch
// in a fixed array inside the library.
//
// What it costs.  The array is MLXB_NOALLOC_SCRATCH_FLOATS float32 (4 MiB), plus
// MLXB_NOALLOC_COUNTERS int32 ticket counters (256 KiB) for n_rows * n_q_heads.
// Every GPU on which the library is loaded holds it from load until the process
// exits, whether or not this function is ever called.
//
// Limits.  n_rows * n_q_heads * n_chunks_max * (head_dim + 2) must not exceed
// MLXB_NOALLOC_SCRATCH_FLOATS; a larger request is refused with MLXB_BAD_ARG and
// a message in mlxb_last_error() (it is never truncated).  Example: 64 rows of a
// 16-head model with 64-wide heads and 1024 positions in chunks of 128 need
// 64*16*8*66 = 540,672 floats.
//
// First call.  The first call on each device looks up the array's device
// address (cudaGetSymbolAddress, with that device current) and remembers it; it
// launches nothing extra but it is a runtime call that must not happen inside a
// stream capture, so make the first call on a device outside any capture.
//
// Sharing.  All calls on a device use the same array, and it keeps whatever the
// previous call left there.  No partial result has to start at zero: each one
// that is read has been written earlier in the same call.  The ticket counters
// do have to be zero at the start of a call; they are zero when the library is
// loaded and the kernel puts each one back to zero itself, so a caller has
// nothing to clear (a call that was aborted by a device fault would leave them
// undefined, as it leaves the whole context).  Two calls that overlap on the GPU (different streams, or graphs
// replayed concurrently) would overwrite each other's partial results: run calls
// on one device one after the other, i.e. on one stream.
//
// Positions.  n_chunks_max * chunk has to cover the largest position among the
// rows.  A row whose position lies at or beyond that product (or is negative) is
// left out: its output row is not written, MLXB_ST_POSITION_RANGE (2) is set in
// *status, and it takes no ticket, so the counters stay zero and later calls are
// not disturbed.  Read *status after the call if positions come from outside.
//
// It calls no cudaMalloc, cudaFree or any other allocating routine.  Inputs and
// the output are the caller's, exactly as for mlxb_attention_decode(); only the
// `partial` argument is gone.
#pragma once

#include <cuda_runtime.h>

#define MLXB_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define MLXB_NOALLOC_COUNTERS (1 << 16)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, a negative MLXB_* code for a refused size or option, or a
// positive cudaError_t.  Arguments as mlxb_attention_decode() without `partial`.
int mlxb_attention_decode_noalloc(int dtype, const void* q, int ldq, const int* rows, const int* positions,
                                  const int* token_req, const int* block_table, int max_pages, int n_pages,
                                  int page, int n_q_heads, int n_kv_heads, int head_dim, int window, float scale,
                                  const void* k_pool, const void* v_pool, int n_chunks_max, int chunk, void* out,
                                  int ldo, int n_rows, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
