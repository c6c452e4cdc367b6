// Declaration of the allocation-free entry point of the tensor-core attention library.
//
// This entry point has no counterpart in the reference (mirceamironenco/tokensprint): it
// exists for callers of this library that cannot allocate device memory.
//
// Who they are.  A host program that embeds the attention kernel without torch and has
// no allocator of its own, a latency-critical loop that must not touch the allocator's
// locks, or a process whose device memory has been handed out in full to other pools, so
// that a cudaMalloc at this point would fail.  The split-key decode path of
// ts_attention_paged_mma needs scratch memory for the partial results of the key splits,
// and there the caller has to bring it.  ts_attention_paged_mma_noalloc brings its own:
// a file-scope device array inside the library.
//
// The limit.  The array holds TS_ATTENTION_NOALLOC_SCRATCH_FLOATS float32 values (8 MiB).
// Every GPU on which this library is loaded holds that array from load until the
// process exits, used or not.  A call needs tokens * query_heads * splits * (head_dim + 2)
// floats (ts_attention_mma_scratch_floats tells); a call that needs more is refused with
// TS_ERR_SCRATCH_LIMIT and nothing is launched.  splits == 1 needs no scratch at all.
//
// Set-up.  The first call on a device looks the array's device address up once
// (cudaGetSymbolAddress, with that device current) and remembers it per device.  Make
// that first call outside any stream capture.
//
// Sharing.  All calls use the same array.  Nothing in it has to start at zero: every
// value the merge step reads was written by the split CTAs of the same call, and stale
// contents of earlier calls are never read.  But two calls that overlap on the GPU (on
// two streams, or from two threads) race on the array and give wrong results; run them
// one after the other on one stream, or give the second caller the entry point that
// takes scratch from outside.
//
// It allocates nothing: no cudaMalloc, cudaFree or allocating library call, on any path.
// Inputs and outputs are the caller's, exactly as for ts_attention_paged_mma.
#pragma once

#define TS_ATTENTION_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TS_ERR_SCRATCH_LIMIT (-3)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as ts_attention_paged_mma without `scratch`.  Returns 0, a cudaError_t,
// TS_ERR_BAD_ARGUMENT (-1), TS_ERR_UNSUPPORTED_SIZE (-2) or TS_ERR_SCRATCH_LIMIT (-3).
int ts_attention_paged_mma_noalloc(const void* q, const void* kcache, const void* vcache, void* out,
                                   const int* cu_q, const int* ctx_len, const int* block_table,
                                   const int* seq_index, int max_blocks, int page, int T, int B,
                                   int max_q, int nq, int nkv, float scale, int window, int splits,
                                   void* stream);

// The stated maximum, for callers that want to size their batches to it.
long long ts_attention_noalloc_scratch_floats(void);

// A sentence for a return code of the entry point above (static storage).
const char* ts_attention_noalloc_error_text(int code);

#ifdef __cplusplus
}
#endif
