// split_attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (WillyBruhn/mini_llm allocates every
// buffer with cudaMalloc when a model or a cache is created and never offers a variant
// without).  It is an addition of this library.
//
// Who needs it: a host program that calls the kernels of libmllm_decode directly through
// their C symbols, without the Python package and so without an allocator that hands out
// cached device memory.  Such a caller has usually fixed its device memory budget when it
// started; a cudaMalloc or cudaFree in its serving loop would also make the whole device wait
// (both calls synchronise it), stalling every other stream for the sake of a few hundred
// kilobytes of scratch.  split_attention needs scratch (partial softmax states per chunk of
// keys, and one counter per (token, head)); mllm_decode_split_attention takes it from the
// caller, this variant brings its own.
//
// How: the scratch is one file-scope array in device memory, present on every GPU that
// loads the library, from load until the process exits:
//     MLLM_STATIC_ACC_FLOATS   floats of partial outputs   (4 MiB)
//     MLLM_STATIC_ML_FLOATS    floats of partial max/sum   (256 KiB)
//     MLLM_STATIC_COUNTERS     int32 counters              (16 KiB)
// A call is refused with a clear error, and launches nothing, if it needs more:
//     n_tokens * n_heads * chunks * head_size <= MLLM_STATIC_ACC_FLOATS
//     n_tokens * n_heads * chunks * 2         <= MLLM_STATIC_ML_FLOATS
//     n_tokens * n_heads                      <= MLLM_STATIC_COUNTERS
// with chunks = ceil(max_blocks * page_size / chunk).
//
// The call allocates nothing and frees nothing (no cudaMalloc, cudaFree or allocating library
// routine).  The FIRST call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and remembers it; make that first call
// before any stream capture begins on that device.
//
// All calls share the one array, and it keeps what the last call left in it.  Each call
// therefore clears the counters it is going to use (a memset on the given stream, before the
// kernel); the partial states need no clearing, every cell that is read was written by the
// same launch.  Two calls whose kernels overlap on the GPU (different streams, or different
// host threads without ordering between them) race on the array: order them.
#pragma once

#define MLLM_STATIC_ACC_FLOATS (1 << 20)
#define MLLM_STATIC_ML_FLOATS (1 << 16)
#define MLLM_STATIC_COUNTERS (1 << 12)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as mllm_decode_split_attention, minus the three scratch
// pointers.  Inputs and outputs are the caller's device memory.  Returns 0 on success; on
// failure a non-zero code, with the text in mllm_decode_last_error().
int mllm_decode_split_attention_static(void* out, long ld_out, const void* q, long ld_q, const void* k_pages,
                                       const void* v_pages, const int* block_table, int max_blocks,
                                       const int* positions, const int* token_item, int n_tokens, int n_heads,
                                       int n_kv_heads, int head_size, int page_size, float scale, int window,
                                       int chunk, void* stream);

#ifdef __cplusplus
}
#endif
