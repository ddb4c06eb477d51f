// Exported entry points of the decode-attention library (attention_decode.cu).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Attention of one query token per sequence over the paged bfloat16 cache, keys cut into
// `n_splits` runs of `chunk`.  The caller brings the scratch through which the splits are joined:
// ws_o needs n_seqs*n_heads*n_splits*d floats and ws_ml n_seqs*n_heads*n_splits*2 (both may be null
// when n_splits is 1).  n_splits * chunk must cover the longest sequence: keys beyond it are not
// attended to.  Returns 0 or a status; llm_attention_decode_last_error() has the message.
int llm_attention_decode(const void *q, long long q_stride, void *out, long long out_stride, const void *kc,
                         const void *vc, const int *tok_pos, const int *page_table, int pt_stride, int n_seqs,
                         int n_heads, int n_kv, int d, int page_size, int chunk, int n_splits, int window, float scale,
                         float *ws_o, float *ws_ml, cudaStream_t stream);

// The same attention for callers that cannot allocate device memory and have no scratch to hand
// over.  (Nothing in ling0322/libllm corresponds to this entry point: its attention wrapper
// allocates its split accumulators on every call, src/flint/cuda/flash_attn.cc:101-186.)
//
// Who that is: a plug-in running inside a host program that has given all device memory to a pool
// of its own; a control loop that may not call cudaMalloc because an allocation can stall the whole
// device; code that runs after the process has been told to stay within a fixed memory budget.
// Such a caller passes inputs and outputs only.  The scratch is an array built into the library,
// LLM_ATTENTION_DECODE_STATIC_FLOATS floats (8 MiB) that every GPU which loads the library holds
// until the process ends, whether this entry point is used or not.
//
// Limits and rules:
//  * n_seqs * n_heads * n_splits * (d + 2) must not exceed LLM_ATTENTION_DECODE_STATIC_FLOATS
//    (llm_attention_decode_static_floats_needed gives the number); a larger call is refused with a
//    message that says so, and nothing is launched.  With n_splits == 1 no scratch is used.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and keeps it.  Make that first call before any stream capture begins on the
//    device, and from one thread.  The array used is the CURRENT device's: a stream that belongs to
//    another device is refused (make the stream's device current first).
//  * All calls share the one array, and it keeps what the last call left in it.  The kernels write
//    every scratch element they later read, so nothing has to be cleared between calls; but two
//    calls whose kernels may run at the same time (different streams) would overwrite each other's
//    partial results.  Put such calls on one stream or order them yourself.
//  * It calls no cudaMalloc, cudaFree or any other allocating routine.
#define LLM_ATTENTION_DECODE_STATIC_FLOATS (2 * 1024 * 1024)
long long llm_attention_decode_static_floats_needed(int n_seqs, int n_heads, int d, int n_splits);
int llm_attention_decode_static(const void *q, long long q_stride, void *out, long long out_stride, const void *kc,
                                const void *vc, const int *tok_pos, const int *page_table, int pt_stride, int n_seqs,
                                int n_heads, int n_kv, int d, int page_size, int chunk, int n_splits, int window,
                                float scale, cudaStream_t stream);

const char *llm_attention_decode_last_error(void);
int llm_attention_decode_supports(int d, int group);

#ifdef __cplusplus
}
#endif
