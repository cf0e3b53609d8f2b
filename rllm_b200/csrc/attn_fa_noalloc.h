// rllm_attention_fa_noalloc: paged attention with split keys for callers that must not
// allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for this library's
// own users.
//
// Who needs it: code that runs where cudaMalloc is off limits. Examples are a host program
// that handed all of the GPU's memory to its own pool at start-up, a plug-in called from
// inside someone else's stream capture or memory-pool scope (where an allocation either
// fails or silently lands in the wrong pool), and a real-time loop that may not take the
// allocator's lock. The ordinary entry point, rllm_attention_fa, asks such a caller for two
// scratch buffers (partial outputs and softmax statistics of the key ranges) that it would
// have to allocate; this one brings its own.
//
// How: the scratch is a fixed array inside the library, RLLM_NOALLOC_SCRATCH_BYTES long
// (8.25 MiB). Every GPU on which the library's code is loaded holds one copy of it until the
// process exits, whether or not this function is ever called there.
//
// Limits and rules:
//  * With splits > 1 the call needs num_tokens * nh * splits * hd floats for partial outputs
//    (at most RLLM_NOALLOC_PART_O_FLOATS) and num_tokens * nh * splits * 2 floats for the
//    statistics (at most RLLM_NOALLOC_PART_ML_FLOATS). A larger problem is refused with
//    ERR_TOO_LARGE (-4) before anything is launched. With splits == 1 no scratch is used.
//  * cu_q[num_seqs] must equal num_tokens: the size check above is made from num_tokens. Rows that
//    cu_q names beyond it are left out of the sum rather than written past the array.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress) with that device current, and remembers it. Make that first call
//    outside any stream capture; `stream` must belong to the current device.
//  * The function calls no cudaMalloc, cudaFree or other allocating routine. Inputs and the
//    output are the caller's, exactly as for rllm_attention_fa.
//  * All calls on a device share the one array, and it keeps whatever the last call left in
//    it. A call never reads a slot it has not written itself, so nothing has to be cleared;
//    but two calls whose kernels overlap on the GPU (different streams, no ordering between
//    them) race on the array and both results are then undefined. Order such calls.
//
// Arguments and return value are those of rllm_attention_fa without the two scratch pointers:
// 0 on success, a negative code for a refused size or alignment, a positive cudaError_t if a
// launch failed.
#pragma once
#include <stddef.h>

#define RLLM_NOALLOC_PART_O_FLOATS ((size_t)2 * 1024 * 1024)
#define RLLM_NOALLOC_PART_ML_FLOATS ((size_t)64 * 1024)
#define RLLM_NOALLOC_SCRATCH_BYTES ((RLLM_NOALLOC_PART_O_FLOATS + RLLM_NOALLOC_PART_ML_FLOATS) * sizeof(float))

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default")))
int rllm_attention_fa_noalloc(const void* q, int q_stride, const void* kcache, const void* vcache,
                              void* out, int out_stride, const int* cu_q, const int* kv_lens,
                              const int* block_table, int bt_stride, int num_seqs, int num_tokens,
                              int max_q_len, int nh, int nkv, int hd, int page_size, float scale,
                              int window, int splits, void* stream);

#ifdef __cplusplus
}
#endif
