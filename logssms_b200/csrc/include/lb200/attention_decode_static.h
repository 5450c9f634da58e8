// lb_attention_decode_static: split-KV paged attention that allocates nothing.
//
// This entry point has no counterpart in the reference (dakingffo/LogSSMs); it exists for callers of
// this library that are not allowed to allocate device memory when they call it:
//   * a host program that carved up the whole device at start-up and forbids cudaMalloc/cudaFree
//     afterwards (a serving process with a fixed memory plan, a plug-in inside another runtime);
//   * a latency-critical loop, where an allocation may synchronise the device or fail late;
//   * a caller written in C or another language that has no tensor allocator (torch's) at hand to
//     create the scratch buffers that `lb_attention_decode` expects from its caller.
// The split-KV kernel needs scratch for the partial results of the key ranges (for every selected
// token, query head and range: head_dim output values plus a running maximum and sum, float32).
// `lb_attention_decode` takes that scratch from the caller.  This variant keeps it in a fixed array in
// the library's own device data segment, so the caller passes inputs and outputs only.
//
// Limits and rules
//   * The array holds LB_ATTN_STATIC_SCRATCH_FLOATS float32 values (4 MiB).  Every GPU that loads the
//     library carries these 4 MiB until the process exits, whether or not this entry point is used.
//   * A call needs sel_tokens * Hq * splits * (head_dim + 2) floats.  A call that needs more is
//     refused with LB_ERR_STATIC_SCRATCH (-4) before anything is launched; use fewer splits, fewer
//     tokens per call, or `lb_attention_decode` with a buffer of your own.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it.  Make that first call outside any stream capture, e.g.
//     once at start-up on a small input.
//   * All calls on a device share the one array and it keeps whatever the last call left in it.  The
//     kernels write every slot they later read within the same call, so nothing has to be cleared
//     between calls; but two calls that may run on the GPU at the same time (different streams, or
//     different host threads on different streams) race on it.  Keep calls on one stream, or order
//     them with events.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine; arguments and results are as
//     for `lb_attention_decode` (see attention_decode.cu).
//
// Returns 0, or a negative refusal code (-1 dtype, -2 a size the kernel does not take, -3 a size
// beyond the kernel's limit, -4 scratch too small), or a positive cudaError_t.  When `err` is not
// null and the call is refused or fails, a one-line message is written there (at most `err_len`
// bytes, always terminated).
#pragma once
#include <stddef.h>

#define LB_ATTN_STATIC_SCRATCH_FLOATS (1u << 20)
#define LB_ERR_STATIC_SCRATCH (-4)

#ifdef __cplusplus
extern "C" {
#endif

int lb_attention_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                               const int* block_table, int bt_stride, const int* token_req,
                               const int* positions, const int* token_list, int sel_tokens, int Hq, int Hkv,
                               int hd, int page_size, float scale, int window, int splits, int dtype,
                               void* stream, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
