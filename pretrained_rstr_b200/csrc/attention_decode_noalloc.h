// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in replikativ/pretrained-rstr: it exists for
// programs that embed this library but are not allowed to call cudaMalloc (or any
// allocating routine) themselves -- hosts whose own allocator owns the GPU, plugins under
// a fixed memory budget, code running where an allocation would synchronise the device.
// It runs the same kernel as prb_attention_decode; the kernel's scratch memory (partial
// results of the key splits and one counter per (token, head)) is held in fixed-size
// device arrays inside the library instead of being passed in.
//
// Limits: n_list * n_heads * max_splits * (head_dim + 4) <= 1,048,576 floats and
// n_list * n_heads <= 16,384 (see prb_attention_decode_noalloc_limits); larger launches
// are refused with -3 and nothing runs.  Every GPU that loads the library holds about
// 4.1 MiB for these arrays until the process exits.
//
// The first call on a device looks up the arrays' device addresses (once per device);
// make that call before any stream capture.  Calls share the arrays: do not let two calls
// run on the GPU at the same time.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

void prb_attention_decode_noalloc_limits(long* workspace_floats, int* counters);

int prb_attention_decode_noalloc(void* out, long out_stride, const void* q, long q_stride,
                                 const void* k_pages, const void* v_pages, const int* block_table,
                                 const int* seq_of_token, const int* positions,
                                 const int* token_list, const int* token_count, int n_list,
                                 int n_heads, int kv_heads, int head_dim, int page_size,
                                 int max_pages, int num_pages, float scale, int window,
                                 int max_splits, int split_keys, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
