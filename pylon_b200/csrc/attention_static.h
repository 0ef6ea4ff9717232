// Declaration of the allocation-free attention entry point (attention_static.cu).
//
// This entry point has no counterpart in raun6k/Pylon: the reference never hands its
// callers a C interface, and its attention call allocates through PyTorch.  It exists for
// users of this library who must not allocate device memory at the moment they need
// attention: code that runs after an engine has given every free byte of the GPU to its
// cache pool (a later cudaMalloc there simply fails), code inside a latency-critical loop
// where an allocator call may synchronise the device, and hosts that embed the library
// without PyTorch's allocator at all.  Such callers own their inputs and outputs already;
// the only memory the attention needs beyond those is its scratch for partial results and a
// counter per (row, KV head), and this entry point keeps both inside the library.
#pragma once

#include <cuda_runtime.h>

// Floats of scratch built into the library: 4 Mi floats = 16 MiB, held on every GPU that
// loads the library until the process exits.
#define PYLON_STATIC_SCRATCH_FLOATS (4u * 1024u * 1024u)
// Built-in counters, one per (row, KV head) of a call.
#define PYLON_STATIC_COUNTERS (64u * 1024u)

extern "C" {

// Same arguments and result as pylon_paged_attention_mma without the scratch pointer, the
// counters and the number of decode blocks (chosen here); see attention_static.cu for the
// rules of use.
int pylon_paged_attention_mma_static(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                     void* out, const int* q_start, const int* kv_len, const int* block_table,
                                     int table_width, int page_size, int num_pages, int nq, int nkv, int window,
                                     float scale, int num_rows, int total_tokens, int max_q, int num_splits,
                                     cudaStream_t stream);

// Floats of built-in scratch (PYLON_STATIC_SCRATCH_FLOATS), for callers that size their batches by it.
long long pylon_static_scratch_floats();

// 0, or non-zero after a kernel of an earlier call on the current device gave up waiting for one of
// its TMA copies (that call's output is void); -1 if the word cannot be read.  Synchronises the device.
int pylon_static_error_word();

// Zeroes the built-in counters and the error word of the current device (after the word was non-zero, before the
// next call).  Synchronises the device; allocates nothing.  0, or -2 with an error text.
int pylon_static_reset();

// For tests of the error handling: writes one counter and the error word from the host.
int pylon_static_inject(int pair, unsigned count, int error_code);
}
