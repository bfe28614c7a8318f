// Split-KV paged decode attention for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of
// this library that run under a fixed memory plan - a host runtime that sized every buffer at
// start-up, a plug-in living inside somebody else's allocator, a capture-heavy serving loop in
// which a cudaMalloc would serialise the device - and therefore cannot hand the kernel the
// float workspace its split-KV path needs (partial outputs and log-sum-exps per split).
//
// The workspace lives in a file-scope `static __device__` array inside the library instead:
//   * capacity B200_NOALLOC_SCRATCH_FLOATS floats (16 MiB); every GPU that loads the library
//     carries that much until the process exits;
//   * a call needs num_splits * batch * num_q_heads * (head_dim + 1) floats and is refused
//     (return value < 0, see b200_noalloc_last_error) when that exceeds the capacity;
//   * the array is shared by ALL calls in the process: two calls that overlap on the GPU
//     (different streams, or graphs replayed concurrently) race on it.  Serialise them.
//   * nothing has to be cleared between calls - every element the reduction reads is written
//     earlier in the same call - but the array does keep the previous call's contents.
//
// The first call on each device looks the array's device address up (the name is only a
// host-side handle, not a device pointer) and raises the kernel's shared-memory limit; with
// CUDA's lazy module loading it is also the moment the driver places the kernels and the
// array on that device.  Make that first call outside any stream capture.  No call allocates
// or frees anything through cudaMalloc / cudaFree or an allocating library routine.
#pragma once
#include <stdint.h>

#define B200_NOALLOC_SCRATCH_FLOATS (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// out          [batch, num_q_heads, head_dim]            same 16-bit type as q
// q            [batch, num_q_heads, head_dim]            one query token per sequence, packed
// kv_cache     [num_blocks, 2, block_size, num_kv_heads, head_dim]
//              cache_dtype 0: same type as q; 1: int8 and 2: e4m3, both with kv_scales
// kv_scales    [num_blocks, 2, block_size, num_kv_heads] f32, or NULL for cache_dtype 0
// block_table  [batch, max_blocks] int32, seq_lens [batch] int32
// dtype        0 = bf16, 1 = fp16;  head_dim in {64, 128, 256};  num_splits >= 1
// stream       a cudaStream_t (NULL = legacy default stream)
// Every size is validated before anything is launched (head_dim, head counts, block_size, max_blocks, num_blocks);
// sequence lengths beyond max_blocks * block_size are clamped by the kernel.
// Returns 0 on success, a negative code otherwise.
int b200_paged_decode_noalloc(void* out, const void* q, const void* kv_cache, const float* kv_scales,
                              const int* block_table, const int* seq_lens, int batch, int num_q_heads,
                              int num_kv_heads, int head_dim, int block_size, int max_blocks, int64_t num_blocks,
                              int num_splits, float scale, int dtype, int cache_dtype, void* stream);

// Text of the last error reported by the function above on the calling thread ("" if none).
const char* b200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
