// Allocation-free variant of the split-KV decode attention: same kernels as
// paged_attention_decode, workspace in a static device array (see decode_noalloc.h).
#include "decode_noalloc.h"

#include <cuda_runtime.h>
#include <stdio.h>

#include "ops.h"

namespace {

// Partial outputs [splits, batch, heads, head_dim] followed by log-sum-exps [splits, batch, heads].
static __device__ __align__(256) float g_noalloc_scratch[B200_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};   // device address of the array, per device
thread_local char g_err[256] = "";

int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}

// Once per device, with that device current: turn the symbol into its device address.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(-2, "no current CUDA device");
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_err, sizeof(g_err), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return -3;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" const char* b200_noalloc_last_error(void) { return g_err; }

extern "C" int b200_paged_decode_noalloc(void* out, const void* q, const void* kv_cache, const float* kv_scales,
                                         const int* block_table, const int* seq_lens, int batch, int num_q_heads,
                                         int num_kv_heads, int head_dim, int block_size, int max_blocks,
                                         int64_t num_blocks, int num_splits, float scale, int dtype, int cache_dtype,
                                         void* stream) {
  g_err[0] = 0;
  if (!out || !q || !kv_cache || !block_table || !seq_lens) return fail(-1, "null tensor pointer");
  // every size is checked before anything is computed from it or launched: the pointers come from an embedder
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(-5, "unsupported head_dim (64, 128 and 256 are built)");
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0)
    return fail(-1, "num_q_heads must be a positive multiple of num_kv_heads");
  if (block_size <= 0 || block_size % 16 != 0) return fail(-1, "block_size must be a positive multiple of 16");
  if (max_blocks <= 0) return fail(-1, "max_blocks must be positive");
  if (num_blocks <= 0) return fail(-1, "num_blocks must be positive");
  if (batch < 0) return fail(-1, "batch must not be negative");
  if (batch == 0) return 0;
  if (num_splits < 1) num_splits = 1;
  if (cache_dtype != 0 && kv_scales == nullptr) return fail(-1, "quantised caches need kv_scales");
  if (dtype != 0 && dtype != 1) return fail(-1, "dtype must be 0 (bf16) or 1 (fp16)");
  const uint64_t need = (uint64_t)num_splits * (uint64_t)batch * (uint64_t)num_q_heads * (uint64_t)(head_dim + 1);
  if (num_splits > 1 && need > (uint64_t)B200_NOALLOC_SCRATCH_FLOATS) {
    snprintf(g_err, sizeof(g_err),
             "workspace of %llu floats (splits %d x batch %d x heads %d x (head_dim %d + 1)) exceeds the built-in "
             "scratch of %u floats; lower num_splits or the batch",
             (unsigned long long)need, num_splits, batch, num_q_heads, head_dim, B200_NOALLOC_SCRATCH_FLOATS);
    return -4;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;

  b200::DecodeParams p{};
  p.out = out;
  p.q = q;
  p.q_stride = (int64_t)num_q_heads * head_dim;
  p.kv_cache = kv_cache;
  p.kv_scales = kv_scales;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.query_start_loc = nullptr;
  p.sinks = nullptr;
  p.lse_out = nullptr;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.num_blocks = num_blocks;
  p.num_splits = num_splits;
  p.total_tokens = batch;
  p.scale = scale;
  p.softcap = 0.f;
  p.k_scale = 1.f;
  p.v_scale = 1.f;
  p.window = -1;
  p.causal = 1;
  p.status = nullptr;
  if (num_splits > 1) {
    p.part_out = scratch;
    p.part_lse = scratch + (uint64_t)num_splits * batch * num_q_heads * head_dim;
  }
  const int kind = cache_dtype == 0 ? 0 : (cache_dtype == 1 ? 1 : 2);
  if (b200::paged_attention_decode(p, head_dim, kind, dtype, batch, 1, reinterpret_cast<cudaStream_t>(stream)) != 0)
    return fail(-5, "unsupported head_dim (64, 128 and 256 are built)");
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "launch failed: %s", cudaGetErrorString(e));
    return -6;
  }
  return 0;
}
