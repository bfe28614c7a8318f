// Small fused memory-bound kernels:
//   fused_qk_norm_rope        per-head RMSNorm(q), RMSNorm(k) + RoPE (NeoX / GPT-J, partial rotary) in place
//                             on the packed qkv GEMM output - one warp per (token, head)
//   qkv_norm_rope_insert      the same for a whole [q | k | v | index_q | index_k] row, with q / index_q gathered into
//                             contiguous outputs and k, v, index_k written into their paged caches (head_dim 128;
//                             fused_minimax_m3_qknorm_rope_kv_insert_kernel.cu:262-480 of the reference)
//   mla_rope_and_cache        RoPE on q_pe / k_pe + insert [kv_c | k_pe] into the bf16 MLA cache, one pass
//   concat_mla_q              q_out[T,H,576] = [ql_nope(512) | q_pe(64)]
//   permute_cols              out[:, j] = a[:, perm[j]]   (GPTQ act-order activation gather)
//   gather_mla_cache          paged MLA cache -> contiguous [sum L, 576] workspace; 656-byte fp8 records are
//                             up-converted (e4m3 * scale | bf16 rope) on the way
//   gather_indexer_k          paged block-planar indexer K (fp8 + f32 scale) -> contiguous [sum L,128] / [sum L]
// Parity: csrc/fused_qknorm_rope_kernel.cu:104-686, cache_kernels_fused.cu:24, concat_mla_q.cuh:14,
// permute_cols.cu:17, cache_kernels.cu:642-713 and :1074-1443 of the reference.
#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------------------------
// qkv [T, (Hq + Hk + Hv) * D]; cos_sin fp32 [max_pos, rot] = [cos(rot/2) | sin(rot/2)].  D = 32 * PER.
template <typename T, int PER>
__global__ void fused_qk_norm_rope_kernel(T* __restrict__ qkv, const T* __restrict__ q_weight,
                                          const T* __restrict__ k_weight, const float* __restrict__ cos_sin,
                                          const int64_t* __restrict__ positions, int tokens, int hq, int hk, int hv,
                                          int rot, int is_neox, float eps, int gemma) {
  constexpr int D = 32 * PER;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = hq + hk;
  if (gw >= tokens * heads) return;
  const int t = gw / heads, h = gw % heads;
  T* p = qkv + (size_t)t * (hq + hk + hv) * D + (size_t)h * D + lane * PER;
  const T* w = (h < hq ? q_weight : k_weight) + lane * PER;
  float v[PER];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = to_f(p[i]);
    ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / D + eps);
#pragma unroll
  for (int i = 0; i < PER; ++i) v[i] = to_f(from_f<T>(v[i] * inv * (to_f(w[i]) + (gemma ? 1.f : 0.f))));
  if (rot > 0) {
    const float* cs = cos_sin + (size_t)positions[t] * rot;
    const int half = rot >> 1;
    if (is_neox) {
      // pair (i, i + half): the partner sits `half / PER` lanes away at the same register index
      const int dl = half / PER;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int idx = lane * PER + i;
        const bool lo = idx < half;
        const int src = lo ? lane + dl : lane - dl;
        const float other = __shfl_sync(0xffffffffu, v[i], src & 31);
        if (idx < rot) {
          const int j = lo ? idx : idx - half;
          const float c = cs[j], s = cs[half + j];
          v[i] = lo ? v[i] * c - other * s : v[i] * c + other * s;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        const int idx = lane * PER + i;
        if (idx < rot) {
          const float c = cs[idx >> 1], s = cs[half + (idx >> 1)];
          const float x = v[i], y = v[i + 1];
          v[i] = x * c - y * s;
          v[i + 1] = y * c + x * s;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) p[i] = from_f<T>(v[i]);
}

// ---------------------------------------------------------------------------------------------------------
// One CTA per token.  q_pe [T, H, 64] and k_pe [T, 64] rotated in place; cache [slots, 576] receives [kv_c | k_pe].
template <typename T>
__global__ void mla_rope_and_cache_kernel(T* __restrict__ q_pe, T* __restrict__ k_pe, const T* __restrict__ kv_c,
                                          T* __restrict__ cache, const float* __restrict__ cos_sin,
                                          const int64_t* __restrict__ positions, const int64_t* __restrict__ slots,
                                          int heads, int64_t q_tok_stride, int64_t kpe_stride, int64_t kvc_stride,
                                          int is_neox, int64_t num_slots) {
  const int t = blockIdx.x;
  const float* cs = cos_sin + (size_t)positions[t] * 64;
  auto rotate = [&](T* x, int pair) {
    const int i0 = is_neox ? pair : 2 * pair, i1 = is_neox ? pair + 32 : 2 * pair + 1;
    const float c = cs[pair], s = cs[32 + pair];
    const float a = to_f(x[i0]), b = to_f(x[i1]);
    x[i0] = from_f<T>(a * c - b * s);
    x[i1] = from_f<T>(b * c + a * s);
  };
  for (int i = threadIdx.x; i < heads * 32; i += blockDim.x)
    rotate(q_pe + (size_t)t * q_tok_stride + (size_t)(i >> 5) * 64, i & 31);
  T* kp = k_pe + (size_t)t * kpe_stride;
  if (threadIdx.x < 32) rotate(kp, threadIdx.x);
  __syncthreads();
  const int64_t slot = slots[t];
  if (slot < 0 || slot >= num_slots) return;
  T* dst = cache + (size_t)slot * 576;
  const T* src = kv_c + (size_t)t * kvc_stride;
  for (int v = threadIdx.x; v < 64; v += blockDim.x)
    reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(src)[v];
  for (int v = threadIdx.x; v < 8; v += blockDim.x)
    reinterpret_cast<uint4*>(dst + 512)[v] = reinterpret_cast<const uint4*>(kp)[v];
}

template <typename T>
__global__ void concat_mla_q_kernel(T* __restrict__ out, const T* __restrict__ nope, const T* __restrict__ pe,
                                    int64_t rows, int64_t nope_stride, int64_t pe_stride) {
  const int64_t r = blockIdx.x;     // one (token, head) row per CTA of 72 16-byte vectors
  if (r >= rows) return;
  for (int v = threadIdx.x; v < 72; v += blockDim.x) {
    const uint4 x = v < 64 ? reinterpret_cast<const uint4*>(nope + r * nope_stride)[v]
                           : reinterpret_cast<const uint4*>(pe + r * pe_stride)[v - 64];
    reinterpret_cast<uint4*>(out + r * 576)[v] = x;
  }
}

template <typename T>
__global__ void permute_cols_kernel(T* __restrict__ out, const T* __restrict__ a, const int* __restrict__ perm,
                                    int cols, int64_t lda) {
  const int64_t r = blockIdx.x;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) out[r * cols + j] = a[r * lda + perm[j]];
}

// ---------------------------------------------------------------------------------------------------------
// dst [total, 576] T; sequence b occupies rows [cu_seq_lens[b], cu_seq_lens[b+1]) and reads its tokens
// seq_starts[b] + i (seq_starts optional) through block_table.  One warp per token.
template <typename T>
__global__ void gather_mla_cache_kernel(T* __restrict__ dst, const uint8_t* __restrict__ cache,
                                        const int* __restrict__ block_table, const int* __restrict__ cu_seq_lens,
                                        const int* __restrict__ seq_starts, int batch, int max_blocks, int block_size,
                                        int records) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = cu_seq_lens[batch];
  if (gw >= total) return;
  int lo = 0, hi = batch;                       // binary search: cu[b] <= gw < cu[b+1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_seq_lens[mid] <= gw) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int pos = gw - cu_seq_lens[b] + (seq_starts ? seq_starts[b] : 0);
  const int64_t blk = block_table[(size_t)b * max_blocks + pos / block_size];
  const int64_t slot = blk * block_size + pos % block_size;
  T* out = dst + (size_t)gw * 576;
  if (!records) {
    const uint4* src = reinterpret_cast<const uint4*>(cache + (size_t)slot * 576 * sizeof(T));
    for (int v = lane; v < 72; v += 32) reinterpret_cast<uint4*>(out)[v] = src[v];
    return;
  }
  const uint8_t* rec = cache + (size_t)slot * 656;
  const float* sc = reinterpret_cast<const float*>(rec + 512);
  for (int v = lane; v < 64; v += 32) {         // 8 fp8 values -> 8 T
    const uint2 q = reinterpret_cast<const uint2*>(rec)[v];
    const float s = sc[v >> 4];
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = fp8_e4m3_to_float((uint8_t)(q.x >> (8 * i))) * s;
#pragma unroll
    for (int i = 0; i < 4; ++i) f[4 + i] = fp8_e4m3_to_float((uint8_t)(q.y >> (8 * i))) * s;
    reinterpret_cast<uint4*>(out)[v] = pack8<T>(f);
  }
  const __nv_bfloat16* pe = reinterpret_cast<const __nv_bfloat16*>(rec + 528);
  for (int i = lane; i < 64; i += 32) out[512 + i] = from_f<T>(__bfloat162float(pe[i]));
}

// cache uint8 [blocks, bs*(128+4)] block-planar; dst_k uint8 [total,128], dst_s f32 [total].
__global__ void gather_indexer_k_kernel(uint8_t* __restrict__ dst_k, float* __restrict__ dst_s,
                                        const uint8_t* __restrict__ cache, const int* __restrict__ block_table,
                                        const int* __restrict__ cu_seq_lens, int batch, int max_blocks, int block_size) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = cu_seq_lens[batch];
  if (gw >= total) return;
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_seq_lens[mid] <= gw) lo = mid; else hi = mid;
  }
  const int pos = gw - cu_seq_lens[lo];
  const int64_t blk = block_table[(size_t)lo * max_blocks + pos / block_size];
  const int off = pos % block_size;
  const uint8_t* base = cache + (size_t)blk * block_size * 132;
  if (lane < 8) reinterpret_cast<uint4*>(dst_k + (size_t)gw * 128)[lane] = reinterpret_cast<const uint4*>(base + off * 128)[lane];
  if (lane == 8) dst_s[gw] = reinterpret_cast<const float*>(base + block_size * 128)[off];
}

// ---------------------------------------------------------------------------------------------------------
// Norm + RoPE + cache inserts of a whole attention input row in one launch (head_dim 128, 4 dims per lane).
// Row of `qkv`: [q (hq) | k (hk) | v (hk) | index_q (niq) | index_k (1)] x 128; one warp per (token, slot):
//   q, index_q   RMSNorm (gemma form, skipped when the weight is null) + partial RoPE -> q_out / iq_out, contiguous
//                [T, heads, 128] so that the attention kernel can address them with a flat tensor map
//   k            norm + RoPE, written back in place and into the K plane of the paged cache
//   v            copied into the V plane
//   index_k      norm + RoPE -> index cache row of the token's slot
// iq_out and the index cache are 16-bit or e4m3 bytes (direct saturating cast: normalised values are O(1)).
// Tokens at or beyond `insert_tokens` and negative slots get no cache rows.
template <typename T>
__device__ __forceinline__ void norm_rope4(float (&v)[4], const T* w, const float* cs, int rot, int is_neox, float eps,
                                           int gemma, int lane) {
  if (w != nullptr) {
    float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / 128.f + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = to_f(from_f<T>(v[i] * inv * (to_f(w[lane * 4 + i]) + (gemma ? 1.f : 0.f))));
  }
  if (rot <= 0) return;
  const int half = rot >> 1;
  if (is_neox) {
    const int dl = half / 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = lane * 4 + i;
      const bool lo = idx < half;
      const float other = __shfl_sync(0xffffffffu, v[i], (lo ? lane + dl : lane - dl) & 31);
      if (idx < rot) {
        const int j = lo ? idx : idx - half;
        const float c = cs[j], s = cs[half + j];
        v[i] = lo ? v[i] * c - other * s : v[i] * c + other * s;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; i += 2) {
      const int idx = lane * 4 + i;
      if (idx < rot) {
        const float c = cs[idx >> 1], s = cs[half + (idx >> 1)];
        const float x = v[i], y = v[i + 1];
        v[i] = x * c - y * s;
        v[i + 1] = y * c + x * s;
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]) {
  T o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = from_f<T>(v[i]);
  *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(o);
}
__device__ __forceinline__ void store4_fp8(uint8_t* p, const float (&v)[4]) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) w |= (uint32_t)float_to_fp8_e4m3(fminf(fmaxf(v[i], -448.f), 448.f)) << (8 * i);
  *reinterpret_cast<uint32_t*>(p) = w;
}

struct QkvInsertParams {
  int tokens, insert_tokens, hq, hk, niq, has_ik, insert_v;
  int rot, is_neox, gemma, idx_fp8, block_size;
  float eps;
  int64_t row_stride;          // elements between two rows of qkv
  int64_t num_slots;
};

template <typename T>
__global__ void __launch_bounds__(256)
qkv_norm_rope_insert_kernel(const QkvInsertParams p, T* __restrict__ qkv, const T* __restrict__ q_w,
                            const T* __restrict__ k_w, const T* __restrict__ iq_w, const T* __restrict__ ik_w,
                            const float* __restrict__ cos_sin, const int64_t* __restrict__ positions,
                            const int64_t* __restrict__ slot_mapping, T* __restrict__ q_out, void* __restrict__ iq_out,
                            T* __restrict__ kv_cache, void* __restrict__ idx_cache) {
  const int lane = threadIdx.x & 31;
  const int v_slots = p.insert_v ? p.hk : 0;
  const int slots = p.hq + p.hk + v_slots + p.niq + p.has_ik;
  const int64_t gw = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (int64_t)p.tokens * slots) return;
  const int t = (int)(gw / slots);
  int s = (int)(gw % slots);
  T* row = qkv + (int64_t)t * p.row_stride;
  const float* cs = cos_sin + (size_t)positions[t] * p.rot;
  const int64_t slot = t < p.insert_tokens ? slot_mapping[t] : -1;
  const bool can_insert = slot >= 0 && slot < p.num_slots;
  const int64_t blk = can_insert ? slot / p.block_size : 0, pos = can_insert ? slot % p.block_size : 0;
  float v[4];
  auto load = [&](const T* src) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = to_f(e[i]);
  };
  if (s < p.hq) {                                                   // ---- q
    load(row + (int64_t)s * 128);
    norm_rope4<T>(v, q_w, cs, p.rot, p.is_neox, p.eps, p.gemma, lane);
    store4<T>(q_out + ((int64_t)t * p.hq + s) * 128 + lane * 4, v);
    return;
  }
  s -= p.hq;
  if (s < p.hk) {                                                   // ---- k
    T* src = row + (int64_t)(p.hq + s) * 128;
    load(src);
    norm_rope4<T>(v, k_w, cs, p.rot, p.is_neox, p.eps, p.gemma, lane);
    store4<T>(src + lane * 4, v);
    if (can_insert && kv_cache != nullptr)
      store4<T>(kv_cache + (((blk * 2 + 0) * p.block_size + pos) * p.hk + s) * 128 + lane * 4, v);
    return;
  }
  s -= p.hk;
  if (s < v_slots) {                                                // ---- v
    if (!can_insert) return;
    load(row + (int64_t)(p.hq + p.hk + s) * 128);
    store4<T>(kv_cache + (((blk * 2 + 1) * p.block_size + pos) * p.hk + s) * 128 + lane * 4, v);
    return;
  }
  s -= v_slots;
  const int64_t idx_base = (int64_t)(p.hq + 2 * p.hk) * 128;       // index_q / index_k follow q | k | v
  if (s < p.niq) {                                                  // ---- index_q
    load(row + idx_base + (int64_t)s * 128);
    norm_rope4<T>(v, iq_w, cs, p.rot, p.is_neox, p.eps, p.gemma, lane);
    const int64_t o = ((int64_t)t * p.niq + s) * 128 + lane * 4;
    if (p.idx_fp8) store4_fp8(static_cast<uint8_t*>(iq_out) + o, v);
    else store4<T>(static_cast<T*>(iq_out) + o, v);
    return;
  }
  // ---- index_k
  load(row + idx_base + (int64_t)p.niq * 128);
  norm_rope4<T>(v, ik_w, cs, p.rot, p.is_neox, p.eps, p.gemma, lane);
  if (!can_insert || idx_cache == nullptr) return;
  const int64_t o = slot * 128 + lane * 4;
  if (p.idx_fp8) store4_fp8(static_cast<uint8_t*>(idx_cache) + o, v);
  else store4<T>(static_cast<T*>(idx_cache) + o, v);
}

// Returns 0, or 1 for an unsupported rotary width.
int qkv_norm_rope_insert(void* qkv, int64_t row_stride, const void* q_w, const void* k_w, const void* iq_w,
                         const void* ik_w, const float* cos_sin, const int64_t* positions, const int64_t* slot_mapping,
                         void* q_out, void* iq_out, void* kv_cache, void* idx_cache, int tokens, int insert_tokens, int hq,
                         int hk, int niq, int has_ik, int insert_v, int rot, int is_neox, int gemma, int idx_fp8,
                         int block_size, int64_t num_slots, float eps, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot > 128 || (rot & 1) || (is_neox && rot > 0 && ((rot / 2) % 4))) return 1;
  QkvInsertParams p{tokens, insert_tokens, hq, hk, niq, has_ik, insert_v, rot, is_neox, gemma, idx_fp8, block_size,
                    eps, row_stride, num_slots};
  const int64_t warps = (int64_t)tokens * (hq + hk + (insert_v ? hk : 0) + niq + has_ik);
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (dtype == 0)
    qkv_norm_rope_insert_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        p, (__nv_bfloat16*)qkv, (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, (const __nv_bfloat16*)iq_w,
        (const __nv_bfloat16*)ik_w, cos_sin, positions, slot_mapping, (__nv_bfloat16*)q_out, iq_out,
        (__nv_bfloat16*)kv_cache, idx_cache);
  else
    qkv_norm_rope_insert_kernel<__half><<<blocks, 256, 0, stream>>>(
        p, (__half*)qkv, (const __half*)q_w, (const __half*)k_w, (const __half*)iq_w, (const __half*)ik_w, cos_sin,
        positions, slot_mapping, (__half*)q_out, iq_out, (__half*)kv_cache, idx_cache);
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
int fused_qk_norm_rope(void* qkv, const void* q_weight, const void* k_weight, const float* cos_sin,
                       const int64_t* positions, int tokens, int hq, int hk, int hv, int head_dim, int rot, int is_neox,
                       float eps, int gemma, int dtype, cudaStream_t stream) {
  const int warps = tokens * (hq + hk);
  if (warps <= 0) return 0;
  const int per = head_dim / 32;
  if (head_dim % 32 || (per != 2 && per != 4 && per != 8) || rot > head_dim || (rot & 1)) return 1;
  if (is_neox && rot > 0 && ((rot / 2) % per)) return 1;
  const int blocks = ceil_div(warps * 32, 256);
#define QK(T, P) fused_qk_norm_rope_kernel<T, P><<<blocks, 256, 0, stream>>>((T*)qkv, (const T*)q_weight, (const T*)k_weight, \
      cos_sin, positions, tokens, hq, hk, hv, rot, is_neox, eps, gemma)
  if (dtype == 0) { if (per == 2) QK(__nv_bfloat16, 2); else if (per == 4) QK(__nv_bfloat16, 4); else QK(__nv_bfloat16, 8); }
  else            { if (per == 2) QK(__half, 2); else if (per == 4) QK(__half, 4); else QK(__half, 8); }
#undef QK
  return 0;
}

void mla_rope_and_cache(void* q_pe, void* k_pe, const void* kv_c, void* cache, const float* cos_sin,
                        const int64_t* positions, const int64_t* slots, int tokens, int heads, int64_t q_tok_stride,
                        int64_t kpe_stride, int64_t kvc_stride, int is_neox, int64_t num_slots, int dtype,
                        cudaStream_t stream) {
  if (tokens <= 0) return;
  if (dtype == 0)
    mla_rope_and_cache_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>((__nv_bfloat16*)q_pe, (__nv_bfloat16*)k_pe, (const __nv_bfloat16*)kv_c, (__nv_bfloat16*)cache, cos_sin, positions, slots, heads, q_tok_stride, kpe_stride, kvc_stride, is_neox, num_slots);
  else
    mla_rope_and_cache_kernel<__half><<<tokens, 128, 0, stream>>>((__half*)q_pe, (__half*)k_pe, (const __half*)kv_c, (__half*)cache, cos_sin, positions, slots, heads, q_tok_stride, kpe_stride, kvc_stride, is_neox, num_slots);
}

void concat_mla_q(void* out, const void* nope, const void* pe, int64_t rows, int64_t nope_stride, int64_t pe_stride,
                  int dtype, cudaStream_t stream) {
  if (rows <= 0) return;
  if (dtype == 0)
    concat_mla_q_kernel<__nv_bfloat16><<<(unsigned)rows, 96, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)nope, (const __nv_bfloat16*)pe, rows, nope_stride, pe_stride);
  else
    concat_mla_q_kernel<__half><<<(unsigned)rows, 96, 0, stream>>>((__half*)out, (const __half*)nope, (const __half*)pe, rows, nope_stride, pe_stride);
}

void permute_cols(void* out, const void* a, const int* perm, int64_t rows, int cols, int64_t lda, int dtype,
                  cudaStream_t stream) {
  if (rows <= 0) return;
  if (dtype == 0)
    permute_cols_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)a, perm, cols, lda);
  else
    permute_cols_kernel<__half><<<(unsigned)rows, 256, 0, stream>>>((__half*)out, (const __half*)a, perm, cols, lda);
}

void gather_mla_cache(void* dst, const void* cache, const int* block_table, const int* cu_seq_lens,
                      const int* seq_starts, int batch, int max_blocks, int block_size, int max_total, int records,
                      int dtype, cudaStream_t stream) {
  if (max_total <= 0) return;
  const int blocks = ceil_div(max_total * 32, 256);
  if (dtype == 0)
    gather_mla_cache_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)dst, (const uint8_t*)cache, block_table, cu_seq_lens, seq_starts, batch, max_blocks, block_size, records);
  else
    gather_mla_cache_kernel<__half><<<blocks, 256, 0, stream>>>((__half*)dst, (const uint8_t*)cache, block_table, cu_seq_lens, seq_starts, batch, max_blocks, block_size, records);
}

void gather_indexer_k(void* dst_k, float* dst_s, const void* cache, const int* block_table, const int* cu_seq_lens,
                      int batch, int max_blocks, int block_size, int max_total, cudaStream_t stream) {
  if (max_total <= 0) return;
  gather_indexer_k_kernel<<<ceil_div(max_total * 32, 256), 256, 0, stream>>>((uint8_t*)dst_k, dst_s, (const uint8_t*)cache,
                                                                          block_table, cu_seq_lens, batch, max_blocks, block_size);
}

}  // namespace b200
