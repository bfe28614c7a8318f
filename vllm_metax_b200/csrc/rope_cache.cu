// Rotary embedding and paged-KV-cache writes.
//
//  * rope_and_cache: RoPE on q and k in place AND scatter of (rotated k, v) into
//    the paged cache in one pass - one warp per (token, head); the head is staged
//    in shared memory so any rotary width / pairing style works.  Cache element
//    types: same as activations, e4m3 with a static scale, or int8 / e4m3 with a
//    per-(token, head) symmetric scale written to a side tensor.  Passing null
//    pointers turns the kernel into plain RoPE or plain reshape_and_cache.
//  * block copy, MLA latent cache writes (bf16 576-wide and the 656-byte fp8
//    record), DSA indexer key quantise + insert, gathers.
//
// Cache layout: [num_blocks, 2, block_size, num_kv_heads, head_dim]; scales
// [num_blocks, 2, block_size, num_kv_heads] f32.
// Parity: csrc/pos_encoding_kernels.cu:77, cache_kernels.cu:250-605,
// cache_kernels_fused.cu:24 of the reference.
#include "common.cuh"

namespace b200 {

enum CacheKind : int { kCacheSame = 0, kCacheFp8Static = 1, kCacheInt8Dyn = 2, kCacheFp8Dyn = 3 };

constexpr int kRopeWarps = 8;
constexpr int kMaxHeadDim = 576;

template <typename T>
__global__ void __launch_bounds__(kRopeWarps * 32)
rope_and_cache_kernel(const int64_t* __restrict__ positions, T* __restrict__ q, T* __restrict__ k,
                      const T* __restrict__ v, const float* __restrict__ cos_sin, int rot, int head_dim, int num_q,
                      int num_kv, int64_t q_stride, int64_t k_stride, int64_t v_stride, int is_neox, int rot_offset,
                      int inverse, void* __restrict__ kv_cache, float* __restrict__ kv_scales,
                      const int64_t* __restrict__ slot_mapping, int block_size, int64_t num_slots, int cache_kind,
                      float k_scale, float v_scale, int tokens, StatusWord* status) {
  __shared__ float stage[kRopeWarps][kMaxHeadDim];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = num_q + 2 * num_kv;
  const int64_t gw = (int64_t)blockIdx.x * kRopeWarps + w;
  if (gw >= (int64_t)tokens * heads_total) return;
  const int t = (int)(gw / heads_total);
  const int h = (int)(gw % heads_total);
  const bool is_q = h < num_q;
  const bool is_k = !is_q && h < num_q + num_kv;
  const bool is_v = !is_q && !is_k;
  if (is_q && (q == nullptr || positions == nullptr)) return;
  if (is_k && k == nullptr) return;
  if (is_v && (v == nullptr || kv_cache == nullptr)) return;
  const int hh = is_q ? h : (is_k ? h - num_q : h - num_q - num_kv);
  T* src = is_q ? q + t * q_stride + (int64_t)hh * head_dim
                : (is_k ? k + t * k_stride + (int64_t)hh * head_dim
                        : const_cast<T*>(v) + t * v_stride + (int64_t)hh * head_dim);
  float* buf = stage[w];
  for (int e = lane; e < head_dim; e += 32) buf[e] = to_f(src[e]);
  __syncwarp();
  const bool do_rope = !is_v && positions != nullptr && rot > 0;
  const int half = rot >> 1;
  const float* cs = do_rope ? cos_sin + positions[t] * (int64_t)rot : nullptr;

  // cache destination
  int64_t slot = -1;
  if (!is_q && kv_cache != nullptr) {
    slot = slot_mapping[t];
    if (slot >= num_slots) {
      report_status(status, kBadIndex, 10, (int)num_slots, (int)slot);
      slot = -1;
    }
  }
  const int64_t blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? (int)(slot % block_size) : 0;
  const int64_t cache_row = ((blk * 2 + (is_v ? 1 : 0)) * block_size + off) * num_kv + hh;  // (token, head) index

  constexpr int kPer = (kMaxHeadDim + 31) / 32;
  float outv[kPer];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int e = lane + 32 * j;
    if (e >= head_dim) break;
    float x = buf[e];
    const int r = e - rot_offset;
    if (do_rope && r >= 0 && r < rot) {
      int p;
      float other;
      bool first;
      if (is_neox) {
        first = r < half;
        p = first ? r : r - half;
        other = buf[rot_offset + (first ? r + half : r - half)];
      } else {
        first = (r & 1) == 0;
        p = r >> 1;
        other = buf[rot_offset + (first ? r + 1 : r - 1)];
      }
      const float c = cs[p];
      const float s = inverse ? -cs[half + p] : cs[half + p];
      x = first ? (x * c - other * s) : (x * c + other * s);
      x = to_f(from_f<T>(x));  // value as stored in the activation dtype
      src[e] = from_f<T>(x);
    }
    outv[j] = x;
    amax = fmaxf(amax, fabsf(x));
  }
  if (slot < 0) return;
  const int64_t base = cache_row * head_dim;
  if (cache_kind == kCacheSame) {
    T* dst = reinterpret_cast<T*>(kv_cache) + base;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int e = lane + 32 * j;
      if (e < head_dim) dst[e] = from_f<T>(outv[j]);
    }
  } else if (cache_kind == kCacheFp8Static) {
    uint8_t* dst = reinterpret_cast<uint8_t*>(kv_cache) + base;
    const float inv = 1.f / (is_v ? v_scale : k_scale);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int e = lane + 32 * j;
      if (e < head_dim) dst[e] = float_to_fp8_e4m3(outv[j] * inv);
    }
  } else {
    amax = warp_max(amax);
    const float qmax = cache_kind == kCacheInt8Dyn ? 127.f : 448.f;
    const float sc = fmaxf(amax / qmax, 1e-8f);
    if (lane == 0) kv_scales[cache_row] = sc;
    uint8_t* dst = reinterpret_cast<uint8_t*>(kv_cache) + base;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int e = lane + 32 * j;
      if (e >= head_dim) break;
      const float y = outv[j] / sc;
      if (cache_kind == kCacheInt8Dyn) {
        int qi = __float2int_rn(y);
        qi = max(-128, min(127, qi));
        dst[e] = (uint8_t)(int8_t)qi;
      } else {
        dst[e] = float_to_fp8_e4m3(y);
      }
    }
  }
}

// Vector path for the common serving case: NeoX pairing over the whole head (rot == head_dim), cache of the
// activation dtype.  One thread owns the 16-byte vector at offset 8j of a head and its rotation partner at
// head_dim/2 + 8j, so every load and store is a full 16-byte access and eight neighbouring threads cover a
// 128-byte line; q and k are rotated in place, k and v go to their cache slot in the same pass.
template <typename T>
__global__ void __launch_bounds__(256)
rope_and_cache_vec_kernel(const int64_t* __restrict__ positions, T* __restrict__ q, T* __restrict__ k,
                          const T* __restrict__ v, const float* __restrict__ cos_sin, int head_dim, int num_q,
                          int num_kv, int64_t q_stride, int64_t k_stride, int64_t v_stride, int inverse,
                          T* __restrict__ kv_cache, const int64_t* __restrict__ slot_mapping, int block_size,
                          int64_t num_slots, int tokens, StatusWord* status) {
  const int per_head = head_dim >> 4;                       // (vector, partner) items per head
  const int heads_total = num_q + 2 * num_kv;
  const int items = heads_total * per_head;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (int64_t)tokens * items) return;
  const int t = (int)(gid / items);
  const int it = (int)(gid % items);
  const int h = it / per_head, j = it % per_head;
  const int half = head_dim >> 1;
  const bool is_q = h < num_q;
  const bool is_k = !is_q && h < num_q + num_kv;
  const int hh = is_q ? h : (is_k ? h - num_q : h - num_q - num_kv);
  T* src = is_q ? q + t * q_stride + (int64_t)hh * head_dim
                : (is_k ? k + t * k_stride + (int64_t)hh * head_dim
                        : const_cast<T*>(v) + t * v_stride + (int64_t)hh * head_dim);
  uint4 a = *reinterpret_cast<const uint4*>(src + 8 * j);
  uint4 b = *reinterpret_cast<const uint4*>(src + half + 8 * j);
  if (is_q || is_k) {
    const float* cs = cos_sin + positions[t] * (int64_t)head_dim;
    const float4 c0 = *reinterpret_cast<const float4*>(cs + 8 * j), c1 = *reinterpret_cast<const float4*>(cs + 8 * j + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(cs + half + 8 * j),
                 s1 = *reinterpret_cast<const float4*>(cs + half + 8 * j + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float x1[8], x2[8], o1[8], o2[8];
    unpack8<T>(a, x1);
    unpack8<T>(b, x2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = inverse ? -sn[i] : sn[i];
      o1[i] = x1[i] * c[i] - x2[i] * sg;
      o2[i] = x2[i] * c[i] + x1[i] * sg;
    }
    a = pack8<T>(o1);
    b = pack8<T>(o2);
    *reinterpret_cast<uint4*>(src + 8 * j) = a;
    *reinterpret_cast<uint4*>(src + half + 8 * j) = b;
  }
  if (is_q || kv_cache == nullptr) return;
  const int64_t slot = slot_mapping[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    report_status(status, kBadIndex, 10, (int)num_slots, (int)slot);
    return;
  }
  const int64_t blk = slot / block_size;
  const int off = (int)(slot % block_size);
  T* dst = kv_cache + ((((blk * 2 + (is_k ? 0 : 1)) * block_size + off) * num_kv + hh) * (int64_t)head_dim);
  *reinterpret_cast<uint4*>(dst + 8 * j) = a;
  *reinterpret_cast<uint4*>(dst + half + 8 * j) = b;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

void rope_and_cache(const int64_t* positions, void* q, void* k, const void* v, const float* cos_sin, int rot,
                    int head_dim, int num_q, int num_kv, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                    int is_neox, int rot_offset, int inverse, void* kv_cache, float* kv_scales,
                    const int64_t* slot_mapping, int block_size, int64_t num_slots, int cache_kind, float k_scale,
                    float v_scale, int tokens, int dtype, void* status, cudaStream_t stream) {
  if (tokens <= 0) return;
  if (is_neox && rot == head_dim && rot_offset == 0 && head_dim % 16 == 0 && positions && q && k && v && cos_sin &&
      (kv_cache == nullptr || cache_kind == kCacheSame) && q_stride % 8 == 0 && k_stride % 8 == 0 &&
      v_stride % 8 == 0 && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(kv_cache) && aligned16(cos_sin)) {
    const int64_t items = (int64_t)tokens * (num_q + 2 * num_kv) * (head_dim / 16);
    const int blocks_v = (int)((items + 255) / 256);
    if (dtype == 0)
      rope_and_cache_vec_kernel<__nv_bfloat16><<<blocks_v, 256, 0, stream>>>(
          positions, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, cos_sin, head_dim, num_q, num_kv,
          q_stride, k_stride, v_stride, inverse, (__nv_bfloat16*)kv_cache, slot_mapping, block_size, num_slots, tokens,
          (StatusWord*)status);
    else
      rope_and_cache_vec_kernel<__half><<<blocks_v, 256, 0, stream>>>(
          positions, (__half*)q, (__half*)k, (const __half*)v, cos_sin, head_dim, num_q, num_kv, q_stride, k_stride,
          v_stride, inverse, (__half*)kv_cache, slot_mapping, block_size, num_slots, tokens, (StatusWord*)status);
    return;
  }
  const int64_t warps = (int64_t)tokens * (num_q + 2 * num_kv);
  const int blocks = (int)((warps + kRopeWarps - 1) / kRopeWarps);
  if (dtype == 0)
    rope_and_cache_kernel<__nv_bfloat16><<<blocks, kRopeWarps * 32, 0, stream>>>(
        positions, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, cos_sin, rot, head_dim, num_q,
        num_kv, q_stride, k_stride, v_stride, is_neox, rot_offset, inverse, kv_cache, kv_scales, slot_mapping,
        block_size, num_slots, cache_kind, k_scale, v_scale, tokens, (StatusWord*)status);
  else
    rope_and_cache_kernel<__half><<<blocks, kRopeWarps * 32, 0, stream>>>(
        positions, (__half*)q, (__half*)k, (const __half*)v, cos_sin, rot, head_dim, num_q, num_kv, q_stride,
        k_stride, v_stride, is_neox, rot_offset, inverse, kv_cache, kv_scales, slot_mapping, block_size, num_slots,
        cache_kind, k_scale, v_scale, tokens, (StatusWord*)status);
}

// ---------------------------------------------------------------- block copy
// pairs[i] = (src_block, dst_block); block_bytes is a multiple of 16.
__global__ void copy_blocks_kernel(uint8_t* cache, const int64_t* __restrict__ pairs, int64_t block_bytes) {
  const int64_t src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
  const uint4* s = reinterpret_cast<const uint4*>(cache + src * block_bytes);
  uint4* d = reinterpret_cast<uint4*>(cache + dst * block_bytes);
  for (int64_t i = threadIdx.x; i < block_bytes / 16; i += blockDim.x) d[i] = s[i];
}
void copy_blocks(void* cache, const int64_t* pairs, int num_pairs, int64_t block_bytes, cudaStream_t stream) {
  if (num_pairs <= 0) return;
  copy_blocks_kernel<<<num_pairs, 256, 0, stream>>>((uint8_t*)cache, pairs, block_bytes);
}

// ---------------------------------------------------------------- MLA latent cache
// bf16: cache[slot] = [kv_c(rank) | k_pe(rope)];  fp8_ds_mla (rank 512, rope 64): 656-byte record
// [512 e4m3 | 4 f32 scales (amax/448 per 128) | 64 bf16].
template <typename T>
__global__ void concat_and_cache_mla_kernel(const T* __restrict__ kv_c, const T* __restrict__ k_pe,
                                            void* __restrict__ cache, const int64_t* __restrict__ slot_mapping,
                                            int rank, int rope, int64_t kvc_stride, int64_t kpe_stride,
                                            int64_t num_slots, int fp8_record, StatusWord* status) {
  const int t = blockIdx.x;
  const int64_t slot = slot_mapping[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) report_status(status, kBadIndex, 11, (int)num_slots, (int)slot);
    return;
  }
  const T* c = kv_c + t * kvc_stride;
  const T* p = k_pe + t * kpe_stride;
  if (!fp8_record) {
    T* dst = reinterpret_cast<T*>(cache) + slot * (int64_t)(rank + rope);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = c[i];
    for (int i = threadIdx.x; i < rope; i += blockDim.x) dst[rank + i] = p[i];
    return;
  }
  // 4 warps quantise the four 128-wide tiles, warp 4 (if present) / all copy rope
  uint8_t* rec = reinterpret_cast<uint8_t*>(cache) + slot * 656;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (w < 4) {
    float x[4];
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[i] = to_f(c[w * 128 + lane * 4 + i]);
      m = fmaxf(m, fabsf(x[i]));
    }
    m = warp_max(m);
    const float sc = fmaxf(m / 448.f, 1e-12f);
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) packed |= (uint32_t)float_to_fp8_e4m3(x[i] / sc) << (8 * i);
    reinterpret_cast<uint32_t*>(rec)[w * 32 + lane] = packed;
    if (lane == 0) reinterpret_cast<float*>(rec + 512)[w] = sc;
  } else {
    for (int i = lane; i < 64; i += 32)
      reinterpret_cast<__nv_bfloat16*>(rec + 528)[i] = __float2bfloat16_rn(to_f(p[i]));
  }
}
void concat_and_cache_mla(const void* kv_c, const void* k_pe, void* cache, const int64_t* slot_mapping, int tokens,
                          int rank, int rope, int64_t kvc_stride, int64_t kpe_stride, int64_t num_slots,
                          int fp8_record, int dtype, void* status, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = fp8_record ? 160 : 256;
  if (dtype == 0)
    concat_and_cache_mla_kernel<__nv_bfloat16><<<tokens, th, 0, stream>>>(
        (const __nv_bfloat16*)kv_c, (const __nv_bfloat16*)k_pe, cache, slot_mapping, rank, rope, kvc_stride,
        kpe_stride, num_slots, fp8_record, (StatusWord*)status);
  else
    concat_and_cache_mla_kernel<__half><<<tokens, th, 0, stream>>>((const __half*)kv_c, (const __half*)k_pe, cache,
                                                                   slot_mapping, rank, rope, kvc_stride, kpe_stride,
                                                                   num_slots, fp8_record, (StatusWord*)status);
}

// ---------------------------------------------------------------- DSA indexer K cache
// k [T, 128] -> e4m3 + one f32 scale; block-planar cache: per block [bs*128 B values][bs*4 B scales].
template <typename T>
__global__ void indexer_k_quant_and_cache_kernel(const T* __restrict__ k, uint8_t* __restrict__ cache,
                                                 const int64_t* __restrict__ slot_mapping, int head_dim,
                                                 int block_size, int64_t num_slots, int64_t k_stride, int ue8m0,
                                                 int tokens, StatusWord* status, int kind) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= tokens) return;
  const int64_t slot = slot_mapping[gw];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (lane == 0) report_status(status, kBadIndex, 12, (int)num_slots, (int)slot);
    return;
  }
  const T* src = k + gw * k_stride;
  float x[4];
  float m = 0.f;
  const int per = head_dim / 32;  // 4 for head_dim 128
  for (int i = 0; i < per; ++i) {
    x[i] = to_f(src[lane * per + i]);
    m = fmaxf(m, fabsf(x[i]));
  }
  m = warp_max(m);
  // kind 0: e4m3 keys (scale = amax / 448); kind 1: int8 keys (scale = amax / 127, round to nearest)
  float sc = fmaxf(m / (kind == 1 ? 127.f : 448.f), 1e-10f);
  if (ue8m0) sc = ue8m0_ceil(sc);
  const int64_t blk = slot / block_size;
  const int off = (int)(slot % block_size);
  uint8_t* bbase = cache + blk * (int64_t)block_size * (head_dim + 4);
  uint8_t* dst = bbase + (int64_t)off * head_dim;
  for (int i = 0; i < per; ++i)
    dst[lane * per + i] = kind == 1 ? (uint8_t)(int8_t)max(-127, min(127, __float2int_rn(x[i] / sc)))
                                    : float_to_fp8_e4m3(x[i] / sc);
  if (lane == 0) reinterpret_cast<float*>(bbase + (int64_t)block_size * head_dim)[off] = sc;
}
void indexer_k_quant_and_cache(const void* k, void* cache, const int64_t* slot_mapping, int tokens, int head_dim,
                               int block_size, int64_t num_slots, int64_t k_stride, int ue8m0, int dtype, void* status,
                               cudaStream_t stream, int kind) {
  if (tokens <= 0) return;
  const int th = 256;
  const int blocks = ceil_div(tokens * 32, th);
  if (dtype == 0)
    indexer_k_quant_and_cache_kernel<__nv_bfloat16><<<blocks, th, 0, stream>>>(
        (const __nv_bfloat16*)k, (uint8_t*)cache, slot_mapping, head_dim, block_size, num_slots, k_stride, ue8m0,
        tokens, (StatusWord*)status, kind);
  else
    indexer_k_quant_and_cache_kernel<__half><<<blocks, th, 0, stream>>>((const __half*)k, (uint8_t*)cache,
                                                                        slot_mapping, head_dim, block_size, num_slots,
                                                                        k_stride, ue8m0, tokens, (StatusWord*)status, kind);
}

}  // namespace b200
