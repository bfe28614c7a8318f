// DeepSeek-V4 latent cache records: query normalisation + RoPE and the KV insert in one launch, and the
// dequantising gather that reads records back.
//
// A token's 512-wide latent (448 "nope" + 64 "rope" dims) is stored as a 584-byte record:
//   448 x e4m3 (7 blocks of 64, one power-of-two scale each) | 64 x bf16 (rope dims, already rotated) | 8 scale bytes
//   (7 biased exponents, UE8M0, + 1 pad).
// Inside a cache block the data parts of all tokens come first (block_size x 576 bytes), then the scale bytes
// (block_size x 8), so both arrays stay 16-byte / 8-byte aligned per token.
//
//   v4_qnorm_rope_kv_insert   one warp per (token, slot), 16 dims per lane:
//       slot <  Hq          q_out[t, slot] = rope(rmsnorm(q[t, slot]))        (weightless RMSNorm over 512 dims)
//       slot <  Hq_padded   q_out[t, slot] = 0                                (head padding the attention kernel reads)
//       slot == Hq_padded   record(slot_mapping[t]) = quant(rope(kv[t]))      (skipped for t >= insert tokens, slot < 0)
//     RoPE is the interleaved (GPT-J) form on dims [448, 512) with an fp32 cos|sin table row per position.
//   v4_gather_dequant         dst[i] = bf16(record(slots[i])), slots < 0 -> zeros.
//   v4_inv_rope               attention output: inverse RoPE on the rope dims + regrouping of the heads for the grouped
//                             output projection (vllm_metax/models/deepseek_v4/ops/fused_inv_rope_quant.py:9-166)
//   v4_indexer_q              indexer query: RoPE + per-(token, head) int8 quantisation, scale folded into the head
//                             weights (vllm_metax/models/deepseek_v4/ops/fused_indexer_q.py:36-205)
// Memory-bound elementwise work: every global access is a 16-byte vector, one pass over the data.
// Covers csrc/libtorch_stable/fused_deepseek_v4_qnorm_rope_kv_insert_kernel.cu:165-480 of the reference and the
// read side of its _gather_k_cache_kernel (vllm_metax/models/deepseek_v4/ops/cache_utils.py:7).
#include "common.cuh"
#include "ops.h"

namespace b200 {

constexpr int kV4Head = 512, kV4Rope = 64, kV4Nope = kV4Head - kV4Rope, kV4QBlock = 64;
constexpr int kV4DataBytes = kV4Nope + 2 * kV4Rope;   // 576
constexpr int kV4ScaleBytes = kV4Nope / kV4QBlock + 1;  // 8

__device__ __forceinline__ void v4_load16(const __nv_bfloat16* p, float (&e)[16]) {
  float a[8], b[8];
  unpack8<__nv_bfloat16>(reinterpret_cast<const uint4*>(p)[0], a);
  unpack8<__nv_bfloat16>(reinterpret_cast<const uint4*>(p)[1], b);
#pragma unroll
  for (int i = 0; i < 8; ++i) { e[i] = a[i]; e[8 + i] = b[i]; }
}
__device__ __forceinline__ void v4_store16(__nv_bfloat16* p, const float (&e)[16]) {
  float a[8], b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { a[i] = e[i]; b[i] = e[8 + i]; }
  reinterpret_cast<uint4*>(p)[0] = pack8<__nv_bfloat16>(a);
  reinterpret_cast<uint4*>(p)[1] = pack8<__nv_bfloat16>(b);
}

__global__ void __launch_bounds__(256)
v4_qnorm_rope_kv_insert_kernel(const __nv_bfloat16* __restrict__ q_in, int64_t q_stride_t, int64_t q_stride_h,
                               const __nv_bfloat16* __restrict__ kv, int64_t kv_stride,
                               __nv_bfloat16* __restrict__ q_out, uint8_t* __restrict__ cache, int64_t block_stride,
                               const int64_t* __restrict__ slot_mapping, const int64_t* __restrict__ positions,
                               const float* __restrict__ cos_sin, int tokens, int insert_tokens, int hq, int hq_pad,
                               int block_size, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (int64_t)tokens * (hq_pad + 1)) return;
  const int t = (int)(w / (hq_pad + 1)), slot = (int)(w % (hq_pad + 1));
  const int d0 = lane * 16;
  const bool rope_lane = d0 >= kV4Nope;

  if (slot >= hq && slot < hq_pad) {   // head padding
    uint4* o = reinterpret_cast<uint4*>(q_out + ((int64_t)t * hq_pad + slot) * kV4Head + d0);
    o[0] = make_uint4(0, 0, 0, 0);
    o[1] = make_uint4(0, 0, 0, 0);
    return;
  }
  const bool is_kv = slot == hq_pad;
  int64_t cache_slot = -1;
  if (is_kv) {
    if (t >= insert_tokens) return;
    cache_slot = slot_mapping[t];
    if (cache_slot < 0) return;
  }
  float e[16];
  v4_load16(is_kv ? kv + (int64_t)t * kv_stride + d0 : q_in + (int64_t)t * q_stride_t + (int64_t)slot * q_stride_h + d0, e);

  if (!is_kv) {   // weightless RMSNorm over the whole head
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) ss += e[i] * e[i];
    const float inv = rsqrtf(warp_sum(ss) / (float)kV4Head + eps);
#pragma unroll
    for (int i = 0; i < 16; ++i) e[i] *= inv;
  }
  if (rope_lane) {   // interleaved pairs (2i, 2i+1); table row = cos[32] | sin[32]
    const float* row = cos_sin + positions[t] * kV4Rope;
    const int p0 = (d0 - kV4Nope) >> 1;   // first pair of this lane
    const float4 c0 = reinterpret_cast<const float4*>(row + p0)[0], c1 = reinterpret_cast<const float4*>(row + p0)[1];
    const float4 s0 = reinterpret_cast<const float4*>(row + 32 + p0)[0], s1 = reinterpret_cast<const float4*>(row + 32 + p0)[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float x = e[2 * i], y = e[2 * i + 1];
      e[2 * i] = x * c[i] - y * s[i];
      e[2 * i + 1] = y * c[i] + x * s[i];
    }
  }
  if (!is_kv) {
    v4_store16(q_out + ((int64_t)t * hq_pad + slot) * kV4Head + d0, e);
    return;
  }
  // ---- KV record
  const int64_t blk = cache_slot / block_size, pos = cache_slot % block_size;
  uint8_t* base = cache + blk * block_stride;
  uint8_t* data = base + pos * kV4DataBytes;
  uint8_t* scales = base + (int64_t)block_size * kV4DataBytes + pos * kV4ScaleBytes;
#pragma unroll
  for (int i = 0; i < 16; ++i) e[i] = __bfloat162float(__float2bfloat16_rn(e[i]));   // the cache sees bf16 values
  if (rope_lane) {
    v4_store16(reinterpret_cast<__nv_bfloat16*>(data + kV4Nope) + (d0 - kV4Nope), e);
    return;
  }
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(e[i]));
  m = fmaxf(m, __shfl_xor_sync(0x0fffffffu, m, 1));      // 4 lanes = one 64-wide block (nope lanes 0..27 only)
  m = fmaxf(m, __shfl_xor_sync(0x0fffffffu, m, 2));
  m = fmaxf(m, 1e-4f);
  const float ex = ceilf(log2f(m / 448.f));
  const float inv = exp2f(-ex);
  uint32_t pk[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    pk[j] = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float v = fminf(fmaxf(e[4 * j + i] * inv, -448.f), 448.f);
      pk[j] |= (uint32_t)float_to_fp8_e4m3(v) << (8 * i);
    }
  }
  *reinterpret_cast<uint4*>(data + d0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  if ((lane & 3) == 0) scales[lane >> 2] = (uint8_t)fminf(fmaxf(ex + 127.f, 0.f), 255.f);
  if (lane == 0) scales[kV4Nope / kV4QBlock] = 0;
}

__global__ void __launch_bounds__(256)
v4_gather_dequant_kernel(__nv_bfloat16* __restrict__ dst, const uint8_t* __restrict__ cache, int64_t block_stride,
                         const int64_t* __restrict__ slots, int n, int block_size) {
  const int lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int d0 = lane * 16;
  __nv_bfloat16* out = dst + i * kV4Head + d0;
  const int64_t s = slots[i];
  if (s < 0) {
    reinterpret_cast<uint4*>(out)[0] = make_uint4(0, 0, 0, 0);
    reinterpret_cast<uint4*>(out)[1] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int64_t blk = s / block_size, pos = s % block_size;
  const uint8_t* base = cache + blk * block_stride;
  const uint8_t* data = base + pos * kV4DataBytes;
  if (d0 >= kV4Nope) {
    const uint4* src = reinterpret_cast<const uint4*>(data + kV4Nope + (d0 - kV4Nope) * 2);
    reinterpret_cast<uint4*>(out)[0] = src[0];
    reinterpret_cast<uint4*>(out)[1] = src[1];
    return;
  }
  const uint8_t sc = base[(int64_t)block_size * kV4DataBytes + pos * kV4ScaleBytes + (lane >> 2)];
  const float scale = exp2f((float)sc - 127.f);
  const uint4 raw = *reinterpret_cast<const uint4*>(data + d0);
  const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
  float e[16];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int k = 0; k < 4; ++k) e[4 * j + k] = fp8_e4m3_to_float((uint8_t)(wds[j] >> (8 * k))) * scale;
  v4_store16(out, e);
}

// Attention output -> o_proj input: the rope dims of every head are rotated BACK (inverse of the interleaved
// RoPE) and the heads are regrouped [T, G * hpg, 512] -> [G, T, hpg * 512] for the grouped output projection.
template <typename T>
__global__ void __launch_bounds__(256)
v4_inv_rope_kernel(T* __restrict__ out, const T* __restrict__ o, int64_t o_stride_t, int64_t o_stride_h,
                   const int64_t* __restrict__ positions, const float* __restrict__ cos_sin, int tokens, int heads,
                   int hpg) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (int64_t)tokens * heads) return;
  const int t = (int)(w / heads), h = (int)(w % heads);
  const int d0 = lane * 16;
  const T* src = o + (int64_t)t * o_stride_t + (int64_t)h * o_stride_h + d0;
  uint4 a = reinterpret_cast<const uint4*>(src)[0], b = reinterpret_cast<const uint4*>(src)[1];
  if (d0 >= kV4Nope) {
    float e[16], x[8], y[8];
    unpack8<T>(a, x);
    unpack8<T>(b, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) { e[i] = x[i]; e[8 + i] = y[i]; }
    const float* row = cos_sin + positions[t] * kV4Rope;
    const int p0 = (d0 - kV4Nope) >> 1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float c = row[p0 + i], s = row[32 + p0 + i];
      const float u = e[2 * i], v = e[2 * i + 1];
      e[2 * i] = u * c + v * s;
      e[2 * i + 1] = v * c - u * s;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { x[i] = e[i]; y[i] = e[8 + i]; }
    a = pack8<T>(x);
    b = pack8<T>(y);
  }
  const int g = h / hpg, hi = h % hpg;
  T* dst = out + ((int64_t)g * tokens + t) * ((int64_t)hpg * kV4Head) + (int64_t)hi * kV4Head + d0;
  reinterpret_cast<uint4*>(dst)[0] = a;
  reinterpret_cast<uint4*>(dst)[1] = b;
}

// Indexer query: interleaved RoPE on the last `rot` dims of every 128-wide head, symmetric int8 quantisation with
// one scale per (token, head) (round half away from zero), and the scale folded into the head weight:
// w_out = w * q_scale * softmax_scale * head_scale, so the logits kernel needs no per-head dequantisation.
template <typename T>
__global__ void __launch_bounds__(256)
v4_indexer_q_kernel(int8_t* __restrict__ q8, float* __restrict__ w_out, const T* __restrict__ q, int64_t q_stride_t,
                    int64_t q_stride_h, const T* __restrict__ weights, int64_t w_stride,
                    const int64_t* __restrict__ positions, const float* __restrict__ cos_sin, int tokens, int heads,
                    int rot, float softmax_scale, float head_scale) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (int64_t)tokens * heads) return;
  const int t = (int)(w / heads), h = (int)(w % heads);
  const int d0 = lane * 4, nope = 128 - rot;
  const uint2 raw = *reinterpret_cast<const uint2*>(q + (int64_t)t * q_stride_t + (int64_t)h * q_stride_h + d0);
  const T* e = reinterpret_cast<const T*>(&raw);
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = to_f(e[i]);
  if (d0 >= nope) {
    const float* row = cos_sin + positions[t] * rot;
    const int half = rot >> 1, p0 = (d0 - nope) >> 1;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float c = row[p0 + i], s = row[half + p0 + i];
      const float x = v[2 * i], y = v[2 * i + 1];
      v[2 * i] = __bfloat162float(__float2bfloat16_rn(x * c - y * s));       // the unfused path materialises bf16
      v[2 * i + 1] = __bfloat162float(__float2bfloat16_rn(y * c + x * s));
    }
  }
  float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  m = warp_max(m);
  const float scale = m > 0.f ? m / 127.f : 1.f;
  uint32_t pk = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float r = v[i] / scale;
    float qv = r >= 0.f ? floorf(r + 0.5f) : ceilf(r - 0.5f);
    qv = fminf(fmaxf(qv, -127.f), 127.f);
    pk |= (uint32_t)(uint8_t)(int8_t)(int)qv << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(q8 + ((int64_t)t * heads + h) * 128 + d0) = pk;
  if (lane == 0)
    w_out[(int64_t)t * heads + h] = to_f(weights[(int64_t)t * w_stride + h]) * scale * softmax_scale * head_scale;
}

void v4_inv_rope(void* out, const void* o, int64_t o_stride_t, int64_t o_stride_h, const int64_t* positions,
                 const float* cos_sin, int tokens, int heads, int hpg, int dtype, cudaStream_t stream) {
  const int64_t warps = (int64_t)tokens * heads;
  if (warps <= 0) return;
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (dtype == 0)
    v4_inv_rope_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)o, o_stride_t,
                                                                  o_stride_h, positions, cos_sin, tokens, heads, hpg);
  else
    v4_inv_rope_kernel<__half><<<blocks, 256, 0, stream>>>((__half*)out, (const __half*)o, o_stride_t, o_stride_h,
                                                           positions, cos_sin, tokens, heads, hpg);
}

void v4_indexer_q(void* q8, float* w_out, const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* weights,
                  int64_t w_stride, const int64_t* positions, const float* cos_sin, int tokens, int heads, int rot,
                  float softmax_scale, float head_scale, int dtype, cudaStream_t stream) {
  const int64_t warps = (int64_t)tokens * heads;
  if (warps <= 0) return;
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (dtype == 0)
    v4_indexer_q_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        (int8_t*)q8, w_out, (const __nv_bfloat16*)q, q_stride_t, q_stride_h, (const __nv_bfloat16*)weights, w_stride,
        positions, cos_sin, tokens, heads, rot, softmax_scale, head_scale);
  else
    v4_indexer_q_kernel<__half><<<blocks, 256, 0, stream>>>((int8_t*)q8, w_out, (const __half*)q, q_stride_t, q_stride_h,
                                                            (const __half*)weights, w_stride, positions, cos_sin, tokens,
                                                            heads, rot, softmax_scale, head_scale);
}

void v4_qnorm_rope_kv_insert(const void* q_in, int64_t q_stride_t, int64_t q_stride_h, const void* kv, int64_t kv_stride,
                             void* q_out, void* cache, int64_t block_stride, const int64_t* slot_mapping,
                             const int64_t* positions, const float* cos_sin, int tokens, int insert_tokens, int hq,
                             int hq_pad, int block_size, float eps, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int64_t warps = (int64_t)tokens * (hq_pad + 1);
  v4_qnorm_rope_kv_insert_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(q_in), q_stride_t, q_stride_h, static_cast<const __nv_bfloat16*>(kv), kv_stride,
      static_cast<__nv_bfloat16*>(q_out), static_cast<uint8_t*>(cache), block_stride, slot_mapping, positions, cos_sin,
      tokens, insert_tokens, hq, hq_pad, block_size, eps);
}

void v4_gather_dequant(void* dst, const void* cache, int64_t block_stride, const int64_t* slots, int n, int block_size,
                       cudaStream_t stream) {
  if (n <= 0) return;
  v4_gather_dequant_kernel<<<(n + 7) / 8, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(dst),
                                                            static_cast<const uint8_t*>(cache), block_stride, slots, n,
                                                            block_size);
}

}  // namespace b200
