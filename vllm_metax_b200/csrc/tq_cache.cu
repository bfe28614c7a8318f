// TurboQuant KV cache (head_dim 128): 3-4 bit keys and values in one combined slot per (token, kv head).
//
//   keys    "mse" formats: k = |k| * u.  u is rotated by the orthonormal 128-point Hadamard transform, every rotated
//           coordinate (x sqrt(128), ~N(0,1)) is replaced by the nearest of 2^b Lloyd-Max levels, and |k| is stored as
//           fp16 - divided by the norm of the level vector when norm correction is on, so that the reconstructed key
//           has exactly the original length.  Scores need no inverse rotation: q.k = (Hq).(Hk), the query is rotated
//           once per step.  "fp8" format: e4m3 bytes, no rotation.
//   values  uniform b-bit codes with an fp16 scale and minimum per (token, head).
//   slot    [ key codes | value codes | key norm f16 | value scale f16 | value min f16 | pad to 16 bytes ]
//           4-bit codes: two per byte, lane L of a warp owns dims 4L..4L+3 = bytes 2L, 2L+1.
//           3-bit codes: low two bits of the 4 dims in byte L of a 32-byte plane, high bits in nibble L of a 16-byte plane.
//   cache   uint8 [blocks, block_size, kv_heads, slot_bytes]
//
//   tq_store     one warp per (token, kv head): butterflies in registers + 5 shuffle stages, codes, norms.
//   tq_decode    one CTA per (sequence, kv head, split): 4 warps walk 32-token chunks; slots are staged in shared
//                memory, lane = token for the scores (level lookups against the rotated queries of the whole GQA
//                group), lane = 4 dims for the value accumulation; online softmax per warp, merged across warps and
//                across splits (second kernel).
//   tq_dequant   slots -> 16-bit K and V rows (continuation prefill reads its cached prefix this way).
// Replaces the Triton store / decode kernels behind the reference's TURBOQUANT backend
// (vllm_metax/v1/attention/backends/turboquant_attn.py:95-942).
#include "common.cuh"
#include "ops.h"

namespace b200 {

__constant__ float kTqLevels4[16] = {-2.7326f, -2.0690f, -1.6181f, -1.2562f, -0.9424f, -0.6568f, -0.3881f, -0.1284f,
                                     0.1284f,  0.3881f,  0.6568f,  0.9424f,  1.2562f,  1.6181f,  2.0690f,  2.7326f};
__constant__ float kTqLevels3[8] = {-2.1520f, -1.3439f, -0.7560f, -0.2451f, 0.2451f, 0.7560f, 1.3439f, 2.1520f};

struct TqFormat {
  int kbits, vbits, nc;      // kbits 3, 4 or 8 (fp8)
  int k_bytes, v_bytes;      // code bytes
  int v_off, meta_off, slot_bytes;
};

__host__ __device__ inline TqFormat tq_format(int kbits, int vbits, int nc) {
  TqFormat f;
  f.kbits = kbits; f.vbits = vbits; f.nc = nc;
  f.k_bytes = kbits == 8 ? 128 : kbits * 16;
  f.v_bytes = vbits * 16;
  f.v_off = f.k_bytes;
  f.meta_off = f.k_bytes + f.v_bytes;
  f.slot_bytes = (f.meta_off + 6 + 15) / 16 * 16;
  return f;
}

// 128-point Walsh-Hadamard transform over a warp (4 values per lane), orthonormal.
__device__ __forceinline__ void wht128(float (&v)[4], int lane) {
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? o - v[i] : v[i] + o;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] *= 0.08838834764831845f;   // 1 / sqrt(128)
}

__device__ __forceinline__ int tq_nearest(float z, int bits) {
  const float* lv = bits == 4 ? kTqLevels4 : kTqLevels3;
  const int n = 1 << bits;
  int code = 0;
  for (int i = 1; i < n; ++i) code += z > 0.5f * (lv[i - 1] + lv[i]) ? 1 : 0;
  return code;
}

// codes of this lane's 4 dims -> slot (collective over the warp for the 3-bit high plane)
__device__ __forceinline__ void tq_put_codes(uint8_t* base, const int (&c)[4], int bits, int lane) {
  if (bits == 4) {
    *reinterpret_cast<uint16_t*>(base + 2 * lane) =
        (uint16_t)(c[0] | (c[1] << 4) | (c[2] << 8) | (c[3] << 12));
  } else {
    base[lane] = (uint8_t)((c[0] & 3) | ((c[1] & 3) << 2) | ((c[2] & 3) << 4) | ((c[3] & 3) << 6));
    const int hi = (c[0] >> 2) | ((c[1] >> 2) << 1) | ((c[2] >> 2) << 2) | ((c[3] >> 2) << 3);
    const int other = __shfl_xor_sync(0xffffffffu, hi, 1);
    if ((lane & 1) == 0) base[32 + (lane >> 1)] = (uint8_t)(hi | (other << 4));
  }
}
__device__ __forceinline__ void tq_get_codes(const uint8_t* base, int (&c)[4], int bits, int lane) {
  if (bits == 4) {
    const uint32_t w = *reinterpret_cast<const uint16_t*>(base + 2 * lane);
    c[0] = w & 15; c[1] = (w >> 4) & 15; c[2] = (w >> 8) & 15; c[3] = (w >> 12) & 15;
  } else {
    const uint32_t lo = base[lane];
    const uint32_t hi = (base[32 + (lane >> 1)] >> ((lane & 1) * 4)) & 15;
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = ((lo >> (2 * i)) & 3) | (((hi >> i) & 1) << 2);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
tq_store_kernel(uint8_t* __restrict__ cache, const T* __restrict__ k, const T* __restrict__ v, int64_t k_stride,
                int64_t v_stride, const int64_t* __restrict__ slot_mapping, int tokens, int heads, int64_t num_slots,
                TqFormat f) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (int64_t)tokens * heads) return;
  const int t = (int)(w / heads), h = (int)(w % heads);
  const int64_t slot = slot_mapping[t];
  if (slot < 0 || slot >= num_slots) return;
  uint8_t* dst = cache + (slot * heads + h) * f.slot_bytes;
  float kv[4], vv[4];
  {
    const uint2 rk = *reinterpret_cast<const uint2*>(k + (int64_t)t * k_stride + h * 128 + lane * 4);
    const uint2 rv = *reinterpret_cast<const uint2*>(v + (int64_t)t * v_stride + h * 128 + lane * 4);
    const T* ek = reinterpret_cast<const T*>(&rk);
    const T* ev = reinterpret_cast<const T*>(&rv);
#pragma unroll
    for (int i = 0; i < 4; ++i) { kv[i] = to_f(ek[i]); vv[i] = to_f(ev[i]); }
  }
  float stored_norm = 1.f;
  if (f.kbits == 8) {
    uint32_t pk = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) pk |= (uint32_t)float_to_fp8_e4m3(fminf(fmaxf(kv[i], -448.f), 448.f)) << (8 * i);
    *reinterpret_cast<uint32_t*>(dst + 4 * lane) = pk;
  } else {
    const float norm = sqrtf(warp_sum(kv[0] * kv[0] + kv[1] * kv[1] + kv[2] * kv[2] + kv[3] * kv[3]));
    const float inv = norm > 0.f ? 1.f / norm : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) kv[i] *= inv;
    wht128(kv, lane);
    const float* lv = f.kbits == 4 ? kTqLevels4 : kTqLevels3;
    int c[4];
    float cc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      c[i] = tq_nearest(kv[i] * 11.313708498984761f, f.kbits);     // x sqrt(128): unit-variance coordinates
      cc += lv[c[i]] * lv[c[i]];
    }
    tq_put_codes(dst, c, f.kbits, lane);
    const float lnorm = sqrtf(warp_sum(cc) * (1.f / 128.f));          // length of the reconstructed unit vector
    stored_norm = f.nc && lnorm > 0.f ? norm / lnorm : norm;
  }
  float mn = fminf(fminf(vv[0], vv[1]), fminf(vv[2], vv[3])), mx = fmaxf(fmaxf(vv[0], vv[1]), fmaxf(vv[2], vv[3]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const int vmax = (1 << f.vbits) - 1;
  // the stored fp16 scale and minimum are what the reader multiplies with: quantise against the rounded values
  const float scale = __half2float(__float2half_rn(fmaxf((mx - mn) / (float)vmax, 1e-8f)));
  const float zero = __half2float(__float2half_rn(mn));
  int c[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = min(vmax, max(0, __float2int_rn((vv[i] - zero) / scale)));
  tq_put_codes(dst + f.v_off, c, f.vbits, lane);
  if (lane == 0) {
    __half* meta = reinterpret_cast<__half*>(dst + f.meta_off);
    meta[0] = __float2half_rn(stored_norm);
    meta[1] = __float2half_rn(scale);
    meta[2] = __float2half_rn(zero);
  }
}

// slots -> K and V rows.  One warp per (row, kv head); slots < 0 give zeros.
template <typename T>
__global__ void __launch_bounds__(256)
tq_dequant_kernel(T* __restrict__ k_out, T* __restrict__ v_out, const uint8_t* __restrict__ cache,
                  const int64_t* __restrict__ slots, int rows, int heads, TqFormat f) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (int64_t)rows * heads) return;
  const int r = (int)(w / heads), h = (int)(w % heads);
  const int64_t slot = slots[r];
  float kv[4] = {0.f, 0.f, 0.f, 0.f}, vv[4] = {0.f, 0.f, 0.f, 0.f};
  if (slot >= 0) {
    const uint8_t* src = cache + (slot * heads + h) * f.slot_bytes;
    const __half* meta = reinterpret_cast<const __half*>(src + f.meta_off);
    if (f.kbits == 8) {
      const uint32_t pk = *reinterpret_cast<const uint32_t*>(src + 4 * lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) kv[i] = fp8_e4m3_to_float((uint8_t)(pk >> (8 * i)));
    } else {
      const float* lv = f.kbits == 4 ? kTqLevels4 : kTqLevels3;
      int c[4];
      tq_get_codes(src, c, f.kbits, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) kv[i] = lv[c[i]] * 0.08838834764831845f;
      wht128(kv, lane);                                               // the transform is its own inverse
      const float n = __half2float(meta[0]);
#pragma unroll
      for (int i = 0; i < 4; ++i) kv[i] *= n;
    }
    int c[4];
    tq_get_codes(src + f.v_off, c, f.vbits, lane);
    const float s = __half2float(meta[1]), z = __half2float(meta[2]);
#pragma unroll
    for (int i = 0; i < 4; ++i) vv[i] = c[i] * s + z;
  }
  T ok[4], ov[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { ok[i] = from_f<T>(kv[i]); ov[i] = from_f<T>(vv[i]); }
  *reinterpret_cast<uint2*>(k_out + ((int64_t)r * heads + h) * 128 + lane * 4) = *reinterpret_cast<const uint2*>(ok);
  *reinterpret_cast<uint2*>(v_out + ((int64_t)r * heads + h) * 128 + lane * 4) = *reinterpret_cast<const uint2*>(ov);
}

// ------------------------------------------------------------------------------------------------ decode
constexpr int kTqWarps = 4, kTqMaxGroup = 8;

template <typename T, int G>
__global__ void __launch_bounds__(kTqWarps * 32)
tq_decode_kernel(T* __restrict__ out, float* __restrict__ part_out, float* __restrict__ part_lse,
                 const T* __restrict__ q, int64_t q_stride, const uint8_t* __restrict__ cache,
                 const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_lens, int hq, int hkv,
                 int block_size, int64_t num_blocks, int splits, float scale, TqFormat f) {
  extern __shared__ __align__(16) uint8_t tq_smem[];
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_rot = reinterpret_cast<float*>(tq_smem);                       // [G][128], pre-scaled
  float* lv_s = q_rot + G * 128;                                           // [16] key levels
  float* merge = lv_s + 16;                                                // [warps][G][128 + 2]
  uint8_t* stage = reinterpret_cast<uint8_t*>(merge + kTqWarps * G * 130) + (size_t)warp * 32 * f.slot_bytes;

  // ---- queries of the group: rotated (mse keys) and scaled once
  for (int g = warp; g < G; g += kTqWarps) {
    const int head = kvh * G + g;
    float v[4];
    const uint2 raw = *reinterpret_cast<const uint2*>(q + (int64_t)b * q_stride + (int64_t)head * 128 + lane * 4);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = to_f(e[i]);
    if (f.kbits != 8) {
      wht128(v, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] *= 0.08838834764831845f;          // levels are in sqrt(128) units
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) q_rot[g * 128 + lane * 4 + i] = v[i] * scale;
  }
  if (threadIdx.x < 16) lv_s[threadIdx.x] = f.kbits == 3 ? kTqLevels3[threadIdx.x & 7] : kTqLevels4[threadIdx.x];
  __syncthreads();

  const int L = seq_lens[b];
  const int per = ((L + splits - 1) / splits + 31) / 32 * 32;
  const int t_begin = split * per, t_end = min(L, t_begin + per);
  float m[G], l[G], acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[g][i] = 0.f;
  }
  const int vec_per_slot = f.slot_bytes >> 4;
  for (int t0 = t_begin + warp * 32; t0 < t_end; t0 += kTqWarps * 32) {
    const int t = t0 + lane;
    const bool live = t < t_end;
    // stage this lane's token
    uint4* mine = reinterpret_cast<uint4*>(stage + (size_t)lane * f.slot_bytes);
    if (live) {
      int blk = block_table[(int64_t)b * max_blocks + t / block_size];
      blk = blk >= 0 && blk < num_blocks ? blk : 0;
      const uint4* src = reinterpret_cast<const uint4*>(
          cache + (((int64_t)blk * block_size + t % block_size) * hkv + kvh) * f.slot_bytes);
      for (int i = 0; i < vec_per_slot; ++i) mine[i] = src[i];
    }
    __syncwarp();
    // ---- scores: lane = token
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    if (live) {
      const uint8_t* row = stage + (size_t)lane * f.slot_bytes;
      if (f.kbits == 8) {
        for (int d = 0; d < 128; d += 4) {
          const uint32_t pk = *reinterpret_cast<const uint32_t*>(row + d);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float kd = fp8_e4m3_to_float((uint8_t)(pk >> (8 * i)));
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = fmaf(kd, q_rot[g * 128 + d + i], s[g]);
          }
        }
      } else if (f.kbits == 4) {
        for (int d = 0; d < 128; d += 8) {
          const uint32_t pk = *reinterpret_cast<const uint32_t*>(row + (d >> 1));
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float kd = lv_s[(pk >> (4 * i)) & 15];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = fmaf(kd, q_rot[g * 128 + d + i], s[g]);
          }
        }
      } else {
        for (int d = 0; d < 128; d += 8) {            // 8 dims = 2 bytes of the low plane + 1 byte of the high plane
          const uint32_t lo = *reinterpret_cast<const uint16_t*>(row + (d >> 2));
          const uint32_t hi = row[32 + (d >> 3)];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float kd = lv_s[((lo >> (2 * i)) & 3) | (((hi >> i) & 1) << 2)];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = fmaf(kd, q_rot[g * 128 + d + i], s[g]);
          }
        }
      }
      const float n = f.kbits == 8 ? 1.f : __half2float(*reinterpret_cast<const __half*>(row + f.meta_off));
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] *= n;
    }
    // ---- online softmax (per warp) and value accumulation: lane = 4 dims
    float p[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float sv = live ? s[g] : -INFINITY;
      const float mx = fmaxf(m[g], warp_max(sv));
      const float corr = m[g] == -INFINITY ? 0.f : __expf(m[g] - mx);
      p[g] = live ? __expf(sv - mx) : 0.f;
      l[g] = l[g] * corr + warp_sum(p[g]);
      m[g] = mx;
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[g][i] *= corr;
    }
    const int n_live = min(32, t_end - t0);
    for (int j = 0; j < n_live; ++j) {
      const uint8_t* row = stage + (size_t)j * f.slot_bytes;
      int c[4];
      tq_get_codes(row + f.v_off, c, f.vbits, lane);
      const __half* meta = reinterpret_cast<const __half*>(row + f.meta_off);
      const float vs = __half2float(meta[1]), vz = __half2float(meta[2]);
      float vv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) vv[i] = c[i] * vs + vz;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pj = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[g][i] = fmaf(pj, vv[i], acc[g][i]);
      }
    }
    __syncwarp();
  }
  // ---- merge the warps
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float* dstm = merge + ((size_t)warp * G + g) * 130;
#pragma unroll
    for (int i = 0; i < 4; ++i) dstm[lane * 4 + i] = acc[g][i];
    if (lane == 0) { dstm[128] = m[g]; dstm[129] = l[g]; }
  }
  __syncthreads();
  for (int g = warp; g < G; g += kTqWarps) {
    float mx = -INFINITY;
    for (int w2 = 0; w2 < kTqWarps; ++w2) mx = fmaxf(mx, merge[((size_t)w2 * G + g) * 130 + 128]);
    float lt = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int w2 = 0; w2 < kTqWarps; ++w2) {
      const float* src = merge + ((size_t)w2 * G + g) * 130;
      const float c = src[128] == -INFINITY ? 0.f : __expf(src[128] - mx);
      lt += src[129] * c;
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] += src[lane * 4 + i] * c;
    }
    const int head = kvh * G + g;
    if (splits == 1) {
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      T ov[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) ov[i] = from_f<T>(o[i] * inv);
      *reinterpret_cast<uint2*>(out + ((int64_t)b * hq + head) * 128 + lane * 4) = *reinterpret_cast<const uint2*>(ov);
    } else {
      float* po = part_out + (((int64_t)split * gridDim.x + b) * hq + head) * 128;
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) po[lane * 4 + i] = o[i] * inv;
      if (lane == 0) part_lse[((int64_t)split * gridDim.x + b) * hq + head] = lt > 0.f ? mx + __logf(lt) : -INFINITY;
    }
  }
}

template <typename T>
__global__ void tq_merge_kernel(T* __restrict__ out, const float* __restrict__ part_out, const float* __restrict__ part_lse,
                                int rows, int splits) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);    // (sequence, head)
  if (r >= rows) return;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_lse[(int64_t)s * rows + r]);
  float wsum = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < splits; ++s) {
    const float lse = part_lse[(int64_t)s * rows + r];
    const float w = lse == -INFINITY ? 0.f : __expf(lse - mx);
    wsum += w;
    const float4 v = *reinterpret_cast<const float4*>(part_out + ((int64_t)s * rows + r) * 128 + lane * 4);
    o[0] += w * v.x; o[1] += w * v.y; o[2] += w * v.z; o[3] += w * v.w;
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  T ov[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) ov[i] = from_f<T>(o[i] * inv);
  *reinterpret_cast<uint2*>(out + (int64_t)r * 128 + lane * 4) = *reinterpret_cast<const uint2*>(ov);
}

int tq_slot_bytes(int kbits, int vbits) { return tq_format(kbits, vbits, 0).slot_bytes; }

static bool tq_ok(int kbits, int vbits) { return (kbits == 3 || kbits == 4 || kbits == 8) && (vbits == 3 || vbits == 4); }

int tq_store(void* cache, const void* k, const void* v, int64_t k_stride, int64_t v_stride, const int64_t* slot_mapping,
             int tokens, int heads, int64_t num_slots, int kbits, int vbits, int nc, int dtype, cudaStream_t stream) {
  if (!tq_ok(kbits, vbits)) return 1;
  const int64_t warps = (int64_t)tokens * heads;
  if (warps <= 0) return 0;
  const TqFormat f = tq_format(kbits, vbits, nc);
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (dtype == 0)
    tq_store_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((uint8_t*)cache, (const __nv_bfloat16*)k,
                                                               (const __nv_bfloat16*)v, k_stride, v_stride, slot_mapping,
                                                               tokens, heads, num_slots, f);
  else
    tq_store_kernel<__half><<<blocks, 256, 0, stream>>>((uint8_t*)cache, (const __half*)k, (const __half*)v, k_stride,
                                                        v_stride, slot_mapping, tokens, heads, num_slots, f);
  return 0;
}

int tq_dequant(void* k_out, void* v_out, const void* cache, const int64_t* slots, int rows, int heads, int kbits, int vbits,
               int nc, int dtype, cudaStream_t stream) {
  if (!tq_ok(kbits, vbits)) return 1;
  const int64_t warps = (int64_t)rows * heads;
  if (warps <= 0) return 0;
  const TqFormat f = tq_format(kbits, vbits, nc);
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (dtype == 0)
    tq_dequant_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out,
                                                                 (const uint8_t*)cache, slots, rows, heads, f);
  else
    tq_dequant_kernel<__half><<<blocks, 256, 0, stream>>>((__half*)k_out, (__half*)v_out, (const uint8_t*)cache, slots,
                                                          rows, heads, f);
  return 0;
}

template <typename T, int G>
static void tq_decode_launch(void* out, float* part_out, float* part_lse, const void* q, int64_t q_stride,
                             const void* cache, const int* block_table, int max_blocks, const int* seq_lens, int batch,
                             int hq, int hkv, int block_size, int64_t num_blocks, int splits, float scale,
                             const TqFormat& f, cudaStream_t stream) {
  const size_t smem = (size_t)(G * 128 + 16 + kTqWarps * G * 130) * 4 + (size_t)kTqWarps * 32 * f.slot_bytes;
  auto kern = tq_decode_kernel<T, G>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  kern<<<dim3(batch, hkv, splits), kTqWarps * 32, smem, stream>>>(
      (T*)out, part_out, part_lse, (const T*)q, q_stride, (const uint8_t*)cache, block_table, max_blocks, seq_lens, hq, hkv,
      block_size, num_blocks, splits, scale, f);
  if (splits > 1) {
    const int rows = batch * hq;
    tq_merge_kernel<T><<<(rows + 7) / 8, 256, 0, stream>>>((T*)out, part_out, part_lse, rows, splits);
  }
}

// Returns 0, 1 (format), 2 (GQA group not in {1, 2, 4, 8}).
int tq_decode(void* out, float* part_out, float* part_lse, const void* q, int64_t q_stride, const void* cache,
              const int* block_table, int max_blocks, const int* seq_lens, int batch, int hq, int hkv, int block_size,
              int64_t num_blocks, int splits, float scale, int kbits, int vbits, int nc, int dtype, cudaStream_t stream) {
  if (!tq_ok(kbits, vbits)) return 1;
  if (batch <= 0) return 0;
  const TqFormat f = tq_format(kbits, vbits, nc);
  const int G = hq / hkv;
#define TQ_GO(T, GG) tq_decode_launch<T, GG>(out, part_out, part_lse, q, q_stride, cache, block_table, max_blocks, seq_lens, \
                                             batch, hq, hkv, block_size, num_blocks, splits, scale, f, stream)
#define TQ_G(T)                        \
  do {                                 \
    if (G == 1) TQ_GO(T, 1);           \
    else if (G == 2) TQ_GO(T, 2);      \
    else if (G == 4) TQ_GO(T, 4);      \
    else if (G == 8) TQ_GO(T, 8);      \
    else return 2;                     \
  } while (0)
  if (dtype == 0) TQ_G(__nv_bfloat16);
  else TQ_G(__half);
#undef TQ_G
#undef TQ_GO
  return 0;
}

}  // namespace b200
