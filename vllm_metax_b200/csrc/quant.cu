// Activation quantisation kernels and attention-state merge.
//   per_token_group_quant   1 x group (64/128) dynamic fp8 e4m3 or int8, f32 scales (optionally
//                           rounded up to a power of two = ue8m0 semantics), row- or column-major scales
//   scaled_fp8_quant        static per-tensor | dynamic per-tensor | dynamic per-token
//   scaled_int8_quant       static / dynamic per-token, symmetric or with zero point (azp)
//   merge_attn_states       LSE-weighted merge of two partial attention results
// Parity: csrc/quantization/w8a8/fp8/per_token_group_quant.cu:100-431, w8a8/fp8/common.cu:13-138,
// w8a8/int8/scaled_quant.cu:100-212, attention/merge_attn_states.cu:19-130 of the reference.
#include "common.cuh"

namespace b200 {

// One warp per (token, group); lanes hold group/32 consecutive elements each.
template <typename T>
__global__ void per_token_group_quant_kernel(uint8_t* __restrict__ q, float* __restrict__ scales,
                                             const T* __restrict__ x, int64_t rows, int K, int group, int int8,
                                             int ue8m0, int col_major_scales, float eps) {
  const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int ngroups = K / group;
  if (gw >= rows * ngroups) return;
  const int64_t row = gw / ngroups;
  const int g = (int)(gw % ngroups);
  const T* src = x + row * K + (int64_t)g * group;
  const int per = group / 32;   // 2, 4 or 8
  float v[8];
  float m = 0.f;
  for (int i = 0; i < per; ++i) {
    v[i] = to_f(src[lane * per + i]);
    m = fmaxf(m, fabsf(v[i]));
  }
  m = fmaxf(warp_max(m), eps);
  float s = m / (int8 ? 127.f : 448.f);
  if (ue8m0) s = ue8m0_ceil(s);
  if (lane == 0) scales[col_major_scales ? (int64_t)g * rows + row : row * ngroups + g] = s;
  uint8_t* dst = q + row * K + (int64_t)g * group;
  const float inv = 1.f / s;
  for (int i = 0; i < per; ++i) {
    if (int8) {
      int qi = __float2int_rn(v[i] * inv);
      dst[lane * per + i] = (uint8_t)(int8_t)max(-128, min(127, qi));
    } else {
      dst[lane * per + i] = float_to_fp8_e4m3(v[i] * inv);
    }
  }
}

// mode 0: static scale (scale[0]); 1: dynamic per-token (writes scale[row]); per-tensor dynamic is done by the
// host as amax (torch) + mode 0.
template <typename T>
__global__ void scaled_fp8_quant_kernel(uint8_t* __restrict__ q, float* __restrict__ scale, const T* __restrict__ x,
                                        int K, int mode, float scale_ub) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const T* src = x + row * K;
  float s;
  if (mode == 0) {
    s = scale[0];
  } else {
    float m = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) m = fmaxf(m, fabsf(to_f(src[i])));
    m = block_max(m, red);
    if (scale_ub > 0.f) m = fminf(m, scale_ub);
    s = fmaxf(m / 448.f, 1.f / (448.f * 512.f));
    if (threadIdx.x == 0) scale[row] = s;
  }
  const float inv = 1.f / s;
  for (int i = threadIdx.x; i < K; i += blockDim.x) q[row * K + i] = float_to_fp8_e4m3(to_f(src[i]) * inv);
}

// mode 0: static symmetric; 1: static with azp; 2: dynamic symmetric; 3: dynamic with azp.
template <typename T>
__global__ void scaled_int8_quant_kernel(int8_t* __restrict__ q, float* __restrict__ scale, int* __restrict__ azp,
                                         const T* __restrict__ x, int K, int mode) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const T* src = x + row * K;
  float s, zp = 0.f;
  if (mode == 0) {
    s = scale[0];
  } else if (mode == 1) {
    s = scale[0];
    zp = (float)azp[0];
  } else if (mode == 2) {
    float m = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) m = fmaxf(m, fabsf(to_f(src[i])));
    m = block_max(m, red);
    s = fmaxf(m, 1e-10f) / 127.f;
    if (threadIdx.x == 0) scale[row] = s;
  } else {
    float mx = -INFINITY, mn = INFINITY;
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
      const float v = to_f(src[i]);
      mx = fmaxf(mx, v);
      mn = fminf(mn, v);
    }
    mx = block_max(mx, red);
    mn = -block_max(-mn, red);
    s = fmaxf((mx - mn) / 255.f, 1e-10f);
    zp = nearbyintf(-128.f - mn / s);
    if (threadIdx.x == 0) { scale[row] = s; azp[row] = (int)zp; }
  }
  const float inv = 1.f / s;
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    int qi = __float2int_rn(to_f(src[i]) * inv) + (int)zp;
    q[row * K + i] = (int8_t)max(-128, min(127, qi));
  }
}

// out/lse = merge of (prefix_out, prefix_lse) and (suffix_out, suffix_lse); *_out [T,H,D], *_lse [H,T].
template <typename T>
__global__ void merge_attn_states_kernel(T* __restrict__ out, float* __restrict__ out_lse, const T* __restrict__ p_out,
                                         const float* __restrict__ p_lse, const T* __restrict__ s_out,
                                         const float* __restrict__ s_lse, int tokens, int heads, int D) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one thread per 8 elements
  const int per_row = D / 8;
  if (idx >= (int64_t)tokens * heads * per_row) return;
  const int v = (int)(idx % per_row);
  const int64_t th = idx / per_row;
  const int h = (int)(th % heads);
  const int64_t t = th / heads;
  float pl = p_lse[(int64_t)h * tokens + t], sl = s_lse[(int64_t)h * tokens + t];
  if (isinf(pl) && pl > 0) pl = -INFINITY;
  if (isinf(sl) && sl > 0) sl = -INFINITY;
  const float mx = fmaxf(pl, sl);
  const float ms = isinf(mx) ? 0.f : mx;
  const float pw = __expf(pl - ms), sw = __expf(sl - ms);
  const float tot = pw + sw;
  const float inv = tot > 0.f ? 1.f / tot : 0.f;
  float a[8], b[8];
  unpack8<T>(reinterpret_cast<const uint4*>(p_out + th * D)[v], a);
  unpack8<T>(reinterpret_cast<const uint4*>(s_out + th * D)[v], b);
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = (a[i] * pw + b[i] * sw) * inv;
  reinterpret_cast<uint4*>(out + th * D)[v] = pack8<T>(a);
  if (out_lse && v == 0) out_lse[(int64_t)h * tokens + t] = tot > 0.f ? logf(tot) + ms : -INFINITY;
}

#define LAUNCH16(dtype, K, ...) \
  if (dtype == 0) { K<__nv_bfloat16> __VA_ARGS__; } else { K<__half> __VA_ARGS__; }

void per_token_group_quant(void* q, float* scales, const void* x, int64_t rows, int K, int group, int int8, int ue8m0,
                           int col_major, float eps, int dtype, cudaStream_t stream) {
  if (rows <= 0) return;
  const int64_t warps = rows * (K / group);
  const int th = 256;
  const int blocks = (int)((warps * 32 + th - 1) / th);
  if (dtype == 0)
    per_token_group_quant_kernel<__nv_bfloat16><<<blocks, th, 0, stream>>>((uint8_t*)q, scales, (const __nv_bfloat16*)x, rows, K, group, int8, ue8m0, col_major, eps);
  else
    per_token_group_quant_kernel<__half><<<blocks, th, 0, stream>>>((uint8_t*)q, scales, (const __half*)x, rows, K, group, int8, ue8m0, col_major, eps);
}

void scaled_fp8_quant(void* q, float* scale, const void* x, int64_t rows, int K, int mode, float scale_ub, int dtype,
                      cudaStream_t stream) {
  if (rows <= 0) return;
  if (dtype == 0)
    scaled_fp8_quant_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, stream>>>((uint8_t*)q, scale, (const __nv_bfloat16*)x, K, mode, scale_ub);
  else
    scaled_fp8_quant_kernel<__half><<<(unsigned)rows, 256, 0, stream>>>((uint8_t*)q, scale, (const __half*)x, K, mode, scale_ub);
}

void scaled_int8_quant(void* q, float* scale, int* azp, const void* x, int64_t rows, int K, int mode, int dtype,
                       cudaStream_t stream) {
  if (rows <= 0) return;
  if (dtype == 0)
    scaled_int8_quant_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, stream>>>((int8_t*)q, scale, azp, (const __nv_bfloat16*)x, K, mode);
  else
    scaled_int8_quant_kernel<__half><<<(unsigned)rows, 256, 0, stream>>>((int8_t*)q, scale, azp, (const __half*)x, K, mode);
}

void merge_attn_states(void* out, float* out_lse, const void* p_out, const float* p_lse, const void* s_out,
                       const float* s_lse, int tokens, int heads, int D, int dtype, cudaStream_t stream) {
  const int64_t n = (int64_t)tokens * heads * (D / 8);
  if (n <= 0) return;
  const int th = 256;
  const int blocks = (int)((n + th - 1) / th);
  if (dtype == 0)
    merge_attn_states_kernel<__nv_bfloat16><<<blocks, th, 0, stream>>>((__nv_bfloat16*)out, out_lse, (const __nv_bfloat16*)p_out, p_lse, (const __nv_bfloat16*)s_out, s_lse, tokens, heads, D);
  else
    merge_attn_states_kernel<__half><<<blocks, th, 0, stream>>>((__half*)out, out_lse, (const __half*)p_out, p_lse, (const __half*)s_out, s_lse, tokens, heads, D);
}

}  // namespace b200
