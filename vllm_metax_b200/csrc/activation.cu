// Gated and plain activations, optionally fused with fp8 quantisation.
//   act_and_mul:  out[t, :d] = act(x[t, :d]) * x[t, d:]      (silu, gelu, gelu_tanh, fatrelu, relu2)
//   mul_and_silu, swigluoai (interleaved gate/up with clamp), swiglustep (clamped)
//   plain: gelu_new / gelu_fast / gelu_quick / silu / relu2
//   fused: act_and_mul + static fp8, act_and_mul + per-128 block fp8 (optionally ue8m0 scales)
// Parity: csrc/activation_kernels.cu:102-561, quantization/activation_kernels.cu:43,
// quantization/fused_kernels/fused_silu_mul_block_quant.cu:15 of the reference.
#include "common.cuh"

namespace b200 {

enum Act : int {
  kSilu = 0, kGelu = 1, kGeluTanh = 2, kFatRelu = 3, kRelu2 = 4, kMulSilu = 5, kSwigluOai = 6, kSwigluStep = 7,
  kGeluNew = 8, kGeluFast = 9, kGeluQuick = 10
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

__device__ __forceinline__ float unary_act(int act, float x, float p0) {
  switch (act) {
    case kSilu: return silu_f(x);
    case kGelu: return gelu_f(x);
    case kGeluTanh: return gelu_tanh_f(x);
    case kFatRelu: return x > p0 ? x : 0.f;
    case kRelu2: { float r = fmaxf(x, 0.f); return r * r; }
    case kGeluNew: return gelu_tanh_f(x);
    case kGeluFast: return 0.5f * x * (1.f + tanhf(x * 0.7978845608f * (1.f + 0.044715f * x * x)));
    case kGeluQuick: return x / (1.f + __expf(-1.702f * x));
    default: return x;
  }
}

// gate/up combination for one element pair
__device__ __forceinline__ float gated(int act, float g, float u, float p0, float p1) {
  switch (act) {
    case kMulSilu: return g * silu_f(u);
    case kSwigluOai: {  // p0 = alpha, p1 = limit
      g = fminf(g, p1);
      u = fminf(fmaxf(u, -p1), p1);
      return (u + 1.f) * g / (1.f + __expf(-p0 * g));
    }
    case kSwigluStep: {  // p1 = limit
      float s = fminf(silu_f(g), p1);
      u = fminf(fmaxf(u, -p1), p1);
      return s * u;
    }
    default: return unary_act(act, g, p0) * u;
  }
}

template <typename T>
__global__ void act_and_mul_kernel(T* __restrict__ out, const T* __restrict__ x, int d, int64_t x_stride,
                                   int64_t out_stride, int act, float p0, float p1) {
  const int64_t t = blockIdx.x;
  const T* row = x + t * x_stride;
  T* o = out + t * out_stride;
  if (act == kSwigluOai) {  // interleaved: gate = x[2i], up = x[2i+1]
    for (int i = threadIdx.x; i < d; i += blockDim.x)
      o[i] = from_f<T>(gated(act, to_f(row[2 * i]), to_f(row[2 * i + 1]), p0, p1));
    return;
  }
  const int nvec = ((d & 7) == 0 && (x_stride & 7) == 0 && (out_stride & 7) == 0) ? d >> 3 : 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float g[8], u[8];
    unpack8<T>(reinterpret_cast<const uint4*>(row)[v], g);
    unpack8<T>(reinterpret_cast<const uint4*>(row + d)[v], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = gated(act, g[i], u[i], p0, p1);
    reinterpret_cast<uint4*>(o)[v] = pack8<T>(g);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < d; i += blockDim.x)
    o[i] = from_f<T>(gated(act, to_f(row[i]), to_f(row[d + i]), p0, p1));
}

template <typename T>
__global__ void activation_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t n, int act, float p0) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = from_f<T>(unary_act(act, to_f(x[i]), p0));
}

// act_and_mul followed by fp8 quantisation.  group == 0: static scale (scale_in[0]);
// group > 0: one dynamic scale per `group` outputs, written to scale_out[t, d/group].
// The activation output is rounded to T before quantisation, as the unfused pipeline would.
template <typename T>
__global__ void act_and_mul_quant_kernel(uint8_t* __restrict__ out_q, float* __restrict__ scale_out,
                                         const float* __restrict__ scale_in, const T* __restrict__ x, int d, int act,
                                         float p0, float p1, int group, int ue8m0) {
  const int64_t t = blockIdx.x;
  const T* row = x + t * (int64_t)(2 * d);
  uint8_t* o = out_q + t * (int64_t)d;
  if (group == 0) {
    const float inv = 1.f / scale_in[0];
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float y = to_f(from_f<T>(gated(act, to_f(row[i]), to_f(row[d + i]), p0, p1)));
      o[i] = float_to_fp8_e4m3(y * inv);
    }
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int ngroups = d / group;
  for (int g = warp; g < ngroups; g += nw) {
    float y[8];  // group <= 256
    float m = 0.f;
    const int per = group / 32;
    for (int j = 0; j < per; ++j) {
      const int i = g * group + lane + 32 * j;
      y[j] = to_f(from_f<T>(gated(act, to_f(row[i]), to_f(row[d + i]), p0, p1)));
      m = fmaxf(m, fabsf(y[j]));
    }
    m = fmaxf(warp_max(m), 1e-10f);
    float s = m / 448.f;
    if (ue8m0) s = ue8m0_ceil(s);
    if (lane == 0) scale_out[t * ngroups + g] = s;
    for (int j = 0; j < per; ++j) o[g * group + lane + 32 * j] = float_to_fp8_e4m3(y[j] / s);
  }
}

void act_and_mul(void* out, const void* x, int tokens, int d, int64_t x_stride, int64_t out_stride, int act, float p0,
                 float p1, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  int th = d / 8;
  th = th < 64 ? 64 : (th > 1024 ? 1024 : (th + 31) / 32 * 32);
  if (dtype == 0)
    act_and_mul_kernel<__nv_bfloat16><<<tokens, th, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, d,
                                                                 x_stride, out_stride, act, p0, p1);
  else
    act_and_mul_kernel<__half><<<tokens, th, 0, stream>>>((__half*)out, (const __half*)x, d, x_stride, out_stride, act,
                                                          p0, p1);
}

void activation(void* out, const void* x, int64_t n, int act, float p0, int dtype, cudaStream_t stream) {
  if (n <= 0) return;
  const int th = 256;
  int64_t blocks = (n + th - 1) / th;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == 0)
    activation_kernel<__nv_bfloat16><<<(int)blocks, th, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, n, act, p0);
  else
    activation_kernel<__half><<<(int)blocks, th, 0, stream>>>((__half*)out, (const __half*)x, n, act, p0);
}

void act_and_mul_quant(void* out_q, float* scale_out, const float* scale_in, const void* x, int tokens, int d, int act,
                       float p0, float p1, int group, int ue8m0, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = 256;
  if (dtype == 0)
    act_and_mul_quant_kernel<__nv_bfloat16><<<tokens, th, 0, stream>>>((uint8_t*)out_q, scale_out, scale_in,
                                                                       (const __nv_bfloat16*)x, d, act, p0, p1, group, ue8m0);
  else
    act_and_mul_quant_kernel<__half><<<tokens, th, 0, stream>>>((uint8_t*)out_q, scale_out, scale_in, (const __half*)x,
                                                                d, act, p0, p1, group, ue8m0);
}

}  // namespace b200
