// RMSNorm family: plain, fused residual-add, Gemma (+1 weight), per-head
// (q/k norm) and the variants that quantise their output (static fp8, dynamic
// per-token fp8/int8, per-128-block fp8).  One CTA per token row; the row is
// staged once in shared memory so global memory is read exactly once.
// Parity: csrc/layernorm_kernels.cu:15,100,172 and layernorm_quant_kernels.cu:23-161,
// quantization/fused_kernels/fused_layernorm_dynamic_per_token_quant.cu:49-95 of the reference.
#include "common.cuh"

namespace b200 {

// mode bits
constexpr int kNormGemma = 1;   // weight + 1

template <typename T, bool ADD_RESIDUAL>
__global__ void rms_norm_kernel(T* __restrict__ out, T* __restrict__ x, T* __restrict__ residual,
                                const T* __restrict__ weight, float eps, int hidden, int64_t x_stride,
                                int64_t out_stride, int mode) {
  extern __shared__ __align__(16) uint8_t smem_row[];
  __shared__ float red[32];
  T* row = reinterpret_cast<T*>(smem_row);
  const int64_t t = blockIdx.x;
  const T* xin = x + t * x_stride;
  T* res = ADD_RESIDUAL ? residual + t * (int64_t)hidden : nullptr;
  const int nvec = hidden >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8<T>(reinterpret_cast<const uint4*>(xin)[v], f);
    if (ADD_RESIDUAL) {
      float r[8];
      unpack8<T>(reinterpret_cast<const uint4*>(res)[v], r);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += r[i];
      uint4 packed = pack8<T>(f);
      reinterpret_cast<uint4*>(res)[v] = packed;
      unpack8<T>(packed, f);  // the norm sees the rounded residual
    }
    reinterpret_cast<uint4*>(row)[v] = pack8<T>(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  for (int i = (nvec << 3) + threadIdx.x; i < hidden; i += blockDim.x) {
    float f = to_f(xin[i]);
    if (ADD_RESIDUAL) {
      f += to_f(res[i]);
      T rr = from_f<T>(f);
      res[i] = rr;
      f = to_f(rr);
    }
    row[i] = from_f<T>(f);
    ss += f * f;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  const float wadd = (mode & kNormGemma) ? 1.f : 0.f;
  T* o = out + t * out_stride;
  __syncthreads();
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8], w[8];
    unpack8<T>(reinterpret_cast<const uint4*>(row)[v], f);
    unpack8<T>(reinterpret_cast<const uint4*>(weight)[v], w);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * (w[i] + wadd);
    reinterpret_cast<uint4*>(o)[v] = pack8<T>(f);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f<T>(to_f(row[i]) * inv * (to_f(weight[i]) + wadd));
}

// Register-resident variant for rows of 128 * VPT vectors (hidden = 1024 * VPT elements): every thread issues
// all of its 16-byte loads before the first use, keeps the row in registers between the two passes and writes
// once; the only shared-memory traffic is the block reduction.
template <typename T, bool ADD_RESIDUAL, int VPT>
__global__ void __launch_bounds__(128)
rms_norm_reg_kernel(T* __restrict__ out, T* __restrict__ x, T* __restrict__ residual, const T* __restrict__ weight,
                    float eps, int hidden, int64_t x_stride, int64_t out_stride, int mode) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const uint4* xin = reinterpret_cast<const uint4*>(x + t * x_stride);
  uint4* res = ADD_RESIDUAL ? reinterpret_cast<uint4*>(residual + t * (int64_t)hidden) : nullptr;
  uint4 xv[VPT], rv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) xv[i] = xin[threadIdx.x + i * 128];
  if (ADD_RESIDUAL) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) rv[i] = res[threadIdx.x + i * 128];
  }
  float f[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    unpack8<T>(xv[i], f[i]);
    if (ADD_RESIDUAL) {
      float r[8];
      unpack8<T>(rv[i], r);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[i][e] += r[e];
      const uint4 packed = pack8<T>(f[i]);
      res[threadIdx.x + i * 128] = packed;
      unpack8<T>(packed, f[i]);  // the norm sees the rounded residual
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += f[i][e] * f[i][e];
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  const float wadd = (mode & kNormGemma) ? 1.f : 0.f;
  uint4* o = reinterpret_cast<uint4*>(out + t * out_stride);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    float w[8];
    unpack8<T>(reinterpret_cast<const uint4*>(weight)[threadIdx.x + i * 128], w);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[i][e] = f[i][e] * inv * (w[e] + wadd);
    o[threadIdx.x + i * 128] = pack8<T>(f[i]);
  }
}

// Per-head RMSNorm over the last dim (head_dim <= 256): one warp per (token, head).
template <typename T>
__global__ void head_rms_norm_kernel(T* __restrict__ x, const T* __restrict__ weight, float eps, int num_rows,
                                     int heads, int head_dim, int64_t token_stride) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= num_rows * heads) return;
  const int t = gw / heads, h = gw % heads;
  T* p = x + t * token_stride + (int64_t)h * head_dim;
  float v[8];
  float ss = 0.f;
  const int per = head_dim / 32;
  for (int i = 0; i < per; ++i) {
    v[i] = to_f(p[lane * per + i]);
    ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / head_dim + eps);
  for (int i = 0; i < per; ++i) p[lane * per + i] = from_f<T>(v[i] * inv * to_f(weight[lane * per + i]));
}

// RMSNorm (+ optional residual add) followed by quantisation.
//   qmode 0: static per-tensor fp8 (scale[0])        -> out_q e4m3
//   qmode 1: dynamic per-token fp8 (scale_out[t])    -> out_q e4m3
//   qmode 2: dynamic per-token int8 (scale_out[t])   -> out_q int8
//   qmode 3: per-`group` fp8 (scale_out[t, hidden/group]), ue8m0 rounding optional
template <typename T, bool ADD_RESIDUAL>
__global__ void rms_norm_quant_kernel(uint8_t* __restrict__ out_q, float* __restrict__ scale_out,
                                      const float* __restrict__ scale_in, const T* __restrict__ x,
                                      T* __restrict__ residual, const T* __restrict__ weight, float eps, int hidden,
                                      int qmode, int group, int ue8m0, float scale_ub) {
  extern __shared__ __align__(16) uint8_t smem_row[];
  __shared__ float red[32];
  float* row = reinterpret_cast<float*>(smem_row);
  const int64_t t = blockIdx.x;
  const T* xin = x + t * (int64_t)hidden;
  T* res = ADD_RESIDUAL ? residual + t * (int64_t)hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float f = to_f(xin[i]);
    if (ADD_RESIDUAL) {
      f += to_f(res[i]);
      T rr = from_f<T>(f);
      res[i] = rr;
      f = to_f(rr);
    }
    row[i] = f;
    ss += f * f;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  __syncthreads();
  float amax = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    // normalised value is rounded to T first, as the unfused pipeline would
    float y = to_f(from_f<T>(row[i] * inv * to_f(weight[i])));
    row[i] = y;
    amax = fmaxf(amax, fabsf(y));
  }
  uint8_t* oq = out_q + t * (int64_t)hidden;
  if (qmode == 3) {
    __syncthreads();
    const int ngroups = hidden / group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = warp; g < ngroups; g += nw) {
      float m = 0.f;
      for (int i = lane; i < group; i += 32) m = fmaxf(m, fabsf(row[g * group + i]));
      m = fmaxf(warp_max(m), 1e-10f);
      float s = m / 448.f;
      if (ue8m0) s = ue8m0_ceil(s);
      if (lane == 0) scale_out[t * ngroups + g] = s;
      for (int i = lane; i < group; i += 32) oq[g * group + i] = float_to_fp8_e4m3(row[g * group + i] / s);
    }
    return;
  }
  float s;
  if (qmode == 0) {
    s = scale_in[0];
  } else {
    amax = block_max(amax, red);
    if (qmode == 1) {
      if (scale_ub > 0.f) amax = fminf(amax, scale_ub);
      s = fmaxf(amax / 448.f, 1.f / (448.f * 512.f));
    } else {
      s = fmaxf(amax, 1e-10f) / 127.f;
    }
    if (threadIdx.x == 0) scale_out[t] = s;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float y = row[i] / s;
    if (qmode == 2) {
      int q = __float2int_rn(y);
      q = max(-128, min(127, q));
      oq[i] = (uint8_t)(int8_t)q;
    } else {
      oq[i] = float_to_fp8_e4m3(y);
    }
  }
}

static int norm_threads(int hidden, int tokens) {
  int th = hidden / 8;
  const int cap = tokens < 256 ? 1024 : 256;
  th = th < 32 ? 32 : th;
  th = th > cap ? cap : th;
  return (th + 31) / 32 * 32;
}

template <typename T>
static void rms_norm_t(void* out, void* x, void* residual, const void* weight, float eps, int tokens, int hidden,
                       int64_t x_stride, int64_t out_stride, int mode, cudaStream_t stream) {
  const bool vec_ok = hidden % 1024 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 && tokens >= 32 &&
                      ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x) |
                        reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0;
  const int vpt = hidden / 1024;
  if (vec_ok && (vpt == 1 || vpt == 2 || vpt == 4 || vpt == 8)) {
#define REG(ADD, V)                                                                                                \
  rms_norm_reg_kernel<T, ADD, V><<<tokens, 128, 0, stream>>>((T*)out, (T*)x, (T*)residual, (const T*)weight, eps,  \
                                                             hidden, x_stride, out_stride, mode)
#define REGV(ADD)                                                                                                  \
  do {                                                                                                             \
    if (vpt == 1) REG(ADD, 1); else if (vpt == 2) REG(ADD, 2); else if (vpt == 4) REG(ADD, 4); else REG(ADD, 8);   \
  } while (0)
    if (residual) REGV(true); else REGV(false);
#undef REGV
#undef REG
    return;
  }
  const int th = norm_threads(hidden, tokens);
  const size_t sm = (size_t)hidden * sizeof(T);
  if (residual)
    rms_norm_kernel<T, true><<<tokens, th, sm, stream>>>((T*)out, (T*)x, (T*)residual, (const T*)weight, eps, hidden,
                                                         x_stride, out_stride, mode);
  else
    rms_norm_kernel<T, false><<<tokens, th, sm, stream>>>((T*)out, (T*)x, nullptr, (const T*)weight, eps, hidden,
                                                          x_stride, out_stride, mode);
}

// dtype: 0 bf16, 1 fp16, 2 fp32 (fp32 rows must have hidden % 8 == 0 only for the vector path; tail handled)
void rms_norm(void* out, void* x, void* residual, const void* weight, float eps, int tokens, int hidden,
              int64_t x_stride, int64_t out_stride, int dtype, int mode, cudaStream_t stream) {
  if (tokens <= 0) return;
  if (dtype == 0) rms_norm_t<__nv_bfloat16>(out, x, residual, weight, eps, tokens, hidden, x_stride, out_stride, mode, stream);
  else rms_norm_t<__half>(out, x, residual, weight, eps, tokens, hidden, x_stride, out_stride, mode, stream);
}

void head_rms_norm(void* x, const void* weight, float eps, int tokens, int heads, int head_dim, int64_t token_stride,
                   int dtype, cudaStream_t stream) {
  const int rows = tokens * heads;
  if (rows <= 0) return;
  const int th = 256;
  const int blocks = ceil_div(rows * 32, th);
  if (dtype == 0)
    head_rms_norm_kernel<__nv_bfloat16><<<blocks, th, 0, stream>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)weight, eps,
                                                                   tokens, heads, head_dim, token_stride);
  else
    head_rms_norm_kernel<__half><<<blocks, th, 0, stream>>>((__half*)x, (const __half*)weight, eps, tokens, heads,
                                                            head_dim, token_stride);
}

void rms_norm_quant(void* out_q, float* scale_out, const float* scale_in, const void* x, void* residual,
                    const void* weight, float eps, int tokens, int hidden, int dtype, int qmode, int group, int ue8m0,
                    float scale_ub, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = 256;
  const size_t sm = (size_t)hidden * sizeof(float);
#define LAUNCH(T, ADD)                                                                                             \
  rms_norm_quant_kernel<T, ADD><<<tokens, th, sm, stream>>>((uint8_t*)out_q, scale_out, scale_in, (const T*)x,     \
                                                            (T*)residual, (const T*)weight, eps, hidden, qmode,    \
                                                            group, ue8m0, scale_ub)
  if (dtype == 0) {
    if (residual) LAUNCH(__nv_bfloat16, true); else LAUNCH(__nv_bfloat16, false);
  } else {
    if (residual) LAUNCH(__half, true); else LAUNCH(__half, false);
  }
#undef LAUNCH
}

}  // namespace b200
