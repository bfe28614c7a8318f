// Shared device helpers: vector types, bf16/fp16/fp8 conversion, warp/block
// reductions, launch-error plumbing.  sm_100a only.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "status.h"

namespace b200 {

__device__ __forceinline__ void report_status(StatusWord* s, int code, int where, int expected, int observed) {
  if (s != nullptr && atomicCAS(&s->code, 0, code) == 0) {
    s->where = where;
    s->expected = expected;
    s->observed = observed;
  }
}

template <typename T> struct Vec8 { uint4 raw; };

__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }

// 8 x 16-bit elements <-> 8 floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& r, float (&f)[8]) {
  const T* p = reinterpret_cast<const T*>(&r);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f(p[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 r;
  T* p = reinterpret_cast<T*>(&r);
#pragma unroll
  for (int i = 0; i < 8; ++i) p[i] = from_f<T>(f[i]);
  return r;
}

__device__ __forceinline__ float fp8_e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint8_t float_to_fp8_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// Smallest power of two >= s (s > 0, normal): the value a ue8m0 scale can represent.
__device__ __forceinline__ float ue8m0_ceil(float s) {
  uint32_t u = __float_as_uint(s);
  uint32_t e = u >> 23;
  if (u & 0x7FFFFFu) ++e;
  return __uint_as_float(e << 23);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `smem` must hold 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = (lane < nw) ? smem[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* smem) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = (lane < nw) ? smem[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace b200
