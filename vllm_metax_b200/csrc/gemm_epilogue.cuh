// Row-segment epilogue shared by the GEMM kernels: one thread owns one output row and CH
// consecutive fp32 accumulator columns (as read from TMEM), applies bias / residual or the
// SiLU-gate over interleaved (gate, up) columns, converts and stores.
#pragma once
#include "common.cuh"

namespace b200 {

// r[0..CH): accumulators of columns cb0..cb0+CH of row `row`; n_cols = number of valid columns.
template <typename T, int CH>
__device__ __forceinline__ void store_row_segment(const uint32_t (&r)[32], int row, int cb0, int n_cols,
                                                  T* __restrict__ C, int ldc, const T* __restrict__ bias,
                                                  const T* __restrict__ residual, int ldr, int epi) {
  if (epi == 1) {
    T* dst = C + (size_t)row * ldc + (cb0 >> 1);
#pragma unroll
    for (int v = 0; v < CH / 8; ++v) {
      const int col = cb0 + v * 8;
      if (col + 8 <= n_cols) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
        if (bias) {
          float b[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(bias + col), b);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] += b[i];
        }
        T o4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float g = to_f(from_f<T>(f[2 * i])), u = to_f(from_f<T>(f[2 * i + 1]));
          o4[i] = from_f<T>(g / (1.f + __expf(-g)) * u);
        }
        *reinterpret_cast<uint2*>(dst + v * 4) = *reinterpret_cast<const uint2*>(o4);
      }
    }
    return;
  }
  T* dst = C + (size_t)row * ldc + cb0;
  const T* res = residual ? residual + (size_t)row * ldr + cb0 : nullptr;
#pragma unroll
  for (int v = 0; v < CH / 8; ++v) {
    const int col = cb0 + v * 8;
    if (col + 8 <= n_cols) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
      if (bias) {
        float b[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(bias + col), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += b[i];
      }
      if (res) {
        float b[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(res + v * 8), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += b[i];
      }
      *reinterpret_cast<uint4*>(dst + v * 8) = pack8<T>(f);
    } else {
      for (int i = 0; i < 8; ++i) {
        if (col + i < n_cols) {
          float f = __uint_as_float(r[v * 8 + i]);
          if (bias) f += to_f(bias[col + i]);
          if (res) f += to_f(res[v * 8 + i]);
          dst[v * 8 + i] = from_f<T>(f);
        }
      }
    }
  }
}

}  // namespace b200
