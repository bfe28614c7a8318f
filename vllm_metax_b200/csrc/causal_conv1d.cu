// Depthwise causal convolution over ragged token batches with a per-sequence carry (the short convolution in front
// of gated-delta-rule / Mamba style mixers).
//
//   y[t, c] = act( bias[c] + sum_j w[c, j] * x_ext[t - (K-1) + j, c] ),   j = 0 .. K-1
//
// where x_ext is the sequence's tokens preceded by the K-1 inputs kept from its previous step (zeros for a new
// sequence).  Tokens are flat [T, C] with sequences given by query_start_loc; the carry lives in
// state[slot, K-1, C] (oldest first) and is rewritten by a second kernel once the outputs are done, so a decode step
// (one token) and a prefill chunk (thousands) go through the same two launches.
//
// Grid of the forward kernel: (C / 128, ceil(T / kTokPerCta)); threads along channels so every load is coalesced; the
// first 32 threads of a CTA look up each token's sequence (binary search) into shared memory, so the token loop has
// no data-dependent control flow beyond uniform branches and can be unrolled.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "ops.h"

namespace b200 {
namespace {

constexpr int kMaxK = 8;
constexpr int kTokPerCta = 32;

template <typename T>
__device__ __forceinline__ float ld(const T* p) { return (float)*p; }
template <typename T>
__device__ __forceinline__ void st(T* p, float v) { *p = (T)v; }

template <typename T>
__global__ void conv1d_fwd_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t x_stride,
                                  const T* __restrict__ w, const T* __restrict__ bias, const T* __restrict__ state,
                                  const int* __restrict__ qsl, const int* __restrict__ state_idx,
                                  const int* __restrict__ has_init, int batch, int tokens, int channels, int K,
                                  int silu) {
  // per token of this CTA's chunk: first token of its sequence, and the carry slot to read (-1: zeros)
  __shared__ int s_start[kTokPerCta];
  __shared__ int s_slot[kTokPerCta];
  const int t0 = blockIdx.y * kTokPerCta;
  const int t1 = min(tokens, t0 + kTokPerCta);
  if (threadIdx.x < kTokPerCta) {
    const int t = t0 + threadIdx.x;
    int start = -1, slot = -1;
    if (t < t1 && t < qsl[batch]) {
      int lo = 0, hi = batch - 1;               // largest s with qsl[s] <= t
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (qsl[mid] <= t) lo = mid; else hi = mid - 1;
      }
      start = qsl[lo];
      const int sl = state_idx ? state_idx[lo] : -1;
      if (sl >= 0 && state != nullptr && (has_init == nullptr || has_init[lo] != 0)) slot = sl;
    }
    s_start[threadIdx.x] = start;               // -1: padding row after the last sequence, nothing is written
    s_slot[threadIdx.x] = slot;
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float wr[kMaxK];
#pragma unroll
  for (int j = 0; j < kMaxK; ++j) wr[j] = j < K ? ld(w + (int64_t)c * K + j) : 0.f;
  const float b = bias ? ld(bias + c) : 0.f;
#pragma unroll 4
  for (int i = 0; i < kTokPerCta; ++i) {
    const int t = t0 + i;
    const int start = s_start[i];
    if (t >= t1 || start < 0) continue;
    const int slot = s_slot[i];
    float acc = b;
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) {
      if (j >= K) break;
      const int src = t - (K - 1) + j;              // token index of this tap
      float v = 0.f;
      if (src >= start) {
        v = ld(x + (int64_t)src * x_stride + c);
      } else if (slot >= 0) {
        const int back = start - src;               // 1 .. K-1 tokens before the sequence's first new token
        v = ld(state + ((int64_t)slot * (K - 1) + (K - 1 - back)) * channels + c);
      }
      acc += wr[j] * v;
    }
    if (silu) acc = acc / (1.f + __expf(-acc));
    st(out + (int64_t)t * channels + c, acc);
  }
}

// One thread per (sequence, channel): the last K-1 entries of [carry | new tokens] become the new carry.
template <typename T>
__global__ void conv1d_state_kernel(T* __restrict__ state, const T* __restrict__ x, int64_t x_stride,
                                    const int* __restrict__ qsl, const int* __restrict__ state_idx,
                                    const int* __restrict__ has_init, int channels, int K) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= channels) return;
  const int slot = state_idx[s];
  if (slot < 0) return;
  const int start = qsl[s], n = qsl[s + 1] - start;
  if (n <= 0) return;
  const bool carry = has_init == nullptr || has_init[s] != 0;
  T* st_base = state + (int64_t)slot * (K - 1) * channels + c;
  float keep[kMaxK];
#pragma unroll
  for (int j = 0; j < kMaxK - 1; ++j) {
    if (j >= K - 1) break;
    const int pos = n - (K - 1) + j;                // position in the new tokens; negative: still in the old carry
    if (pos >= 0) keep[j] = ld(x + (int64_t)(start + pos) * x_stride + c);
    else keep[j] = carry ? ld(st_base + (int64_t)(K - 1 + pos) * channels) : 0.f;
  }
#pragma unroll
  for (int j = 0; j < kMaxK - 1; ++j) {
    if (j >= K - 1) break;
    st(st_base + (int64_t)j * channels, keep[j]);
  }
}

template <typename T>
void launch(void* out, const void* x, int64_t x_stride, const void* w, const void* bias, void* state, const int* qsl,
            const int* state_idx, const int* has_init, int batch, int tokens, int channels, int K, int silu,
            cudaStream_t stream) {
  const int threads = 128;
  dim3 grid((channels + threads - 1) / threads, (tokens + kTokPerCta - 1) / kTokPerCta);
  conv1d_fwd_kernel<T><<<grid, threads, 0, stream>>>((T*)out, (const T*)x, x_stride, (const T*)w, (const T*)bias,
                                                     (const T*)state, qsl, state_idx, has_init, batch, tokens, channels,
                                                     K, silu);
  if (state != nullptr && state_idx != nullptr) {
    dim3 g2((channels + threads - 1) / threads, batch);
    conv1d_state_kernel<T><<<g2, threads, 0, stream>>>((T*)state, (const T*)x, x_stride, qsl, state_idx, has_init,
                                                       channels, K);
  }
}

}  // namespace

int causal_conv1d(void* out, const void* x, int64_t x_stride, const void* w, const void* bias, void* state,
                  const int* query_start_loc, const int* state_idx, const int* has_init, int batch, int tokens,
                  int channels, int K, int silu, int dtype, cudaStream_t stream) {
  if (K < 2 || K > kMaxK || batch <= 0 || tokens <= 0) return K < 2 || K > kMaxK ? 1 : 0;
  if (dtype == 0)
    launch<__nv_bfloat16>(out, x, x_stride, w, bias, state, query_start_loc, state_idx, has_init, batch, tokens,
                          channels, K, silu, stream);
  else if (dtype == 1)
    launch<__half>(out, x, x_stride, w, bias, state, query_start_loc, state_idx, has_init, batch, tokens, channels, K,
                   silu, stream);
  else
    launch<float>(out, x, x_stride, w, bias, state, query_start_loc, state_idx, has_init, batch, tokens, channels, K,
                  silu, stream);
  return 0;
}

}  // namespace b200
