// Manifold hyper-connection (mHC) residual-stream mixing of DeepSeek-V4: the residual is kept as M parallel
// streams [T, M, H]; every sub-layer reads ONE mixed input and writes back into all streams.
//
//   pre   :  r      = residual[t] flattened to [M*H]
//            mixes  = (r . fn[j]) * rsqrt(mean(r^2) + rms_eps)          j < 2M + M*M      (fn fp32 [2M+M*M, M*H])
//            mixes  = mixes * scale[seg(j)] + base[j]
//            pre_i  = sigmoid(mixes[i]) + pre_eps ;  post_i = sigmoid(mixes[M+i]) * post_mult
//            comb   = sinkhorn(mixes[2M:].view(M, M))   (softmax rows + eps, then alternating column / row
//                                                         normalisation, `iters` rounds in total)
//            x[t]   = sum_i pre_i * residual[t, i, :]                   (the sub-layer's input, T dtype)
//   post  :  residual'[t, n, :] = y[t] * post_n + sum_m comb[m, n] * residual[t, m, :]
//   fused :  post of the previous sub-layer and pre of the next one in ONE pass over the streams
//   head  :  pre only, with M mixes (no post / comb) - the final mix before the output norm
// One CTA handles 4 tokens so that every fn element fetched from L2 feeds 4 tokens; the dot products live in
// registers (4 x 24 accumulators), the 4x4 Sinkhorn runs on one thread per token.
// Parity: models/deepseek_v4/ops/mhc/torch.py:10-299 (reference math) and ops/mhc/tilelang_kernels.py:45-356
// (_mhc_pre_big_fuse, _mhc_post_fwd, mhc_fused_tilelang, hc_head_fuse_tilelang) of the reference.
#include "common.cuh"
#include "ops.h"

namespace b200 {

constexpr int kMhcTT = 4;        // tokens per CTA
constexpr int kMhcMaxM = 4;
constexpr int kMhcMaxMix = 2 * kMhcMaxM + kMhcMaxM * kMhcMaxM;   // 24


template <typename T, bool FUSED>
__global__ void __launch_bounds__(256)
mhc_pre_kernel(const MhcParams p) {
  const int M = p.M, H = p.H, MH = M * H;
  const int nmix = p.head ? M : 2 * M + M * M;
  const int t0 = blockIdx.x * kMhcTT;
  const int nt = min(kMhcTT, p.T - t0);
  const T* res = reinterpret_cast<const T*>(p.residual);
  T* res_out = reinterpret_cast<T*>(p.residual_out);
  const T* y = reinterpret_cast<const T*>(p.y);
  __shared__ float s_red[8][kMhcTT][kMhcMaxMix + 1];
  __shared__ float s_pre[kMhcTT][kMhcMaxM];
  __shared__ float s_post[kMhcTT][kMhcMaxM], s_comb[kMhcTT][kMhcMaxM * kMhcMaxM];

  if (FUSED) {
    for (int i = threadIdx.x; i < kMhcTT * M; i += blockDim.x) {
      const int tt = i / M;
      s_post[tt][i % M] = tt < nt ? p.post_in[(size_t)(t0 + tt) * M + i % M] : 0.f;
    }
    for (int i = threadIdx.x; i < kMhcTT * M * M; i += blockDim.x) {
      const int tt = i / (M * M);
      s_comb[tt][i % (M * M)] = tt < nt ? p.comb_in[(size_t)(t0 + tt) * M * M + i % (M * M)] : 0.f;
    }
    __syncthreads();
  }

  float acc[kMhcTT][kMhcMaxMix];
  float sq[kMhcTT];
#pragma unroll
  for (int tt = 0; tt < kMhcTT; ++tt) {
    sq[tt] = 0.f;
#pragma unroll
    for (int j = 0; j < kMhcMaxMix; ++j) acc[tt][j] = 0.f;
  }
  for (int j = threadIdx.x; j < MH; j += blockDim.x) {
    float r[kMhcTT];
    const int n = j / H, k = j - n * H;
#pragma unroll
    for (int tt = 0; tt < kMhcTT; ++tt) {
      r[tt] = 0.f;
      if (tt < nt) {
        const size_t tok = (size_t)(t0 + tt);
        if (FUSED) {
          float v = to_f(y[tok * H + k]) * s_post[tt][n];
          for (int m = 0; m < M; ++m) v += s_comb[tt][m * M + n] * to_f(res[(tok * M + m) * H + k]);
          const T vr = from_f<T>(v);
          r[tt] = to_f(vr);            // the streams are stored in T: mix what will be read back
          res_out[(tok * M + n) * H + k] = vr;     // out of place: other threads still read the old streams
        } else {
          r[tt] = to_f(res[tok * MH + j]);
        }
        sq[tt] += r[tt] * r[tt];
      }
    }
#pragma unroll
    for (int q = 0; q < kMhcMaxMix; ++q) {
      if (q < nmix) {
        const float f = p.fn[(size_t)q * MH + j];
#pragma unroll
        for (int tt = 0; tt < kMhcTT; ++tt) acc[tt][q] = fmaf(r[tt], f, acc[tt][q]);
      }
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int tt = 0; tt < kMhcTT; ++tt) {
#pragma unroll
    for (int q = 0; q < kMhcMaxMix; ++q) {
      const float v = warp_sum(acc[tt][q]);
      if (lane == 0) s_red[warp][tt][q] = v;
    }
    const float v = warp_sum(sq[tt]);
    if (lane == 0) s_red[warp][tt][kMhcMaxMix] = v;
  }
  __syncthreads();
  if ((int)threadIdx.x < nt) {
    const int tt = threadIdx.x;
    float mix[kMhcMaxMix];
    float ss = 0.f;
    for (int w = 0; w < 8; ++w) ss += s_red[w][tt][kMhcMaxMix];
    const float inv = rsqrtf(ss / (float)MH + p.rms_eps);
    for (int q = 0; q < nmix; ++q) {
      float v = 0.f;
      for (int w = 0; w < 8; ++w) v += s_red[w][tt][q];
      const float sc = p.head ? p.scale[0] : p.scale[q < M ? 0 : (q < 2 * M ? 1 : 2)];
      mix[q] = v * inv * sc + p.base[q];
    }
    const size_t tok = (size_t)(t0 + tt);
    for (int i = 0; i < M; ++i) s_pre[tt][i] = 1.f / (1.f + __expf(-mix[i])) + p.pre_eps;
    if (!p.head) {
      for (int i = 0; i < M; ++i) p.post_out[tok * M + i] = 1.f / (1.f + __expf(-mix[M + i])) * p.post_mult;
      float c[kMhcMaxM][kMhcMaxM];
      for (int a = 0; a < M; ++a) {          // row softmax + eps
        float mx = -INFINITY, sum = 0.f;
        for (int b = 0; b < M; ++b) mx = fmaxf(mx, mix[2 * M + a * M + b]);
        for (int b = 0; b < M; ++b) { c[a][b] = __expf(mix[2 * M + a * M + b] - mx); sum += c[a][b]; }
        for (int b = 0; b < M; ++b) c[a][b] = c[a][b] / sum + p.sinkhorn_eps;
      }
      auto col_norm = [&]() {
        for (int b = 0; b < M; ++b) {
          float s = 0.f;
          for (int a = 0; a < M; ++a) s += c[a][b];
          for (int a = 0; a < M; ++a) c[a][b] /= (s + p.sinkhorn_eps);
        }
      };
      auto row_norm = [&]() {
        for (int a = 0; a < M; ++a) {
          float s = 0.f;
          for (int b = 0; b < M; ++b) s += c[a][b];
          for (int b = 0; b < M; ++b) c[a][b] /= (s + p.sinkhorn_eps);
        }
      };
      col_norm();
      for (int it = 1; it < p.iters; ++it) { row_norm(); col_norm(); }
      for (int a = 0; a < M; ++a)
        for (int b = 0; b < M; ++b) p.comb_out[tok * M * M + a * M + b] = c[a][b];
    }
  }
  __syncthreads();
  // sub-layer input: x[t] = sum_i pre_i * stream_i
  const T* src = FUSED ? res_out : res;
  T* xo = reinterpret_cast<T*>(p.x_out);
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    for (int tt = 0; tt < nt; ++tt) {
      const size_t tok = (size_t)(t0 + tt);
      float v = 0.f;
      for (int i = 0; i < M; ++i) v += s_pre[tt][i] * to_f(src[(tok * M + i) * H + k]);
      xo[tok * H + k] = from_f<T>(v);
    }
  }
}

template <typename T>
__global__ void mhc_post_kernel(T* __restrict__ out, const T* __restrict__ y, const T* __restrict__ res,
                                const float* __restrict__ post, const float* __restrict__ comb, int tokens, int M, int H) {
  const size_t tok = blockIdx.x;
  __shared__ float s_post[kMhcMaxM], s_comb[kMhcMaxM * kMhcMaxM];
  if ((int)threadIdx.x < M) s_post[threadIdx.x] = post[tok * M + threadIdx.x];
  if ((int)threadIdx.x < M * M) s_comb[threadIdx.x] = comb[tok * M * M + threadIdx.x];
  __syncthreads();
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    float r[kMhcMaxM];
    for (int m = 0; m < M; ++m) r[m] = to_f(res[(tok * M + m) * H + k]);
    const float yv = to_f(y[tok * H + k]);
    for (int n = 0; n < M; ++n) {
      float v = yv * s_post[n];
      for (int m = 0; m < M; ++m) v += s_comb[m * M + n] * r[m];
      out[(tok * M + n) * H + k] = from_f<T>(v);
    }
  }
}

// fused != 0 requires residual_out != residual (the new streams are produced while the old ones are still read).
int mhc_pre(const MhcParams& p, int fused, int dtype, cudaStream_t stream) {
  if (p.T <= 0) return 0;
  if (p.M < 1 || p.M > kMhcMaxM) return 1;
  if (fused && p.residual_out == p.residual) return 2;
  const int grid = ceil_div(p.T, kMhcTT);
  if (dtype == 0) {
    if (fused) mhc_pre_kernel<__nv_bfloat16, true><<<grid, 256, 0, stream>>>(p);
    else mhc_pre_kernel<__nv_bfloat16, false><<<grid, 256, 0, stream>>>(p);
  } else {
    if (fused) mhc_pre_kernel<__half, true><<<grid, 256, 0, stream>>>(p);
    else mhc_pre_kernel<__half, false><<<grid, 256, 0, stream>>>(p);
  }
  return 0;
}

void mhc_post(void* out, const void* y, const void* res, const float* post, const float* comb, int tokens, int M, int H,
              int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  if (dtype == 0)
    mhc_post_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)y, (const __nv_bfloat16*)res, post, comb, tokens, M, H);
  else
    mhc_post_kernel<__half><<<tokens, 256, 0, stream>>>((__half*)out, (const __half*)y, (const __half*)res, post, comb, tokens, M, H);
}

}  // namespace b200
