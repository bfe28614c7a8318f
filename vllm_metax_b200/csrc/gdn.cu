// Gated delta rule (linear attention of Qwen3-Next / Kimi-style GDN blocks), recurrent form:
//
//   S  <- exp(g_t) * S                         decay            S: [Dk, Dv] per (sequence, value head), fp32
//   u  <- beta_t * (v_t - S^T k_t)              delta            u: [Dv]
//   S  <- S + k_t u^T
//   o_t = S^T (scale * q_t)
//
// One CTA per (sequence, value head); thread j owns column j of S (Dk = 128 values in registers) and walks the
// sequence's tokens in order: q_t and k_t are staged in shared memory (optionally L2-normalised there), every
// thread does 3 x 128 FMAs per token and no cross-thread reduction, so a token costs two barriers.  The state is
// read from / written to a slot pool (fp32) so that decode steps and chunked prefill continue where the last call
// stopped.  This is the sequential form: right for decode and short prompts; long prompts want the chunked
// (WY-representation) algorithm on the tensor cores, which is not built.
// Covers ChunkGatedDeltaRule.forward (vllm_metax/registry/custom_ops/layers/mamba/qwen_gdn_linear_attn.py:16-88)
// and the fused recurrent decode step of the same block.
#include "common.cuh"
#include "ops.h"

namespace b200 {

template <typename T>
__global__ void __launch_bounds__(128)
gdn_recurrent_kernel(T* __restrict__ out, float* __restrict__ state, const T* __restrict__ q, const T* __restrict__ k,
                     const T* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                     const int* __restrict__ query_start_loc, const int* __restrict__ state_idx, int hq, int hv,
                     int64_t q_stride, int64_t k_stride, int64_t v_stride, float scale, int l2norm,
                     const int* __restrict__ has_initial) {
  constexpr int DK = 128, DV = 128;
  const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int hk = h / (hv / hq);                        // value heads share the q / k head of their group
  const int t0 = query_start_loc[b], t1 = query_start_loc[b + 1];
  const int slot = state_idx ? state_idx[b] : -1;
  __shared__ float s_q[DK], s_k[DK], s_red[8];
  float S[DK];
  float* sp = slot >= 0 ? state + (((int64_t)slot * hv + h) * DK) * DV + j : nullptr;
  if (sp != nullptr && (has_initial == nullptr || has_initial[b] != 0)) {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = sp[(int64_t)i * DV];
  } else {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = 0.f;
  }
  for (int t = t0; t < t1; ++t) {
    float qv = to_f(q[(int64_t)t * q_stride + hk * DK + j]) , kv = to_f(k[(int64_t)t * k_stride + hk * DK + j]);
    if (l2norm) {
      float sq = warp_sum(qv * qv), sk = warp_sum(kv * kv);
      if ((j & 31) == 0) { s_red[j >> 5] = sq; s_red[4 + (j >> 5)] = sk; }
      __syncthreads();
      sq = s_red[0] + s_red[1] + s_red[2] + s_red[3];
      sk = s_red[4] + s_red[5] + s_red[6] + s_red[7];
      qv *= rsqrtf(sq + 1e-6f);
      kv *= rsqrtf(sk + 1e-6f);
    }
    s_q[j] = qv * scale;
    s_k[j] = kv;
    __syncthreads();
    const float decay = __expf(g[(int64_t)t * hv + h]);
    const float bt = beta[(int64_t)t * hv + h];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      S[i] *= decay;
      dot = fmaf(S[i], s_k[i], dot);
    }
    const float u = bt * (to_f(v[(int64_t)t * v_stride + h * DV + j]) - dot);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      S[i] = fmaf(s_k[i], u, S[i]);
      o = fmaf(S[i], s_q[i], o);
    }
    out[((int64_t)t * hv + h) * DV + j] = from_f<T>(o);
    __syncthreads();                                   // s_q / s_k / s_red are rewritten by the next token
  }
  if (sp != nullptr) {
#pragma unroll
    for (int i = 0; i < DK; ++i) sp[(int64_t)i * DV] = S[i];
  }
}

// Returns 0, or 1 when the head sizes are not 128 / the head counts do not divide.
int gdn_recurrent(void* out, float* state, const void* q, const void* k, const void* v, const float* g, const float* beta,
                  const int* query_start_loc, const int* state_idx, int batch, int hq, int hv, int dk, int dv,
                  int64_t q_stride, int64_t k_stride, int64_t v_stride, float scale, int l2norm,
                  const int* has_initial, int dtype, cudaStream_t stream) {
  if (dk != 128 || dv != 128 || hq <= 0 || hv % hq != 0) return 1;
  if (batch <= 0) return 0;
  const dim3 grid(batch, hv);
  if (dtype == 0)
    gdn_recurrent_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        (__nv_bfloat16*)out, state, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, g, beta,
        query_start_loc, state_idx, hq, hv, q_stride, k_stride, v_stride, scale, l2norm, has_initial);
  else
    gdn_recurrent_kernel<__half><<<grid, 128, 0, stream>>>((__half*)out, state, (const __half*)q, (const __half*)k,
                                                           (const __half*)v, g, beta, query_start_loc, state_idx, hq, hv,
                                                           q_stride, k_stride, v_stride, scale, l2norm, has_initial);
  return 0;
}

}  // namespace b200
