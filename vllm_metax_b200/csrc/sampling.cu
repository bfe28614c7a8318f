// Sampling and step-advance kernels.
//   argmax            greedy token per row of logits (bf16 / fp16 / fp32)
//   sample_topk_topp  temperature + top-k + top-p + min-p sampling, one CTA per row:
//                     softmax statistics, bisection on the probability threshold that
//                     realises the (k, p, min-p) cut, then inverse-CDF selection (in
//                     vocabulary order) among the kept tokens with a supplied uniform
//   repetition / presence / frequency penalties in place
//   advance_step      device-side bookkeeping between back-to-back decode iterations
//   embedding         row gather
// Parity: csrc/sampler.cu:14 (apply_repetition_penalties) and the sampler the
// reference takes from upstream; advance is what lets decode run without a host
// round trip per token.
#include "common.cuh"

namespace b200 {

// Greedy token: each row is cut into `splits` slices, one CTA per (row, slice), read as 16-byte vectors where the row
// allows it.  With one slice the CTA writes the token; otherwise it leaves (value, index) in device scratch and the
// last slice of the row to arrive (a ticket per row, reset by that CTA) picks the winner - ties go to the lower index
// at every level, so the answer does not depend on the split.  The scratch is per device and shared by all launches:
// argmax calls on one device must be stream-ordered.
constexpr int kArgmaxMaxSplits = 16;
constexpr int kArgmaxScratchRows = 4096;
static __device__ float g_argmax_val[kArgmaxScratchRows * kArgmaxMaxSplits];
static __device__ int g_argmax_idx[kArgmaxScratchRows * kArgmaxMaxSplits];
static __device__ unsigned g_argmax_ticket[kArgmaxScratchRows];

__device__ __forceinline__ void argmax_take(float& best, int& bi, float v, int i) {
  if (v > best || (v == best && i < bi)) { best = v; bi = i; }
}

template <typename T>
__global__ void __launch_bounds__(512)
argmax_kernel(int64_t* __restrict__ out, const T* __restrict__ logits, int vocab, int64_t stride, int splits) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ bool s_last;
  const int r = blockIdx.x, sp = blockIdx.y;
  const T* row = logits + (int64_t)r * stride;
  constexpr int V = 16 / sizeof(T);
  const int per = ((vocab + splits - 1) / splits + V - 1) / V * V;
  const int lo = sp * per, hi = min(vocab, lo + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int nvec = (hi - lo) / V;
    const uint4* rv = reinterpret_cast<const uint4*>(row + lo);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 u = rv[v];
      const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int j = 0; j < V; ++j) argmax_take(best, bi, to_f(e[j]), lo + v * V + j);
    }
    for (int i = lo + nvec * V + threadIdx.x; i < hi; i += blockDim.x) argmax_take(best, bi, to_f(row[i]), i);
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_take(best, bi, to_f(row[i]), i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_take(best, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w != 0) return;
  const int nw = blockDim.x >> 5;
  best = lane < nw ? sv[lane] : -INFINITY;
  bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_take(best, bi, ov, oi);
  }
  if (splits == 1) {
    if (lane == 0) out[r] = (bi == 0x7fffffff) ? 0 : bi;
    return;
  }
  if (lane == 0) {
    g_argmax_val[r * kArgmaxMaxSplits + sp] = best;
    g_argmax_idx[r * kArgmaxMaxSplits + sp] = bi;
    __threadfence();
    s_last = atomicAdd(&g_argmax_ticket[r], 1u) == (unsigned)(splits - 1);
  }
  __syncwarp();
  if (!s_last) return;
  __threadfence();
  best = lane < splits ? __ldcg(&g_argmax_val[r * kArgmaxMaxSplits + lane]) : -INFINITY;
  bi = lane < splits ? __ldcg(&g_argmax_idx[r * kArgmaxMaxSplits + lane]) : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_take(best, bi, ov, oi);
  }
  if (lane == 0) {
    out[r] = (bi == 0x7fffffff) ? 0 : bi;
    g_argmax_ticket[r] = 0;
  }
}

// One CTA (1024 threads) per row.
template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(int64_t* __restrict__ out, const T* __restrict__ logits, int vocab, int64_t stride,
              const float* __restrict__ temperature, const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const float* __restrict__ uniform) {
  __shared__ float red[32];
  __shared__ int s_ibcast;
  const int b = blockIdx.x;
  const T* row = logits + (int64_t)b * stride;
  const float temp = temperature[b];
  // greedy
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = to_f(row[i]);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  const float gmax = block_max(best, red);
  if (temp <= 0.f) {
    // smallest index attaining the max
    int cand = (best == gmax) ? bi : 0x7fffffff;
    __syncthreads();
    if (threadIdx.x == 0) s_ibcast = 0x7fffffff;
    __syncthreads();
    atomicMin(&s_ibcast, cand);
    __syncthreads();
    if (threadIdx.x == 0) out[b] = s_ibcast;
    return;
  }
  const float inv_t = 1.f / fmaxf(temp, 1e-6f);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += __expf((to_f(row[i]) - gmax) * inv_t);
  z = block_sum(z, red);
  const float inv_z = 1.f / z;
  // probability of token i: p_i = exp((x_i - gmax)/T) / z ; p_max = 1/z
  const int k = (top_k && top_k[b] > 0) ? min(top_k[b], vocab) : vocab;
  const float tp = top_p ? top_p[b] : 1.f;
  const float mp = min_p ? min_p[b] : 0.f;
  float thr = 0.f;  // keep p_i >= thr
  // Same order as upstream's sampler: top-k first, then top-p over the distribution RENORMALISED to the top-k set
  // (the smallest set of its leading tokens whose share of the top-k mass reaches top_p).  Both cuts are
  // thresholds on p_i, found by bisection (keep-set(tau) = {p_i >= tau} shrinks as tau grows).
  float mass_k = 1.f;
  if (k < vocab) {
    float lo = 0.f, hi = inv_z * 1.0000002f + 1e-30f;   // count(lo) = vocab >= k, count(hi) = 0
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        if (__expf((to_f(row[i]) - gmax) * inv_t) * inv_z >= mid) cnt += 1.f;
      cnt = block_sum(cnt, red);
      if (cnt >= (float)k) lo = mid; else hi = mid;      // lo converges to the k-th largest probability
    }
    thr = lo;
    float m = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float pi = __expf((to_f(row[i]) - gmax) * inv_t) * inv_z;
      if (pi >= thr) m += pi;
    }
    mass_k = block_sum(m, red);
  }
  if (tp < 1.f) {
    const float need = tp * mass_k;
    float lo = thr, hi = inv_z * 1.0000002f + 1e-30f;    // mass(lo) = mass_k >= need, mass(hi) = 0
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float m = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float pi = __expf((to_f(row[i]) - gmax) * inv_t) * inv_z;
        if (pi >= mid) m += pi;
      }
      m = block_sum(m, red);
      if (m >= need) lo = mid; else hi = mid;            // largest tau whose keep-set still covers top_p
    }
    thr = lo;
  }
  thr = fmaxf(thr, mp * inv_z);
  // mass of kept set
  float mass = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float pi = __expf((to_f(row[i]) - gmax) * inv_t) * inv_z;
    if (pi >= thr) mass += pi;
  }
  mass = block_sum(mass, red);
  const float target = uniform[b] * mass;
  // inverse CDF in vocabulary order, chunk by chunk
  float run = 0.f;
  int chosen = -1;
  const int nw = blockDim.x >> 5, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int base = 0; base < vocab && chosen < 0; base += blockDim.x) {
    const int i = base + threadIdx.x;
    float pi = 0.f;
    if (i < vocab) {
      pi = __expf((to_f(row[i]) - gmax) * inv_t) * inv_z;
      if (pi < thr) pi = 0.f;
    }
    // inclusive scan within the block
    float x = pi;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) red[w] = x;
    __syncthreads();
    float woff = 0.f;
    for (int j = 0; j < w; ++j) woff += red[j];
    float tot = 0.f;
    for (int j = 0; j < nw; ++j) tot += red[j];
    const float incl = run + woff + x;
    if (threadIdx.x == 0) s_ibcast = 0x7fffffff;
    __syncthreads();
    if (pi > 0.f && incl >= target) atomicMin(&s_ibcast, i);
    __syncthreads();
    if (s_ibcast != 0x7fffffff) chosen = s_ibcast;
    run += tot;
    __syncthreads();
  }
  // numerical tail (target beyond the accumulated mass): fall back to the arg-max
  if (chosen < 0) {
    int cand = (best == gmax) ? bi : 0x7fffffff;
    if (threadIdx.x == 0) s_ibcast = 0x7fffffff;
    __syncthreads();
    atomicMin(&s_ibcast, cand);
    __syncthreads();
    chosen = s_ibcast;
  }
  if (threadIdx.x == 0) out[b] = chosen;
}

// logits[b, v]: seen tokens get logit/penalty (if > 0) or logit*penalty; then presence / frequency.
template <typename T>
__global__ void penalties_kernel(T* __restrict__ logits, const int* __restrict__ prompt_mask_or_null,
                                 const int* __restrict__ output_counts, const float* __restrict__ rep,
                                 const float* __restrict__ presence, const float* __restrict__ frequency, int vocab,
                                 int64_t stride) {
  const int b = blockIdx.y;
  T* row = logits + (int64_t)b * stride;
  const float rp = rep ? rep[b] : 1.f, pp = presence ? presence[b] : 0.f, fp = frequency ? frequency[b] : 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
    const int cnt = output_counts ? output_counts[(int64_t)b * vocab + i] : 0;
    const bool in_prompt = prompt_mask_or_null ? prompt_mask_or_null[(int64_t)b * vocab + i] != 0 : false;
    float v = to_f(row[i]);
    if (cnt > 0 || in_prompt) v = v > 0.f ? v / rp : v * rp;
    if (cnt > 0) v -= fp * (float)cnt + pp;
    row[i] = from_f<T>(v);
  }
}

// After a decode iteration: feed the sampled token back and move every sequence one position on.
__global__ void advance_step_kernel(int64_t* __restrict__ input_ids, int64_t* __restrict__ positions,
                                    int* __restrict__ seq_lens, int64_t* __restrict__ slot_mapping,
                                    const int64_t* __restrict__ sampled, const int* __restrict__ block_table,
                                    int max_blocks, int block_size, int batch, int64_t* __restrict__ token_log,
                                    int log_col, int log_stride) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int64_t tok = sampled[b];
  input_ids[b] = tok;
  if (token_log) token_log[(int64_t)b * log_stride + log_col] = tok;
  const int64_t pos = positions[b] + 1;
  positions[b] = pos;
  seq_lens[b] = (int)pos + 1;
  const int blk = block_table[(int64_t)b * max_blocks + (int)(pos / block_size)];
  slot_mapping[b] = (int64_t)blk * block_size + (pos % block_size);
}

template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table, const int64_t* __restrict__ ids,
                                 int hidden, int64_t vocab, int64_t vocab_start) {
  const int64_t t = blockIdx.x;
  const int64_t id = ids[t] - vocab_start;
  const bool ok = id >= 0 && id < vocab;
  const uint4* src = reinterpret_cast<const uint4*>(table + (ok ? id : 0) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) dst[v] = ok ? src[v] : make_uint4(0, 0, 0, 0);
}

void argmax(int64_t* out, const void* logits, int rows, int vocab, int64_t stride, int dtype, cudaStream_t stream) {
  if (rows <= 0) return;
  int splits = 1;
  if (rows <= kArgmaxScratchRows && rows < 296) {
    splits = (592 + rows - 1) / rows;
    if (splits > kArgmaxMaxSplits) splits = kArgmaxMaxSplits;
    while (splits > 1 && vocab / splits < 4096) --splits;
  }
  const dim3 grid(rows, splits);
  if (dtype == 0) argmax_kernel<__nv_bfloat16><<<grid, 512, 0, stream>>>(out, (const __nv_bfloat16*)logits, vocab, stride, splits);
  else if (dtype == 1) argmax_kernel<__half><<<grid, 512, 0, stream>>>(out, (const __half*)logits, vocab, stride, splits);
  else argmax_kernel<float><<<grid, 512, 0, stream>>>(out, (const float*)logits, vocab, stride, splits);
}

void sample(int64_t* out, const void* logits, int rows, int vocab, int64_t stride, const float* temperature,
            const int* top_k, const float* top_p, const float* min_p, const float* uniform, int dtype,
            cudaStream_t stream) {
  if (rows <= 0) return;
  if (dtype == 0)
    sample_kernel<__nv_bfloat16><<<rows, 1024, 0, stream>>>(out, (const __nv_bfloat16*)logits, vocab, stride,
                                                            temperature, top_k, top_p, min_p, uniform);
  else if (dtype == 1)
    sample_kernel<__half><<<rows, 1024, 0, stream>>>(out, (const __half*)logits, vocab, stride, temperature, top_k,
                                                     top_p, min_p, uniform);
  else
    sample_kernel<float><<<rows, 1024, 0, stream>>>(out, (const float*)logits, vocab, stride, temperature, top_k,
                                                    top_p, min_p, uniform);
}

void apply_penalties(void* logits, const int* prompt_mask, const int* output_counts, const float* rep,
                     const float* presence, const float* frequency, int rows, int vocab, int64_t stride, int dtype,
                     cudaStream_t stream) {
  if (rows <= 0) return;
  dim3 grid(ceil_div(vocab, 256 * 4), rows);
  if (dtype == 0)
    penalties_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)logits, prompt_mask, output_counts, rep,
                                                              presence, frequency, vocab, stride);
  else if (dtype == 1)
    penalties_kernel<__half><<<grid, 256, 0, stream>>>((__half*)logits, prompt_mask, output_counts, rep, presence,
                                                       frequency, vocab, stride);
  else
    penalties_kernel<float><<<grid, 256, 0, stream>>>((float*)logits, prompt_mask, output_counts, rep, presence,
                                                      frequency, vocab, stride);
}

void advance_step(int64_t* input_ids, int64_t* positions, int* seq_lens, int64_t* slot_mapping, const int64_t* sampled,
                  const int* block_table, int max_blocks, int block_size, int batch, int64_t* token_log, int log_col,
                  int log_stride, cudaStream_t stream) {
  if (batch <= 0) return;
  advance_step_kernel<<<ceil_div(batch, 128), 128, 0, stream>>>(input_ids, positions, seq_lens, slot_mapping, sampled,
                                                                block_table, max_blocks, block_size, batch, token_log,
                                                                log_col, log_stride);
}

void embedding(void* out, const void* table, const int64_t* ids, int tokens, int hidden, int64_t vocab,
               int64_t vocab_start, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = hidden / 8 < 256 ? (hidden / 8 < 32 ? 32 : hidden / 8) : 256;
  if (dtype == 0)
    embedding_kernel<__nv_bfloat16><<<tokens, th, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids,
                                                               hidden, vocab, vocab_start);
  else
    embedding_kernel<__half><<<tokens, th, 0, stream>>>((__half*)out, (const __half*)table, ids, hidden, vocab,
                                                        vocab_start);
}

}  // namespace b200
