// Mixture-of-experts routing and token shuffling.
//   topk_gating        softmax | sigmoid | sqrt(softplus) scores (+ selection bias), top-k,
//                      renormalise, scale - one warp per token, any expert count <= 1024
//   grouped_topk       DeepSeek group-limited routing: per-group top-2 sum (or max), keep
//                      topk_group groups, top-k experts inside them
//   moe_align          (token, k) pairs -> expert-contiguous order padded to `block` rows per
//                      expert: sorted_token_ids, expert id per row block, padded total
//   moe_gather         A_perm[i] = x[sorted_token_ids[i] / topk] (zero rows for padding)
//   moe_combine        out[t] = sum_k w[t,k] * Y[position of (t,k)]  (+ optional shared-expert add)
//   moe_sum            out[t] = sum_k in[t,k,:]
// Parity: csrc/moe/topk_softmax_kernels.cu:80-560, topk_softplus_sqrt_kernels.cu:90,
// grouped_topk_kernels.cu:547, moe_align_sum_kernels.cu:25-369 of the reference.
#include "common.cuh"

namespace b200 {

constexpr int kMaxExpertsPerLane = 32;  // 32 lanes x 32 = 1024 experts

__device__ __forceinline__ float score_of(int mode, float x) {
  if (mode == 1) return 1.f / (1.f + __expf(-x));                       // sigmoid
  if (mode == 2) return sqrtf(x > 20.f ? x : log1pf(__expf(x)));        // sqrt(softplus)
  return x;                                                             // softmax handled by caller
}

// mode: 0 softmax, 1 sigmoid, 2 sqrt-softplus.  One warp per token.
template <typename T>
__global__ void topk_gating_kernel(float* __restrict__ weights, int* __restrict__ ids, const T* __restrict__ gating,
                                   const float* __restrict__ bias, int tokens, int experts, int topk, int mode,
                                   int renorm, float scale) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const T* g = gating + (size_t)t * experts;
  float sc[kMaxExpertsPerLane];   // scores of experts lane, lane+32, ...
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxExpertsPerLane; ++j) {
    const int e = lane + 32 * j;
    sc[j] = e < experts ? to_f(g[e]) : -INFINITY;
    mx = fmaxf(mx, sc[j]);
  }
  if (mode == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j) {
      const int e = lane + 32 * j;
      sc[j] = e < experts ? __expf(sc[j] - mx) : 0.f;
      sum += sc[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j) sc[j] *= inv;
  } else {
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j) {
      const int e = lane + 32 * j;
      sc[j] = e < experts ? score_of(mode, sc[j]) : 0.f;
    }
  }
  // selection value = score (+ bias); picked experts are marked by -inf in sel
  float sel[kMaxExpertsPerLane];
#pragma unroll
  for (int j = 0; j < kMaxExpertsPerLane; ++j) {
    const int e = lane + 32 * j;
    sel[j] = e < experts ? sc[j] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < topk; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j) {
      const int e = lane + 32 * j;
      if (sel[j] > bv) { bv = sel[j]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    // owner lane fetches the un-biased score and retires the expert
    float w = 0.f;
    if ((be & 31) == lane) {
#pragma unroll
      for (int j = 0; j < kMaxExpertsPerLane; ++j)
        if (j == (be >> 5)) { w = sc[j]; sel[j] = -INFINITY; }
    }
    w = __shfl_sync(0xffffffffu, w, be & 31);
    wsum += w;
    if (lane == k) { my_w = w; my_id = be; }
  }
  const float mul = (renorm ? 1.f / fmaxf(wsum, 1e-20f) : 1.f) * scale;
  if (lane < topk) {
    weights[(size_t)t * topk + lane] = my_w * mul;
    ids[(size_t)t * topk + lane] = my_id;
  }
}

// DeepSeek grouped top-k, one warp per token; experts <= 1024, groups <= 32, topk <= 32.
template <typename T>
__global__ void grouped_topk_kernel(float* __restrict__ weights, int* __restrict__ ids, const T* __restrict__ gating,
                                    const float* __restrict__ bias, int tokens, int experts, int topk, int n_group,
                                    int topk_group, int sigmoid, int renorm, float scale) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  extern __shared__ float smem_f[];
  const int wib = threadIdx.x >> 5;
  float* sc = smem_f + (size_t)wib * (2 * experts + 32);   // scores
  float* sel = sc + experts;                                // selection values
  float* gsc = sel + experts;                               // group scores [<=32]
  const T* g = gating + (size_t)t * experts;
  float mx = -INFINITY;
  for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, to_f(g[e]));
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) {
    const float x = to_f(g[e]);
    const float s = sigmoid ? 1.f / (1.f + __expf(-x)) : __expf(x - mx);
    sc[e] = s;
    sum += s;
  }
  sum = warp_sum(sum);
  if (!sigmoid) {
    const float inv = 1.f / sum;
    for (int e = lane; e < experts; e += 32) sc[e] *= inv;
  }
  __syncwarp();
  for (int e = lane; e < experts; e += 32) sel[e] = sc[e] + (bias ? bias[e] : 0.f);
  __syncwarp();
  const int per = experts / n_group;
  // group score: lane = group
  if (lane < n_group) {
    float a = -INFINITY, b = -INFINITY;
    for (int i = 0; i < per; ++i) {
      const float v = sel[lane * per + i];
      if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
    }
    gsc[lane] = bias ? a + b : a;
  }
  __syncwarp();
  // keep the topk_group best groups: rank of my group = number of strictly better (or equal, lower id) groups
  bool keep = false;
  if (lane < n_group) {
    int better = 0;
    for (int j = 0; j < n_group; ++j)
      if (gsc[j] > gsc[lane] || (gsc[j] == gsc[lane] && j < lane)) ++better;
    keep = better < topk_group;
  }
  const unsigned keep_mask = __ballot_sync(0xffffffffu, keep);
  for (int e = lane; e < experts; e += 32)
    if (!((keep_mask >> (e / per)) & 1u)) sel[e] = -INFINITY;
  __syncwarp();
  float wsum = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < topk; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < experts; e += 32)
      if (sel[e] > bv) { bv = sel[e]; be = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    if (be == 0x7fffffff) be = 0;
    const float w = sc[be];
    __syncwarp();
    if (lane == 0) sel[be] = -INFINITY;
    __syncwarp();
    wsum += w;
    if (lane == k) { my_w = w; my_id = be; }
  }
  const float mul = (renorm ? 1.f / fmaxf(wsum, 1e-20f) : 1.f) * scale;
  if (lane < topk) {
    weights[(size_t)t * topk + lane] = my_w * mul;
    ids[(size_t)t * topk + lane] = my_id;
  }
}

// ---------------------------------------------------------------- align
// Single CTA (1024 threads = 32 warps): warp w owns the w-th contiguous segment of the (token, k) pairs.
//   1. per-warp histograms in shared memory            hist[w][e]
//   2. per expert: exclusive prefix over the warps, then the padded expert starts
//   3. each warp walks its segment 32 pairs at a time; lanes that hold the same expert find each other with
//      match.any, so the placement is stable (pair order is kept inside an expert) and every pair is read twice.
// numel = tokens * topk.  expert_map (optional): global expert id -> local id or -1 (pairs routed elsewhere are
// dropped and get inv_pos = -1).
constexpr int kAlignWarps = 32;

__device__ __forceinline__ int align_expert_of(const int* __restrict__ topk_ids, const int* __restrict__ expert_map,
                                               int i, int numel, int experts) {
  if (i >= numel) return -1;
  int e = topk_ids[i];
  if (expert_map) e = (e >= 0) ? expert_map[e] : -1;
  return (e >= 0 && e < experts) ? e : -1;
}

__global__ void __launch_bounds__(kAlignWarps * 32)
moe_align_kernel(int* __restrict__ sorted_ids, int* __restrict__ block_expert, int* __restrict__ total_padded,
                 int* __restrict__ inv_pos, const int* __restrict__ topk_ids, const int* __restrict__ expert_map,
                 int numel, int experts, int block, int max_padded) {
  extern __shared__ int sm[];
  int* hist = sm;                                   // [kAlignWarps][experts] counts, then write cursors
  int* starts = sm + kAlignWarps * experts;         // [experts + 1] padded starts
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = ((numel + kAlignWarps - 1) / kAlignWarps + 127) / 128 * 128;   // pairs per warp, 4 x 32 per trip
  const int lo = warp * seg, hi = min(numel, lo + seg);
  for (int i = threadIdx.x; i < kAlignWarps * experts; i += blockDim.x) hist[i] = 0;
  // padding marker everywhere first; real pairs overwrite it in step 3
  for (int i = threadIdx.x; i < max_padded; i += blockDim.x) sorted_ids[i] = numel;
  for (int b = threadIdx.x; b < max_padded / block; b += blockDim.x) block_expert[b] = -1;
  __syncthreads();
  int* mine = hist + warp * experts;
  for (int i0 = lo; i0 < hi; i0 += 128) {
    int e[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) e[j] = align_expert_of(topk_ids, expert_map, i0 + j * 32 + lane, hi, experts);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (e[j] >= 0) atomicAdd(&mine[e[j]], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {      // exclusive prefix over the warps, per expert
    int acc = 0;
    for (int w = 0; w < kAlignWarps; ++w) {
      const int c = hist[w * experts + e];
      hist[w * experts + e] = acc;
      acc += c;
    }
    starts[e + 1] = (acc + block - 1) / block * block;           // padded count for now
  }
  __syncthreads();
  if (warp == 0) {                                               // inclusive scan of the padded counts
    int carry = 0;
    for (int e0 = 0; e0 < experts; e0 += 32) {
      const int e = e0 + lane;
      int v = (e < experts) ? starts[e + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += o;
      }
      if (e < experts) starts[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) { starts[0] = 0; *total_padded = carry; }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    for (int b = starts[e] / block; b < starts[e + 1] / block; ++b) block_expert[b] = e;
    const int s0 = starts[e];
    for (int w = 0; w < kAlignWarps; ++w) hist[w * experts + e] += s0;
  }
  __syncthreads();
  for (int i0 = lo; i0 < hi; i0 += 128) {
    int e[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) e[j] = align_expert_of(topk_ids, expert_map, i0 + j * 32 + lane, hi, experts);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i0 + j * 32 + lane;
      const unsigned peers = __match_any_sync(0xffffffffu, e[j]);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      if (e[j] >= 0) {
        const int pos = mine[e[j]] + rank;
        sorted_ids[pos] = i;
        if (inv_pos) inv_pos[i] = pos;
      } else if (inv_pos && i < hi) {
        inv_pos[i] = -1;
      }
      __syncwarp();
      if (e[j] >= 0 && rank == 0) mine[e[j]] += __popc(peers);
      __syncwarp();
    }
  }
}

template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ sorted_ids,
                                  const int* __restrict__ total_padded, int numel, int topk, int hidden) {
  const int row = blockIdx.x;
  if (row >= *total_padded) return;
  const int id = sorted_ids[row];
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * hidden);
  if (id >= numel) {
    for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(id / topk) * hidden);
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) dst[v] = src[v];
}

// out[t] = sum_k w[t,k] * y[inv_pos[t*topk+k]]  (+ shared[t]); pairs with inv_pos < 0 are skipped.
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ y, const float* __restrict__ weights,
                                   const int* __restrict__ inv_pos, const T* __restrict__ shared, int topk,
                                   int hidden) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (shared) unpack8<T>(reinterpret_cast<const uint4*>(shared + (size_t)t * hidden)[v], acc);
    for (int k = 0; k < topk; ++k) {
      const int pos = inv_pos[(size_t)t * topk + k];
      if (pos < 0) continue;
      const float w = weights[(size_t)t * topk + k];
      float f[8];
      unpack8<T>(reinterpret_cast<const uint4*>(y + (size_t)pos * hidden)[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += w * f[i];
    }
    reinterpret_cast<uint4*>(out + (size_t)t * hidden)[v] = pack8<T>(acc);
  }
}

template <typename T>
__global__ void moe_sum_kernel(T* __restrict__ out, const T* __restrict__ in, int topk, int hidden) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < topk; ++k) a += to_f(in[((size_t)t * topk + k) * hidden + i]);
    out[(size_t)t * hidden + i] = from_f<T>(a);
  }
}

// ---------------------------------------------------------------- launchers
#define DISPATCH_16(dtype, CALL_BF16, CALL_F16, CALL_F32) \
  if (dtype == 0) { CALL_BF16; } else if (dtype == 1) { CALL_F16; } else { CALL_F32; }

void topk_gating(float* weights, int* ids, const void* gating, const float* bias, int tokens, int experts, int topk,
                 int mode, int renorm, float scale, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = 128, blocks = ceil_div(tokens * 32, th);
  DISPATCH_16(dtype,
              (topk_gating_kernel<__nv_bfloat16><<<blocks, th, 0, stream>>>(weights, ids, (const __nv_bfloat16*)gating, bias, tokens, experts, topk, mode, renorm, scale)),
              (topk_gating_kernel<__half><<<blocks, th, 0, stream>>>(weights, ids, (const __half*)gating, bias, tokens, experts, topk, mode, renorm, scale)),
              (topk_gating_kernel<float><<<blocks, th, 0, stream>>>(weights, ids, (const float*)gating, bias, tokens, experts, topk, mode, renorm, scale)))
}

void grouped_topk(float* weights, int* ids, const void* gating, const float* bias, int tokens, int experts, int topk,
                  int n_group, int topk_group, int sigmoid, int renorm, float scale, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = 128, blocks = ceil_div(tokens * 32, th);
  const size_t sm = (size_t)(th / 32) * (2 * experts + 32) * sizeof(float);
  DISPATCH_16(dtype,
              (grouped_topk_kernel<__nv_bfloat16><<<blocks, th, sm, stream>>>(weights, ids, (const __nv_bfloat16*)gating, bias, tokens, experts, topk, n_group, topk_group, sigmoid, renorm, scale)),
              (grouped_topk_kernel<__half><<<blocks, th, sm, stream>>>(weights, ids, (const __half*)gating, bias, tokens, experts, topk, n_group, topk_group, sigmoid, renorm, scale)),
              (grouped_topk_kernel<float><<<blocks, th, sm, stream>>>(weights, ids, (const float*)gating, bias, tokens, experts, topk, n_group, topk_group, sigmoid, renorm, scale)))
}

void moe_align(int* sorted_ids, int* block_expert, int* total_padded, int* inv_pos, const int* topk_ids,
               const int* expert_map, int numel, int experts, int block, int max_padded, cudaStream_t stream) {
  const size_t sm = (size_t)(kAlignWarps * experts + experts + 1) * sizeof(int);
  if (sm > 48 * 1024) cudaFuncSetAttribute(moe_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  moe_align_kernel<<<1, kAlignWarps * 32, sm, stream>>>(sorted_ids, block_expert, total_padded, inv_pos, topk_ids, expert_map,
                                            numel, experts, block, max_padded);
}

void moe_gather(void* out, const void* x, const int* sorted_ids, const int* total_padded, int max_padded, int numel,
                int topk, int hidden, int dtype, cudaStream_t stream) {
  if (max_padded <= 0) return;
  const int th = hidden / 8 < 256 ? (hidden / 8 < 32 ? 32 : hidden / 8) : 256;
  if (dtype == 0)
    moe_gather_kernel<__nv_bfloat16><<<max_padded, th, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, sorted_ids, total_padded, numel, topk, hidden);
  else
    moe_gather_kernel<__half><<<max_padded, th, 0, stream>>>((__half*)out, (const __half*)x, sorted_ids, total_padded, numel, topk, hidden);
}

void moe_combine(void* out, const void* y, const float* weights, const int* inv_pos, const void* shared, int tokens,
                 int topk, int hidden, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = hidden / 8 < 256 ? (hidden / 8 < 32 ? 32 : hidden / 8) : 256;
  if (dtype == 0)
    moe_combine_kernel<__nv_bfloat16><<<tokens, th, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)y, weights, inv_pos, (const __nv_bfloat16*)shared, topk, hidden);
  else
    moe_combine_kernel<__half><<<tokens, th, 0, stream>>>((__half*)out, (const __half*)y, weights, inv_pos, (const __half*)shared, topk, hidden);
}

void moe_sum(void* out, const void* in, int tokens, int topk, int hidden, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int th = hidden < 1024 ? ((hidden + 31) / 32 * 32) : 1024;
  if (dtype == 0)
    moe_sum_kernel<__nv_bfloat16><<<tokens, th, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, topk, hidden);
  else
    moe_sum_kernel<__half><<<tokens, th, 0, stream>>>((__half*)out, (const __half*)in, topk, hidden);
}

}  // namespace b200
