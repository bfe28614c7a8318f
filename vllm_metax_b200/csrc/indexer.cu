// DeepSeek-V3.2 sparse-attention indexer.
//   indexer_logits   logits[t, n] = k_scale[n] * sum_h w[t, h] * relu(q[t, h, :] . k[n, :])  for the keys of
//                    token t's own request visible to it (n < limit[t]); -inf elsewhere.  q and k are e4m3 (or int8);
//                    the products run on m16n8k16 MMAs after an exact fp8 -> bf16 widening, one warp per 16
//                    index heads, 32 keys per step read straight from the paged, block-planar key cache.
//   topk_per_row     indices of the k largest finite entries of every row (radix select: four 8-bit
//                    histogram passes narrow down the k-th key, one sweep collects), -1 padded.
// Replaces deep_gemm fp8_mqa_logits / fp8_paged_mqa_logits and the top-k kernels
// (vllm_metax/utils/deep_gemm.py:306-401, csrc/sampler.cu:545-750, persistent_topk.cuh, cooperative_topk.cuh).
#include "common.cuh"

namespace b200 {

constexpr int kIdxD = 128, kIdxKeys = 32;

__device__ __forceinline__ void idx_ldm(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void idx_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (T, key_chunks); block = 32 * (heads / 16) threads.  q [T, heads, 128] e4m3 bytes, w [T, heads] f32.
__global__ void indexer_logits_kernel(float* __restrict__ logits, int64_t logits_stride, const uint8_t* __restrict__ q,
                                      const float* __restrict__ w, const uint8_t* __restrict__ cache,
                                      const int* __restrict__ block_table, int max_blocks,
                                      const int* __restrict__ seq_lens, const int* __restrict__ query_start_loc,
                                      int batch, int heads, int block_size, int64_t num_blocks, int keys_per_cta,
                                      StatusWord* status, int kind) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_seq, s_lim;
  __shared__ float s_sum[kIdxKeys];
  __shared__ float s_scale[kIdxKeys];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    int lo = 0, hi = batch - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (query_start_loc[mid] <= t) lo = mid; else hi = mid - 1;
    }
    s_seq = lo;
    s_lim = seq_lens[lo] - (query_start_loc[lo + 1] - query_start_loc[lo]) + (t - query_start_loc[lo]) + 1;
  }
  __syncthreads();
  const int seq = s_seq, lim = s_lim;
  const int n0 = blockIdx.y * keys_per_cta;
  const int n1 = min(lim, n0 + keys_per_cta);
  float* out = logits + (int64_t)t * logits_stride;
  // columns of this CTA beyond the limit are -inf
  for (int n = max(n0, lim) + threadIdx.x; n < n0 + keys_per_cta && n < logits_stride; n += blockDim.x) out[n] = -INFINITY;
  if (n0 >= lim) return;
  // q tile: heads x 128 bf16, swizzled rows of 256 bytes
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* ks = qs + heads * kIdxD;
  const int esz = kind == 2 ? 2 : 1;                 // kind 2: bf16 queries and keys, no scales
  const uint8_t* qt = q + (int64_t)t * heads * kIdxD * esz;
  for (int i = threadIdx.x; i < heads * 16; i += blockDim.x) {
    const int r = i >> 4, c = i & 15;
    if (kind == 2) {
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(qs) + r * 256 + ((c ^ (r & 7)) * 16)) =
          *reinterpret_cast<const uint4*>(qt + r * 256 + c * 16);
      continue;
    }
    const uint2 b8 = *reinterpret_cast<const uint2*>(qt + r * kIdxD + c * 8);
    const uint8_t* bb = reinterpret_cast<const uint8_t*>(&b8);
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = kind == 1 ? (float)(int8_t)bb[j] : fp8_e4m3_to_float(bb[j]);   // both exact in bf16
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(qs) + r * 256 + ((c ^ (r & 7)) * 16)) = pack8<__nv_bfloat16>(f);
  }
  __syncthreads();
  uint32_t qf[8][4];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const int mat = lane >> 3;
    const int r = warp * 16 + (mat & 1) * 8 + (lane & 7), c = 2 * kk + (mat >> 1);
    idx_ldm(qf[kk], reinterpret_cast<uint8_t*>(qs) + r * 256 + ((c ^ (r & 7)) * 16));
  }
  const float wA = w[(int64_t)t * heads + warp * 16 + (lane >> 2)];
  const float wB = w[(int64_t)t * heads + warp * 16 + (lane >> 2) + 8];
  const int* btab = block_table + (int64_t)seq * max_blocks;
  const int64_t blk_bytes = kind == 2 ? (int64_t)block_size * kIdxD * 2 : (int64_t)block_size * (kIdxD + 4);

  for (int base = n0; base < n1; base += kIdxKeys) {
    // load + widen 32 keys
    for (int i = threadIdx.x; i < kIdxKeys * 16; i += blockDim.x) {
      const int r = i >> 4, c = i & 15;
      const int n = base + r;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
      if (n < n1) {
        int page = btab[n / block_size];
        if (page < 0 || page >= num_blocks) { report_status(status, kBadIndex, 97, (int)num_blocks, page); page = 0; }
        if (kind == 2) {
          *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(ks) + r * 256 + ((c ^ (r & 7)) * 16)) =
              *reinterpret_cast<const uint4*>(cache + page * blk_bytes + (int64_t)(n % block_size) * 256 + c * 16);
          if (c == 0) s_scale[r] = 1.f;
          continue;
        }
        const uint8_t* src = cache + page * blk_bytes + (int64_t)(n % block_size) * kIdxD + c * 8;
        const uint2 b8 = *reinterpret_cast<const uint2*>(src);
        const uint8_t* bb = reinterpret_cast<const uint8_t*>(&b8);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = kind == 1 ? (float)(int8_t)bb[j] : fp8_e4m3_to_float(bb[j]);   // both exact in bf16
        if (c == 0)
          s_scale[r] = *reinterpret_cast<const float*>(cache + page * blk_bytes + (int64_t)block_size * kIdxD +
                                                       (n % block_size) * 4);
      } else if (c == 0) {
        s_scale[r] = 0.f;
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(ks) + r * 256 + ((c ^ (r & 7)) * 16)) = pack8<__nv_bfloat16>(f);
    }
    if (threadIdx.x < kIdxKeys) s_sum[threadIdx.x] = 0.f;
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
      for (int np = 0; np < 2; ++np) {   // two n-tiles per ldmatrix.x4
        uint32_t kf[4];
        const int mat = lane >> 3;
        const int r = np * 16 + (mat >> 1) * 8 + (lane & 7), c = 2 * kk + (mat & 1);
        idx_ldm(kf, reinterpret_cast<uint8_t*>(ks) + r * 256 + ((c ^ (r & 7)) * 16));
        idx_mma(s[np * 2], qf[kk], kf[0], kf[1]);
        idx_mma(s[np * 2 + 1], qf[kk], kf[2], kf[3]);
      }
    }
    // weighted relu, summed over this warp's 16 heads, then over the warps
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float c0 = wA * fmaxf(s[nt][0], 0.f) + wB * fmaxf(s[nt][2], 0.f);
      float c1 = wA * fmaxf(s[nt][1], 0.f) + wB * fmaxf(s[nt][3], 0.f);
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        c0 += __shfl_xor_sync(0xffffffffu, c0, o);
        c1 += __shfl_xor_sync(0xffffffffu, c1, o);
      }
      if (lane < 4) {
        atomicAdd(&s_sum[nt * 8 + 2 * lane], c0);
        atomicAdd(&s_sum[nt * 8 + 2 * lane + 1], c1);
      }
    }
    __syncthreads();
    if (threadIdx.x < kIdxKeys && base + threadIdx.x < n1) out[base + threadIdx.x] = s_sum[threadIdx.x] * s_scale[threadIdx.x];
    __syncthreads();
  }
}

__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float -> larger key
}

// One CTA per row.  out[row, :k] = indices of the k largest finite values (any order), -1 padded.
__global__ void __launch_bounds__(1024)
topk_per_row_kernel(int* __restrict__ out, const float* __restrict__ x, int64_t stride, const int* __restrict__ row_len,
                    int cols, int k) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_remaining, s_count_gt, s_count_eq;
  const int row = blockIdx.x;
  const float* xr = x + (int64_t)row * stride;
  const int n = row_len ? min(cols, row_len[row]) : cols;
  int* o = out + (int64_t)row * k;
  for (int i = threadIdx.x; i < k; i += blockDim.x) o[i] = -1;
  if (threadIdx.x == 0) { s_prefix = 0; s_mask = 0; s_remaining = k; s_count_gt = 0; s_count_eq = 0; }
  __syncthreads();
  // count finite entries; if they all fit, emit them directly
  int fin = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) fin += (xr[i] > -INFINITY) ? 1 : 0;
  {
    __shared__ int s_fin;
    if (threadIdx.x == 0) s_fin = 0;
    __syncthreads();
    atomicAdd(&s_fin, fin);
    __syncthreads();
    fin = s_fin;
  }
  if (fin <= k) {
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      if (xr[i] > -INFINITY) o[atomicAdd(&s_count_gt, 1)] = i;
    return;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = xr[i];
      if (!(v > -INFINITY)) continue;
      const uint32_t key = float_key(v);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFF], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int rem = s_remaining, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= rem) break;
        rem -= hist[b];
      }
      s_remaining = rem;                       // how many to take from bucket b (and below prefix-equal)
      s_prefix = prefix | ((uint32_t)b << shift);
      s_mask = mask | (0xFFu << shift);
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;               // exact key of the k-th largest element
  const int take_eq = s_remaining;             // ties to take
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = xr[i];
    if (!(v > -INFINITY)) continue;
    const uint32_t key = float_key(v);
    if (key > kth) {
      o[atomicAdd(&s_count_gt, 1)] = i;
    } else if (key == kth) {
      const int e = atomicAdd(&s_count_eq, 1);
      if (e < take_eq) o[k - 1 - e] = i;
    }
  }
}

void indexer_logits(float* logits, int64_t logits_stride, const void* q, const float* w, const void* cache,
                    const int* block_table, int max_blocks, const int* seq_lens, const int* query_start_loc,
                    int tokens, int batch, int heads, int block_size, int64_t num_blocks, int max_len, void* status,
                    cudaStream_t stream, int kind) {
  if (tokens <= 0 || max_len <= 0) return;
  const int keys_per_cta = 1024;
  dim3 grid(tokens, ceil_div(max_len, keys_per_cta));
  const size_t sm = (size_t)(heads + kIdxKeys) * kIdxD * 2;
  indexer_logits_kernel<<<grid, 32 * (heads / 16), sm, stream>>>(
      logits, logits_stride, (const uint8_t*)q, w, (const uint8_t*)cache, block_table, max_blocks, seq_lens,
      query_start_loc, batch, heads, block_size, num_blocks, keys_per_cta, (StatusWord*)status, kind);
}

void topk_per_row(int* out, const float* x, int64_t stride, const int* row_len, int rows, int cols, int k,
                  cudaStream_t stream) {
  if (rows <= 0) return;
  topk_per_row_kernel<<<rows, 1024, 0, stream>>>(out, x, stride, row_len, cols, k);
}

}  // namespace b200
