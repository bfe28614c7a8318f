// Absorbed multi-head latent attention (MQA over the latent KV cache), dense and sparse.
//
//   q      [T, H, 576]   (q_nope . W_UK | q_pe)
//   cache  bf16 [blocks, block_size, 576]   or   uint8 [blocks, block_size, 656] ("fp8_ds_mla":
//          512 e4m3 | 4 f32 scales, one per 128 | 64 bf16 rope)
//   out    [T, H, 512],  lse [H, T]
//
// Dense: token t of sequence b sees cache positions < seq_len - q_len + i + 1.
// Sparse (DeepSeek sparse attention): only the positions listed in topk_indices[t, :] (-1 = none).
//
// One CTA = one query token x 16 heads (one m16 MMA row tile).  The 4 warps share a 3-stage
// cp.async ring of 16-token latent tiles; for each tile the QK^T contraction (576 = 36 k-steps)
// is split four ways and summed through shared memory, every warp then runs the same online
// softmax and multiplies P into ITS 128 of the 512 value columns - the value operand is the
// first 512 columns of the very tile that served as K, read with ldmatrix.trans.
// With 16 heads per rank (TP8 of 128 heads) the kernel is HBM-bound like GQA decode.
// Replaces flash_mla_with_kvcache / flash_mla_sparse_fwd / the Triton split-KV MLA decode
// (vllm_metax/v1/attention/backends/mla/flashmla.py:339-349, flashmla_sparse.py:973-1084,
// ops/triton_decode_attention.py:72-825).
#include "common.cuh"
#include "ops.h"

namespace b200 {

constexpr int kMlaD = 576, kMlaDV = 512, kMlaTile = 16, kMlaStages = 3, kMlaWarps = 4;
constexpr int kMlaRowBytes = kMlaD * 2;          // 1152
constexpr int kMlaCPR = kMlaRowBytes / 16;       // 72 chunks per row
constexpr int kMlaTileBytes = kMlaTile * kMlaRowBytes;
constexpr int kMlaRecBytes = 656;

__device__ __forceinline__ void mla_cp16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mla_ldm(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mla_ldm_t(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
template <typename T>
__device__ __forceinline__ void mla_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mla_mma<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mla_mma<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t mla_pack2(float a, float b) {
  T lo = from_f<T>(a), hi = from_f<T>(b);
  return (uint32_t)(*reinterpret_cast<uint16_t*>(&lo)) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&hi)) << 16);
}

struct MlaSmem {
  static constexpr int kQ = 0;                                   // 16 x 1152
  static constexpr int kRing = kQ + kMlaTileBytes;               // stages x tile (bf16, swizzled)
  static constexpr int kRaw = kRing + kMlaStages * kMlaTileBytes;  // fp8 records staging: stages x 16 x 656
  static constexpr int kRawBytes = kMlaStages * kMlaTile * kMlaRecBytes;
  static constexpr int kSPart = kRaw + kRawBytes;                // 4 x 256 floats
  static constexpr int kTotal = kSPart + kMlaWarps * 256 * 4 + 64;
};

// FP8: cache rows are 656-byte records that are dequantised into the bf16 ring.
template <typename T, bool FP8>
__global__ void __launch_bounds__(kMlaWarps * 32)
mla_decode_kernel(const MlaDecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_seq, s_lim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int h0 = blockIdx.x * 16;
  const int split = blockIdx.z;
  if (threadIdx.x == 0) {
    // sequence of token t: last b with query_start_loc[b] <= t
    int lo = 0, hi = p.batch - 1;
    if (p.query_start_loc) {
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (p.query_start_loc[mid] <= t) lo = mid; else hi = mid - 1;
      }
    } else {
      lo = t;
    }
    s_seq = lo;
    const int q0 = p.query_start_loc ? p.query_start_loc[lo] : lo;
    const int q1 = p.query_start_loc ? p.query_start_loc[lo + 1] : lo + 1;
    s_lim = p.seq_lens[lo] - (q1 - q0) + (t - q0) + 1;
  }
  __syncthreads();
  const int seq = s_seq, lim = s_lim;
  const int n_entries = p.topk_indices ? p.topk : lim;     // logical kv list length
  const int tiles_total = (n_entries + kMlaTile - 1) / kMlaTile;
  const int tiles_per_split = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + tiles_per_split);
  const int* btab = p.block_table + (int64_t)seq * p.max_blocks;
  const int* idx_row = p.topk_indices ? p.topk_indices + (int64_t)t * p.topk : nullptr;
  uint8_t* q_smem = smem + MlaSmem::kQ;
  float* s_part = reinterpret_cast<float*>(smem + MlaSmem::kSPart);

  // ---- Q rows (heads h0..h0+15 of token t), swizzled
  {
    const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)t * p.q_stride;
    for (int i = threadIdx.x; i < 16 * kMlaCPR; i += blockDim.x) {
      const int r = i / kMlaCPR, c = i % kMlaCPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h0 + r < p.num_heads) v = *reinterpret_cast<const uint4*>(qb + (int64_t)(h0 + r) * kMlaD + c * 8);
      *reinterpret_cast<uint4*>(q_smem + r * kMlaRowBytes + ((c ^ (r & 7)) * 16)) = v;
    }
  }

  // position of entry e of the kv list, or -1
  auto pos_of = [&](int e) -> int {
    if (e >= n_entries) return -1;
    if (!idx_row) return e;
    const int v = idx_row[e];
    return (v >= 0 && v < lim) ? v : -1;
  };
  auto issue = [&](int tile, int stage) {
    if (tile >= tile_end) return;
    const uint8_t* cache = reinterpret_cast<const uint8_t*>(p.cache);
    if (!FP8) {
      uint8_t* dst = smem + MlaSmem::kRing + stage * kMlaTileBytes;
      for (int i = threadIdx.x; i < kMlaTile * kMlaCPR; i += blockDim.x) {
        const int r = i / kMlaCPR, c = i % kMlaCPR;
        const int pos = pos_of(tile * kMlaTile + r);
        const uint8_t* src = cache;
        if (pos >= 0) {
          int page = btab[pos / p.block_size];
          if (page < 0 || page >= p.num_blocks) { report_status(p.status, kBadIndex, 95, (int)p.num_blocks, page); page = 0; }
          src = cache + ((int64_t)page * p.block_size + pos % p.block_size) * kMlaRowBytes + c * 16;
        }
        mla_cp16(dst + r * kMlaRowBytes + ((c ^ (r & 7)) * 16), src, pos >= 0);
      }
    } else {
      uint8_t* dst = smem + MlaSmem::kRaw + stage * (kMlaTile * kMlaRecBytes);
      for (int i = threadIdx.x; i < kMlaTile * 41; i += blockDim.x) {
        const int r = i / 41, c = i % 41;
        const int pos = pos_of(tile * kMlaTile + r);
        const uint8_t* src = cache;
        if (pos >= 0) {
          int page = btab[pos / p.block_size];
          if (page < 0 || page >= p.num_blocks) { report_status(p.status, kBadIndex, 96, (int)p.num_blocks, page); page = 0; }
          src = cache + ((int64_t)page * p.block_size + pos % p.block_size) * kMlaRecBytes + c * 16;
        }
        mla_cp16(dst + r * kMlaRecBytes + c * 16, src, pos >= 0);
      }
    }
  };

  const float sl2 = p.scale * 1.4426950408889634f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

#pragma unroll
  for (int s = 0; s < kMlaStages - 1; ++s) {
    issue(tile_begin + s, s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  int stage = 0;
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    issue(tile + kMlaStages - 1, (stage + kMlaStages - 1) % kMlaStages);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group %0;" ::"n"(kMlaStages - 1) : "memory");
    __syncthreads();
    uint8_t* kt = smem + MlaSmem::kRing + stage * kMlaTileBytes;
    if (FP8) {
      // dequantise the 16 records of this stage into the swizzled bf16 tile
      const uint8_t* raw = smem + MlaSmem::kRaw + stage * (kMlaTile * kMlaRecBytes);
      for (int i = threadIdx.x; i < kMlaTile * kMlaCPR; i += blockDim.x) {
        const int r = i / kMlaCPR, c = i % kMlaCPR;
        const uint8_t* rec = raw + r * kMlaRecBytes;
        uint4 outv;
        if (c < 64) {
          const float sc = reinterpret_cast<const float*>(rec + 512)[c >> 4];
          const uint2 b8 = *reinterpret_cast<const uint2*>(rec + c * 8);
          const uint8_t* bb = reinterpret_cast<const uint8_t*>(&b8);
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = fp8_e4m3_to_float(bb[j]) * sc;
          outv = pack8<T>(f);
        } else {
          const __nv_bfloat16* pe = reinterpret_cast<const __nv_bfloat16*>(rec + 528) + (c - 64) * 8;
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(pe[j]);
          outv = pack8<T>(f);
        }
        *reinterpret_cast<uint4*>(kt + r * kMlaRowBytes + ((c ^ (r & 7)) * 16)) = outv;
      }
      __syncthreads();
    }
    // ---- partial S over this warp's 9 k-steps
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < 9; ++kk) {
      const int ks = warp * 9 + kk;
      const int mat = lane >> 3;
      uint32_t qf[4], kf[4];
      {
        const int r = (mat & 1) * 8 + (lane & 7), c = 2 * ks + (mat >> 1);
        mla_ldm(qf, q_smem + r * kMlaRowBytes + ((c ^ (r & 7)) * 16));
      }
      {
        const int r = (mat >> 1) * 8 + (lane & 7), c = 2 * ks + (mat & 1);
        mla_ldm(kf, kt + r * kMlaRowBytes + ((c ^ (r & 7)) * 16));
      }
      mla_mma<T>(s[0], qf, kf[0], kf[1]);
      mla_mma<T>(s[1], qf, kf[2], kf[3]);
    }
    {
      float* mine = s_part + warp * 256;
      const int ra = lane >> 2, c0 = 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        mine[ra * 16 + nt * 8 + c0] = s[nt][0];
        mine[ra * 16 + nt * 8 + c0 + 1] = s[nt][1];
        mine[(ra + 8) * 16 + nt * 8 + c0] = s[nt][2];
        mine[(ra + 8) * 16 + nt * 8 + c0 + 1] = s[nt][3];
      }
    }
    __syncthreads();
    {
      const int ra = lane >> 2, c0 = 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int w = 0; w < kMlaWarps; ++w) {
          const float* pw = s_part + w * 256;
          a0 += pw[ra * 16 + nt * 8 + c0];
          a1 += pw[ra * 16 + nt * 8 + c0 + 1];
          a2 += pw[(ra + 8) * 16 + nt * 8 + c0];
          a3 += pw[(ra + 8) * 16 + nt * 8 + c0 + 1];
        }
        s[nt][0] = a0; s[nt][1] = a1; s[nt][2] = a2; s[nt][3] = a3;
      }
    }
    // ---- mask + online softmax (identical in all four warps)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = nt * 8 + 2 * (lane & 3) + (e & 1);
        float v = s[nt][e] * sl2;
        if (pos_of(tile * kMlaTile + col) < 0) v = -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float corr[2], msafe[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float mnew = fmaxf(m_run[h], mx[h]);
      msafe[h] = (mnew == -INFINITY) ? 0.f : mnew;
      corr[h] = exp2f(m_run[h] - msafe[h]);
      m_run[h] = mnew;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[4];
    {
      float pv[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pv[nt][e] = exp2f(s[nt][e] - msafe[e >> 1]);
          rs[e >> 1] += pv[nt][e];
        }
      pf[0] = mla_pack2<T>(pv[0][0], pv[0][1]);
      pf[1] = mla_pack2<T>(pv[0][2], pv[0][3]);
      pf[2] = mla_pack2<T>(pv[1][0], pv[1][1]);
      pf[3] = mla_pack2<T>(pv[1][2], pv[1][3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
      l_run[h] = l_run[h] * corr[h] + rs[h];
    }
    // ---- O[:, 128w .. 128w+128) = O * corr + P . V
#pragma unroll
    for (int nd = 0; nd < 16; nd += 2) {
      o[nd][0] *= corr[0]; o[nd][1] *= corr[0]; o[nd][2] *= corr[1]; o[nd][3] *= corr[1];
      o[nd + 1][0] *= corr[0]; o[nd + 1][1] *= corr[0]; o[nd + 1][2] *= corr[1]; o[nd + 1][3] *= corr[1];
      uint32_t vf[4];
      const int mat = lane >> 3;
      const int r = (mat & 1) * 8 + (lane & 7);
      const int c = warp * 16 + nd + (mat >> 1);
      mla_ldm_t(vf, kt + r * kMlaRowBytes + ((c ^ (r & 7)) * 16));
      mla_mma<T>(o[nd], pf, vf[0], vf[1]);
      mla_mma<T>(o[nd + 1], pf, vf[2], vf[3]);
    }
    __syncthreads();   // everyone is done with this ring slot and with s_part
    stage = (stage + 1) % kMlaStages;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- write out (normalised) or the split partials
  const int ra = lane >> 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = ra + half * 8;
    const int h = h0 + r;
    if (h >= p.num_heads) continue;
    const float L = l_run[half];
    const float Ms = (m_run[half] == -INFINITY) ? 0.f : m_run[half];
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const float lse = L > 0.f ? Ms * 0.6931471805599453f + logf(L) : -INFINITY;
    if (p.num_splits == 1) {
      T* dst = reinterpret_cast<T*>(p.out) + ((int64_t)t * p.num_heads + h) * kMlaDV + warp * 128;
#pragma unroll
      for (int nd = 0; nd < 16; ++nd) {
        const int col = nd * 8 + 2 * (lane & 3);
        *reinterpret_cast<uint32_t*>(dst + col) = mla_pack2<T>(o[nd][half * 2] * inv, o[nd][half * 2 + 1] * inv);
      }
      if (warp == 0 && (lane & 3) == 0 && p.lse_out) p.lse_out[(int64_t)h * p.total_tokens + t] = lse;
    } else {
      const int64_t prow = ((int64_t)split * p.total_tokens + t) * p.num_heads + h;
      float* dst = p.part_out + prow * kMlaDV + warp * 128;
#pragma unroll
      for (int nd = 0; nd < 16; ++nd) {
        const int col = nd * 8 + 2 * (lane & 3);
        dst[col] = o[nd][half * 2] * inv;
        dst[col + 1] = o[nd][half * 2 + 1] * inv;
      }
      if (warp == 0 && (lane & 3) == 0) p.part_lse[prow] = lse;
    }
  }
}

template <typename T>
__global__ void mla_split_reduce_kernel(T* __restrict__ out, float* __restrict__ lse_out,
                                        const float* __restrict__ part_out, const float* __restrict__ part_lse,
                                        int num_splits, int total_tokens, int heads) {
  const int64_t row = blockIdx.x;
  const int64_t stride = (int64_t)total_tokens * heads;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_lse[s * stride + row]);
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < num_splits; ++s) L += __expf(part_lse[s * stride + row] - Ms);
  for (int c = threadIdx.x; c < kMlaDV; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s)
      acc += part_out[(s * stride + row) * kMlaDV + c] * __expf(part_lse[s * stride + row] - Ms);
    out[row * kMlaDV + c] = from_f<T>(L > 0.f ? acc / L : 0.f);
  }
  if (threadIdx.x == 0 && lse_out)
    lse_out[(row % heads) * (int64_t)total_tokens + row / heads] = L > 0.f ? Ms + logf(L) : -INFINITY;
}

template <typename T, bool FP8>
static void launch_mla(const MlaDecodeParams& p, cudaStream_t stream) {
  auto kern = mla_decode_kernel<T, FP8>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MlaSmem::kTotal);
  dim3 grid((p.num_heads + 15) / 16, p.total_tokens, p.num_splits);
  kern<<<grid, kMlaWarps * 32, MlaSmem::kTotal, stream>>>(p);
  if (p.num_splits > 1)
    mla_split_reduce_kernel<T><<<(unsigned)((int64_t)p.total_tokens * p.num_heads), 256, 0, stream>>>(
        (T*)p.out, p.lse_out, p.part_out, p.part_lse, p.num_splits, p.total_tokens, p.num_heads);
}

void mla_decode(const MlaDecodeParams& p, int fp8_records, int dtype, cudaStream_t stream) {
  if (p.total_tokens <= 0) return;
  if (dtype == 0) {
    if (fp8_records) launch_mla<__nv_bfloat16, true>(p, stream); else launch_mla<__nv_bfloat16, false>(p, stream);
  } else {
    if (fp8_records) launch_mla<__half, true>(p, stream); else launch_mla<__half, false>(p, stream);
  }
}

}  // namespace b200
