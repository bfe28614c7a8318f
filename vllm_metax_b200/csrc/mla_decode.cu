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
// One CTA = one query token x 16 / 32 / 64 heads x one KV split; 8 warps walk 64-token latent tiles through a
// two-slot cp.async ring (see the kernel's comment for the division of work).  The latent rows of a token are
// read once per CTA, so the more heads a CTA covers the less cache traffic; with 16 heads per rank (TP 8 of 128
// heads) the kernel is a stream over the cache like GQA decode.
// Replaces flash_mla_with_kvcache / flash_mla_sparse_fwd / the Triton split-KV MLA decode
// (vllm_metax/v1/attention/backends/mla/flashmla.py:339-349, flashmla_sparse.py:973-1084,
// ops/triton_decode_attention.py:72-825).
#include "common.cuh"
#include "ops.h"

namespace b200 {

constexpr int kMlaD = 576, kMlaDV = 512;
constexpr int kMlaRowBytes = kMlaD * 2;          // 1152
constexpr int kMlaCPR = kMlaRowBytes / 16;       // 72 chunks per row
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

constexpr int kMlaTok = 64;                       // latent rows per tile
constexpr int kMlaThreads = 256;                  // 8 warps: warp w owns tile tokens [8w, 8w+8) and output columns [64w, 64w+64)
constexpr int kMlaTileB = kMlaTok * kMlaRowBytes; // 72 KB

// Shared-memory plan for MT m16 row tiles (16 * MT heads per CTA).
template <int MT, bool FP8>
struct MlaSmem2 {
  static constexpr int kQ = 0;                                        // 16 MT x 1152, swizzled
  static constexpr int kQBytes = 16 * MT * kMlaRowBytes;
  static constexpr int kRawStage = kMlaTok * kMlaRecBytes;            // fp8 records of one tile
  static constexpr int kRing = kQ + kQBytes;                          // 2 stages: bf16 tiles, or raw records when FP8
  static constexpr int kRingBytes = 2 * (FP8 ? kRawStage : kMlaTileB);
  static constexpr int kConv = kRing + kRingBytes;                    // FP8: the dequantised tile
  static constexpr int kConvBytes = FP8 ? kMlaTileB : 0;
  static constexpr int kP = kConv + kConvBytes;                       // 16 MT rows x 64 tokens, 16-bit, swizzled
  static constexpr int kPBytes = 16 * MT * kMlaTok * 2;
  static constexpr int kMax = kP + kPBytes;                           // [8 warps][16 MT] row maxima, later row sums
  static constexpr int kMaxBytes = 8 * 16 * MT * 4;
  static constexpr int kPos = kMax + kMaxBytes;                       // [2][64] cache row of every tile row, -1 = masked
  static constexpr int kTotal = kPos + 2 * kMlaTok * 4 + 16;
};

// One CTA = one query token x 16 MT heads x one KV split.  Per 64-token tile: every warp multiplies ALL of the CTA's
// rows with ITS 8 tokens over the full 576-wide contraction (no cross-warp reduction of partial scores), the row
// maxima are exchanged through shared memory, P goes to shared memory once, and every warp multiplies P into ITS 64
// of the 512 value columns - the value operand is the first 512 columns of the very tile that served as K
// (ldmatrix.trans).  Four CTA barriers per 64 tokens; the latent rows of a token are read once per 16 MT heads.
template <typename T, bool FP8, int MT>
__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_kernel(const MlaDecodeParams p) {
  using S = MlaSmem2<MT, FP8>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_seq, s_lim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int h0 = blockIdx.x * 16 * MT;
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
  const int tiles_total = (n_entries + kMlaTok - 1) / kMlaTok;
  const int tiles_per_split = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + tiles_per_split);
  const int* btab = p.block_table + (int64_t)seq * p.max_blocks;
  const int* idx_row = p.topk_indices ? p.topk_indices + (int64_t)t * p.topk : nullptr;
  uint8_t* q_smem = smem + S::kQ;
  uint8_t* p_smem = smem + S::kP;
  float* s_max = reinterpret_cast<float*>(smem + S::kMax);
  int* s_pos = reinterpret_cast<int*>(smem + S::kPos);
  const long long kv_cap = (long long)p.max_blocks * p.block_size;

  // ---- Q rows (heads h0 .. h0 + 16 MT - 1 of token t), swizzled; rows beyond the head count are zero
  {
    const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)t * p.q_stride;
    for (int i = threadIdx.x; i < 16 * MT * kMlaCPR; i += blockDim.x) {
      const int r = i / kMlaCPR, c = i % kMlaCPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h0 + r < p.num_heads) v = *reinterpret_cast<const uint4*>(qb + (int64_t)(h0 + r) * kMlaD + c * 8);
      *reinterpret_cast<uint4*>(q_smem + r * kMlaRowBytes + ((c ^ (r & 7)) * 16)) = v;
    }
  }

  // cache position of entry e of the kv list, or -1 (beyond the list, masked by causality, or a bad index)
  auto pos_of = [&](int e) -> int {
    if (e >= n_entries) return -1;
    int v = e;
    if (idx_row) v = idx_row[e];
    return (v >= 0 && v < lim && v < kv_cap) ? v : -1;
  };
  // cache rows (page * block_size + offset, or -1) of the entries of tile `tile` into s_pos[slot] (threads 0..63:
  // one page-table lookup per row); after a barrier issue_rows copies the rows 16 bytes at a time
  auto stage_positions = [&](int tile, int slot) {
    if (threadIdx.x < kMlaTok) {
      const int pos = tile < tile_end ? pos_of(tile * kMlaTok + threadIdx.x) : -1;
      int row = -1;
      if (pos >= 0) {
        const int page = btab[pos / p.block_size];
        if (page < 0 || page >= p.num_blocks) report_status(p.status, kBadIndex, 95, (int)p.num_blocks, page);
        else row = page * p.block_size + pos % p.block_size;
      }
      s_pos[slot * kMlaTok + threadIdx.x] = row;
    }
  };
  auto issue_rows = [&](int tile, int slot) {
    if (tile >= tile_end) return;
    const uint8_t* cache = reinterpret_cast<const uint8_t*>(p.cache);
    constexpr int CH = FP8 ? 41 : kMlaCPR;                   // 16-byte chunks per stored row
    constexpr int RB = FP8 ? kMlaRecBytes : kMlaRowBytes;
    uint8_t* dst = smem + S::kRing + slot * (FP8 ? S::kRawStage : kMlaTileB);
    for (int i = threadIdx.x; i < kMlaTok * CH; i += blockDim.x) {
      const int r = i / CH, c = i % CH;
      const int row = s_pos[slot * kMlaTok + r];
      const int dc = FP8 ? c : (c ^ (r & 7));
      mla_cp16(dst + r * RB + dc * 16, cache + (row >= 0 ? (int64_t)row * RB + c * 16 : 0), row >= 0);
    }
  };

  const float sl2 = p.scale * 1.4426950408889634f;
  float m_run[MT][2], l_run[MT][2];
  float o[MT][8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
  }

  stage_positions(tile_begin, 0);
  __syncthreads();
  issue_rows(tile_begin, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  int slot = 0;
  for (int tile = tile_begin; tile < tile_end; ++tile, slot ^= 1) {
    stage_positions(tile + 1, slot ^ 1);
    __syncthreads();                       // positions visible; the other slot and P / s_max are free again
    issue_rows(tile + 1, slot ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const uint8_t* kt = smem + S::kRing + slot * kMlaTileB;
    if (FP8) {
      // dequantise the 64 records of this slot into the swizzled 16-bit tile
      const uint8_t* raw = smem + S::kRing + slot * S::kRawStage;
      uint8_t* conv = smem + S::kConv;
      for (int i = threadIdx.x; i < kMlaTok * kMlaCPR; i += blockDim.x) {
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
        *reinterpret_cast<uint4*>(conv + r * kMlaRowBytes + ((c ^ (r & 7)) * 16)) = outv;
      }
      __syncthreads();
      kt = conv;
    }
    // ---- S[rows, my 8 tokens] over the whole contraction: 18 pairs of k-steps
    // (two accumulator chains per row tile - even / odd k-steps - so consecutive MMAs do not wait on each other)
    float sc[MT][4], sc2[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      sc[mt][0] = sc[mt][1] = sc[mt][2] = sc[mt][3] = 0.f;
      sc2[mt][0] = sc2[mt][1] = sc2[mt][2] = sc2[mt][3] = 0.f;
    }
    {
      const int mat = lane >> 3;
      const int kr = warp * 8 + (lane & 7);                  // my token row of the tile
#pragma unroll 2
      for (int kp = 0; kp < 18; ++kp) {
        uint32_t kf[4];
        {
          const int c = 4 * kp + mat;                         // chunks 4kp .. 4kp+3 = two k-steps
          mla_ldm(kf, kt + kr * kMlaRowBytes + ((c ^ (kr & 7)) * 16));
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int ks = 2 * kp + half;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            uint32_t qf[4];
            const int r = mt * 16 + (mat & 1) * 8 + (lane & 7), c = 2 * ks + (mat >> 1);
            mla_ldm(qf, q_smem + r * kMlaRowBytes + ((c ^ (r & 7)) * 16));
            if (half == 0) mla_mma<T>(sc[mt], qf, kf[0], kf[1]);
            else mla_mma<T>(sc2[mt], qf, kf[2], kf[3]);
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[mt][e] += sc2[mt][e];
    }
    // ---- mask, row maxima of my 8 tokens -> shared memory
    const int ra = lane >> 2, c0 = 2 * (lane & 3);
    const bool ok0 = s_pos[slot * kMlaTok + warp * 8 + c0] >= 0, ok1 = s_pos[slot * kMlaTok + warp * 8 + c0 + 1] >= 0;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      sc[mt][0] = ok0 ? sc[mt][0] * sl2 : -INFINITY;
      sc[mt][1] = ok1 ? sc[mt][1] * sl2 : -INFINITY;
      sc[mt][2] = ok0 ? sc[mt][2] * sl2 : -INFINITY;
      sc[mt][3] = ok1 ? sc[mt][3] * sl2 : -INFINITY;
      float ma = fmaxf(sc[mt][0], sc[mt][1]), mb = fmaxf(sc[mt][2], sc[mt][3]);
      ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 1));
      ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 2));
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
      if ((lane & 3) == 0) {
        s_max[warp * 16 * MT + mt * 16 + ra] = ma;
        s_max[warp * 16 * MT + mt * 16 + ra + 8] = mb;
      }
    }
    __syncthreads();
    // ---- online softmax with the tile-wide maximum; P (16-bit) -> shared memory
    float corr[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; ++w) mx = fmaxf(mx, s_max[w * 16 * MT + mt * 16 + ra + 8 * h]);
        const float mnew = fmaxf(m_run[mt][h], mx);
        const float msafe = (mnew == -INFINITY) ? 0.f : mnew;
        corr[mt][h] = exp2f(m_run[mt][h] - msafe);
        m_run[mt][h] = mnew;
        const float p0 = exp2f(sc[mt][2 * h] - msafe), p1 = exp2f(sc[mt][2 * h + 1] - msafe);
        l_run[mt][h] = l_run[mt][h] * corr[mt][h] + p0 + p1;   // this thread's tokens only; summed at the end
        const int r = mt * 16 + ra + 8 * h;
        // row r, tokens 8 warp + c0, c0 + 1: 16-byte chunk `warp` of the row, swizzled
        *reinterpret_cast<uint32_t*>(p_smem + r * (kMlaTok * 2) + ((warp ^ (r & 7)) * 16) + c0 * 2) = mla_pack2<T>(p0, p1);
      }
    }
    __syncthreads();
    // ---- O[:, 64 warp .. 64 warp + 64) = O * corr + P . V  (4 k-steps of 16 tokens)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nd = 0; nd < 8; ++nd) {
        o[mt][nd][0] *= corr[mt][0]; o[mt][nd][1] *= corr[mt][0];
        o[mt][nd][2] *= corr[mt][1]; o[mt][nd][3] *= corr[mt][1];
      }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pf[MT][4];
      const int mat = lane >> 3;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int r = mt * 16 + (mat & 1) * 8 + (lane & 7), c = 2 * kk + (mat >> 1);
        mla_ldm(pf[mt], p_smem + r * (kMlaTok * 2) + ((c ^ (r & 7)) * 16));
      }
#pragma unroll
      for (int nd = 0; nd < 8; nd += 2) {
        uint32_t vf[4];
        const int r = kk * 16 + (mat & 1) * 8 + (lane & 7);
        const int c = warp * 8 + nd + (mat >> 1);
        mla_ldm_t(vf, kt + r * kMlaRowBytes + ((c ^ (r & 7)) * 16));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mla_mma<T>(o[mt][nd], pf[mt], vf[0], vf[1]);
          mla_mma<T>(o[mt][nd + 1], pf[mt], vf[2], vf[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- row sums over the 8 warps (quad first), then the normalised output or the split partials
  __syncthreads();
  const int ra = lane >> 2;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float l = l_run[mt][h];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if ((lane & 3) == 0) s_max[warp * 16 * MT + mt * 16 + ra + 8 * h] = l;
    }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mt * 16 + ra + half * 8;
      const int h = h0 + r;
      if (h >= p.num_heads) continue;
      float L = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) L += s_max[w * 16 * MT + r];
      const float Ms = (m_run[mt][half] == -INFINITY) ? 0.f : m_run[mt][half];
      const float inv = L > 0.f ? 1.f / L : 0.f;
      const float lse = L > 0.f ? Ms * 0.6931471805599453f + logf(L) : -INFINITY;
      if (p.num_splits == 1) {
        T* dst = reinterpret_cast<T*>(p.out) + ((int64_t)t * p.num_heads + h) * kMlaDV + warp * 64;
#pragma unroll
        for (int nd = 0; nd < 8; ++nd) {
          const int col = nd * 8 + 2 * (lane & 3);
          *reinterpret_cast<uint32_t*>(dst + col) =
              mla_pack2<T>(o[mt][nd][half * 2] * inv, o[mt][nd][half * 2 + 1] * inv);
        }
        if (warp == 0 && (lane & 3) == 0 && p.lse_out) p.lse_out[(int64_t)h * p.total_tokens + t] = lse;
      } else {
        const int64_t prow = ((int64_t)split * p.total_tokens + t) * p.num_heads + h;
        float* dst = p.part_out + prow * kMlaDV + warp * 64;
#pragma unroll
        for (int nd = 0; nd < 8; ++nd) {
          const int col = nd * 8 + 2 * (lane & 3);
          dst[col] = o[mt][nd][half * 2] * inv;
          dst[col + 1] = o[mt][nd][half * 2 + 1] * inv;
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

template <typename T, bool FP8, int MT>
static void launch_mla_mt(const MlaDecodeParams& p, cudaStream_t stream) {
  using S = MlaSmem2<MT, FP8>;
  static_assert(S::kTotal <= 232448, "shared memory budget exceeded");
  auto kern = mla_decode_kernel<T, FP8, MT>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
  dim3 grid((p.num_heads + 16 * MT - 1) / (16 * MT), p.total_tokens, p.num_splits);
  kern<<<grid, kMlaThreads, S::kTotal, stream>>>(p);
}

// Heads per CTA: the latent rows are re-read once per 16 MT heads, so as many heads as shared memory allows.
int mla_decode_heads_per_cta(int num_heads, int fp8_records) {
  if (num_heads <= 16) return 16;
  if (num_heads <= 32 || fp8_records) return 32;
  return 64;
}

template <typename T, bool FP8>
static void launch_mla(const MlaDecodeParams& p, cudaStream_t stream) {
  const int hpc = mla_decode_heads_per_cta(p.num_heads, FP8 ? 1 : 0);
  if (hpc == 16) launch_mla_mt<T, FP8, 1>(p, stream);
  else if (hpc == 32) launch_mla_mt<T, FP8, 2>(p, stream);
  else {
    if constexpr (FP8) launch_mla_mt<T, true, 2>(p, stream);
    else launch_mla_mt<T, false, 4>(p, stream);
  }
}

template <typename T>
static void launch_mla_reduce(const MlaDecodeParams& p, cudaStream_t stream) {
  mla_split_reduce_kernel<T><<<(unsigned)((int64_t)p.total_tokens * p.num_heads), 256, 0, stream>>>(
      (T*)p.out, p.lse_out, p.part_out, p.part_lse, p.num_splits, p.total_tokens, p.num_heads);
}

int mla_decode(const MlaDecodeParams& p, int fp8_records, int dtype, cudaStream_t stream, int impl) {
  if (p.total_tokens <= 0) return 0;
  bool done = false;
  if (impl != 1 && !fp8_records && (impl == 2 || p.num_heads >= 64)) done = mla_decode_tc(p, dtype, stream) == 0;
  if (!done && impl == 2) return -1;
  if (!done) {
    if (dtype == 0) {
      if (fp8_records) launch_mla<__nv_bfloat16, true>(p, stream); else launch_mla<__nv_bfloat16, false>(p, stream);
    } else {
      if (fp8_records) launch_mla<__half, true>(p, stream); else launch_mla<__half, false>(p, stream);
    }
  }
  if (p.num_splits > 1) {
    if (dtype == 0) launch_mla_reduce<__nv_bfloat16>(p, stream); else launch_mla_reduce<__half>(p, stream);
  }
  return 0;
}

}  // namespace b200
