// Absorbed multi-head latent attention decode on tcgen05, dense, 16-bit latent cache.
//
//   q      [T, H, 576]   (q_nope . W_UK | q_pe), 16-bit
//   cache  [blocks, block_size, 576], same type; block_size a multiple of 32
//   out    [T, H, 512],  lse [H, T]
//
// One CTA = one query token x 128 heads x one HALF of the 512 latent output columns x one KV split.
//
// Why halves: the output accumulator of 128 heads x 512 columns in fp32 is the whole tensor memory of an SM
// (512 columns), which leaves no room for the scores.  Two CTAs therefore each keep 256 output columns, and both
// compute the (cheap to duplicate, 576-deep) score product for all heads; the second reader of a cache tile hits L2.
// Per CTA the tensor memory holds S0 | S1 (32 fp32 columns each, double-buffered) and O (256 columns).
//
//   warp 4    TMA producer: the 128 x 576 query tile once (nine 64-wide boxes, heads beyond H are zero-filled by the
//             tensor map), then 32-token cache tiles [32 x 576] through a 2-stage ring, one box per 64-wide chunk; a
//             tile never straddles a page.
//   warp 5    MMA issuer (one thread): S_j = Q . K_j^T (36 instructions of M128 N32 K16, both operands K-major from
//             shared memory); O += P_j . V_j with P_j read from tensor memory (it overwrites the first 16 columns of
//             S_j as packed 16-bit pairs) and V_j = this CTA's 256 latent columns of the SAME shared-memory tile,
//             used in place as an MN-major operand (2 instructions of M128 N256 K16).  S_{j+1} is issued before
//             P_j . V_j so the tensor core works while the softmax of tile j runs.
//   warps 0-3 softmax, thread = head: one tcgen05.ld brings the 32 scores of the row, online softmax in the exp2
//             domain with a lazily moved maximum (the accumulator is rescaled in tensor memory only when a row
//             maximum grows by more than 2^8), P back with tcgen05.st; at the end the normalised output half (or the
//             split partial) and, from the CTA of half 0, the log-sum-exp.
//
// Cache rows past the visible length inside the last tile are multiplied by P = 0, so the cache must hold finite
// values everywhere (it is allocated zeroed).  Every wait is bounded; a wait that runs out records its site in the
// status word, the roles stop issuing and the CTA frees its tensor memory and returns.
//
// Replaces flash_mla_with_kvcache (vllm_metax/v1/attention/backends/mla/flashmla.py:339-349) and the Triton split-KV
// MLA decode (vllm_metax/v1/attention/ops/triton_decode_attention.py:72-825) for ranks that hold 64 heads or more.
#include <type_traits>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"
#include "ops.h"

namespace b200 {
using namespace ptx;

constexpr int kTcBM = 128;                       // head rows per CTA
constexpr int kTcBN = 32;                        // cache tokens per tile
constexpr int kTcD = 576, kTcDV = 512, kTcHalf = 256;
constexpr int kTcKC = kTcD / 64;                 // 64-wide chunks of a cache row
constexpr int kTcQChunk = kTcBM * 128;           // bytes of one 64-wide query chunk
constexpr int kTcKChunk = kTcBN * 128;           // bytes of one 64-wide cache chunk
constexpr int kTcQBytes = kTcKC * kTcQChunk;     // 147456
constexpr int kTcTileBytes = kTcKC * kTcKChunk;  // 36864
constexpr float kTcLazy = 8.f;                   // log2 of the growth of a row maximum that forces a rescale

struct TcSmem {
  static constexpr int kQ = 0;
  static constexpr int kKV = kQ + kTcQBytes;     // 2 stages
  static constexpr int kBar = kKV + 2 * kTcTileBytes;
  static constexpr int kNumBars = 1 + 2 + 2 + 2 + 2 + 1;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
  static constexpr int kDyn = kTotal + 1024;
};
static_assert(TcSmem::kDyn <= 232448, "shared memory budget exceeded");

template <typename T>
__device__ __forceinline__ uint32_t tc_pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t tc_pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t tc_pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float tc_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__global__ void __launch_bounds__(192, 1)
mla_decode_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                     const MlaDecodeParams p) {
  using L = TcSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2] stages
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2] score buffers
  uint64_t* p_full = bars + 7;     // [2]
  uint64_t* o_done = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  __shared__ int s_seq, s_lim;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hf = blockIdx.x;                                  // latent half of the output
  const int h0 = blockIdx.y * kTcBM;
  const int t = (int)(blockIdx.z % (unsigned)p.total_tokens);
  const int split = (int)(blockIdx.z / (unsigned)p.total_tokens);

  constexpr uint32_t kTmemCols = 512;   // S0 [0,32) | S1 [32,64) | O [64,320)
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
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
    }
    mbar_init(o_done, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmKV);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S0 = tmem_base, tmem_S1 = tmem_base + 32, tmem_O = tmem_base + 64;
  const int seq = s_seq;
  const int lim = min(s_lim, p.max_blocks * p.block_size);    // never walk past the block table
  const int tiles_total = lim > 0 ? (lim + kTcBN - 1) / kTcBN : 0;
  const int tiles_per_split = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = split * tiles_per_split;
  const int n = max(0, min(tiles_total, tile_begin + tiles_per_split) - tile_begin);

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n > 0) {
      mbar_expect_tx(q_full, kTcQBytes);
#pragma unroll
      for (int c = 0; c < kTcKC; ++c) tma_load_3d(smem + L::kQ + c * kTcQChunk, &tmQ, q_full, c * 64, h0, t);
      const int* btab = p.block_table + (int64_t)seq * p.max_blocks;
      int issued = 0;
      for (int j = 0; j < n; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1)) {
          report_status(p.status, kWaitTimeout, 60, j, st);
          break;
        }
        const int tok0 = (tile_begin + j) * kTcBN;
        int page = btab[tok0 / p.block_size];
        if (page < 0 || page >= p.num_blocks) {
          report_status(p.status, kBadIndex, 61, (int)p.num_blocks, page);
          page = 0;
        }
        const int off = tok0 % p.block_size;
        uint8_t* dst = smem + L::kKV + st * kTcTileBytes;
        mbar_expect_tx(&kv_full[st], kTcTileBytes);
#pragma unroll
        for (int c = 0; c < kTcKC; ++c) tma_load_3d(dst + c * kTcKChunk, &tmKV, &kv_full[st], c * 64, off, page);
        issued = j + 1;
      }
      // no copy of this CTA is in flight when it returns: the last two tiles have landed (immediate unless a
      // role gave up before consuming them)
      for (int j = max(0, issued - 2); j < issued; ++j) mbar_wait(&kv_full[j & 1], (j >> 1) & 1);
      mbar_wait(q_full, 0);
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc_qk = make_idesc(1, fmt, fmt, kTcBM, kTcBN);
      // P.V: A = P from tensor memory (K-major), B = V in shared memory, MN-major (bit 16)
      constexpr uint32_t idesc_pv = make_idesc(1, fmt, fmt, kTcBM, kTcHalf) | (1u << 16);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) report_status(p.status, kWaitTimeout, 62, 0, 0);
      const uint32_t qa = smem_u32(smem + L::kQ);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&kv_full[st], (j >> 1) & 1)) {
          report_status(p.status, kWaitTimeout, 63, j, st);
          return false;
        }
        tc_fence_after_sync();
        const uint32_t ka = smem_u32(smem + L::kKV + st * kTcTileBytes);
#pragma unroll
        for (int c = 0; c < kTcKC; ++c) {
          const uint64_t dq = make_smem_desc_sw128(qa + c * kTcQChunk);
          const uint64_t dk = make_smem_desc_sw128(ka + c * kTcKChunk);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(st ? tmem_S1 : tmem_S0, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk,
                        (c | k) != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        if (!mbar_wait(&p_full[st], (j >> 1) & 1)) {
          report_status(p.status, kWaitTimeout, 64, j, st);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // this CTA's 256 latent columns = chunks 4 hf .. 4 hf + 3 of the tile; contraction over 32 tokens in two steps
        const uint32_t va = smem_u32(smem + L::kKV + st * kTcTileBytes) + hf * 4 * kTcKChunk;
#pragma unroll
        for (int kk = 0; kk < kTcBN / 16; ++kk) {
          const uint64_t dv = make_smem_desc_sw128_mn(va + kk * 16 * 128, kTcKChunk);
          umma_f16_ts(tmem_O, (st ? tmem_S1 : tmem_S0) + kk * 8, dv, idesc_pv, (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(o_done);
        umma_commit(&kv_empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / output (warps 0..3), thread = head
    const int r = warp * 32 + lane;
    const int h = h0 + r;
    const bool row_valid = h < p.num_heads;
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const int st = j & 1;
      // (every give-up decision is taken by the whole warp: the tensor-memory loads below are warp-collective)
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[st], (j >> 1) & 1))) {
        report_status(p.status, kWaitTimeout, 65, j, st);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t tmem_St = (st ? tmem_S1 : tmem_S0) + lane_base;
      uint32_t sv[32];
      tmem_ld_32x32b_x32(tmem_St, sv);
      tmem_ld_wait();
      float s[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(sv[i]) * sl2;
      const int t0 = (tile_begin + j) * kTcBN;
      if (t0 + kTcBN > lim) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (t0 + i >= lim) s[i] = -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int i = 1; i < 32; ++i) mx = fmaxf(mx, s[i]);
      const bool grow = mx > m_run + kTcLazy;        // also true for the first finite maximum
      float corr = 1.f;
      if (grow) {
        corr = (m_run == -INFINITY) ? 0.f : exp2f(m_run - mx);
        m_run = mx;
        l_run *= corr;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // the product of tile j - 1 must have landed before the accumulator is rescaled
        if (!__all_sync(0xffffffffu, mbar_wait(o_done, (j - 1) & 1))) {
          report_status(p.status, kWaitTimeout, 66, j, st);
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < kTcHalf; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_O + lane_base + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tmem_st_32x32b_x32(tmem_O + lane_base + c, v);
        }
      }
      const float m_off = (m_run == -INFINITY) ? 0.f : m_run;
      float rs = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float e0 = tc_exp2(s[2 * i] - m_off);
        const float e1 = tc_exp2(s[2 * i + 1] - m_off);
        rs += e0 + e1;
        pk[i] = tc_pack2<T>(e0, e1);
      }
      tmem_st_32x32b_x16(tmem_St, pk);
      l_run += rs;
      // P (and a rescaled accumulator) visible to the MMA warp
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&p_full[st]);
    }
    if (ok && n > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(o_done, (n - 1) & 1))) {
        report_status(p.status, kWaitTimeout, 67, n, 0);
        ok = false;
      }
      tc_fence_after_sync();
    }
    const bool have = ok && n > 0 && l_run > 0.f;
    const float inv = have ? 1.f / l_run : 0.f;
    const float lse = have ? m_run * 0.6931471805599453f + logf(l_run) : -INFINITY;
    const int64_t prow = ((int64_t)split * p.total_tokens + t) * p.num_heads + h;
    T* dst16 = reinterpret_cast<T*>(p.out) + ((int64_t)t * p.num_heads + h) * kTcDV + hf * kTcHalf;
    float* dst32 = p.part_out ? p.part_out + prow * kTcDV + hf * kTcHalf : nullptr;
#pragma unroll 1
    for (int c = 0; c < kTcHalf; c += 32) {
      uint32_t v[32];
      if (ok && n > 0) {                                // warp-uniform: ok and n are the same for all lanes of a warp
        tmem_ld_32x32b_x32(tmem_O + lane_base + c, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (!row_valid) continue;
      if (p.num_splits == 1) {
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g8 * 8 + i]) * inv;
          *reinterpret_cast<uint4*>(dst16 + c + g8 * 8) = pack8<T>(f);
        }
      } else {
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4)
          *reinterpret_cast<float4*>(dst32 + c + g4 * 4) =
              make_float4(__uint_as_float(v[g4 * 4]) * inv, __uint_as_float(v[g4 * 4 + 1]) * inv,
                          __uint_as_float(v[g4 * 4 + 2]) * inv, __uint_as_float(v[g4 * 4 + 3]) * inv);
      }
    }
    if (row_valid && hf == 0) {
      if (p.num_splits == 1) {
        if (p.lse_out) p.lse_out[(int64_t)h * p.total_tokens + t] = lse;
      } else {
        p.part_lse[prow] = lse;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Returns 0 when the launch was made, -1 when this kernel does not serve the call (sparse, a block size that is
// not a multiple of 32, unaligned operands, too many (token, split) pairs for one grid dimension).
int mla_decode_tc(const MlaDecodeParams& p, int dtype, cudaStream_t stream) {
  if (p.total_tokens <= 0) return 0;
  if (p.topk_indices != nullptr) return -1;
  if (p.block_size % kTcBN != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(p.q) & 15) || (p.q_stride * 2) % 16 != 0) return -1;
  if (reinterpret_cast<uintptr_t>(p.cache) & 15) return -1;
  if ((int64_t)p.total_tokens * p.num_splits > 65535) return -1;
  if (p.num_splits > 1 && (p.part_out == nullptr || p.part_lse == nullptr)) return -1;
  const CUtensorMapDataType dt = dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // q: [T, H, 576] -> dims (576, H, T), box (64, 128 heads, 1 token)
  uint64_t qd[3] = {(uint64_t)kTcD, (uint64_t)p.num_heads, (uint64_t)p.total_tokens};
  uint64_t qs[2] = {(uint64_t)kTcD * 2, (uint64_t)p.q_stride * 2};
  uint32_t qb[3] = {64, (uint32_t)kTcBM, 1};
  const CUtensorMap tmQ = make_tmap_nd(p.q, dt, 3, qd, qs, qb, CU_TENSOR_MAP_SWIZZLE_128B);
  // cache: [blocks, block_size, 576] -> dims (576, block_size, blocks), box (64, 32 tokens, 1 page)
  uint64_t kd[3] = {(uint64_t)kTcD, (uint64_t)p.block_size, (uint64_t)p.num_blocks};
  uint64_t ks[2] = {(uint64_t)kTcD * 2, (uint64_t)p.block_size * kTcD * 2};
  uint32_t kb[3] = {64, (uint32_t)kTcBN, 1};
  const CUtensorMap tmKV = make_tmap_nd(p.cache, dt, 3, kd, ks, kb, CU_TENSOR_MAP_SWIZZLE_128B);
  dim3 grid(2, (unsigned)((p.num_heads + kTcBM - 1) / kTcBM), (unsigned)(p.total_tokens * p.num_splits));
  if (dtype == 1) {
    auto kern = mla_decode_tc_kernel<__half>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem::kDyn);
    kern<<<grid, 192, TcSmem::kDyn, stream>>>(tmQ, tmKV, p);
  } else {
    auto kern = mla_decode_tc_kernel<__nv_bfloat16>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem::kDyn);
    kern<<<grid, 192, TcSmem::kDyn, stream>>>(tmQ, tmKV, p);
  }
  return 0;
}

}  // namespace b200
