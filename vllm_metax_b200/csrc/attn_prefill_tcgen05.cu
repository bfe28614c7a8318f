// Varlen (ragged) causal attention for prefill / chunked prefill on tcgen05:
// one CTA per (sequence, kv-head group, 128-row query tile).
//
//   rows      the 128 tile rows are (query token, head-in-group) pairs, so all the
//             query heads that share a KV head reuse the same K/V tiles from
//             shared memory (GQA packing); without packing a tile is 128 tokens
//             of one head.
//   warp 0    TMA producer: Q tile once, then 128-token K and V tiles through
//             2-stage rings.  K/V come either from the paged cache (4-D tensor
//             map [D, kv_head, slot-in-block, 2*block+kv], one box per page) or
//             from contiguous [T, H, D] tensors (3-D map).
//   warp 1    MMA issuer: S = Q.K^T into one of two TMEM buffers (so the next
//             tile's QK^T overlaps this tile's softmax), then O_tile = P.V with P
//             read from shared memory (K-major) and V used in place as an
//             MN-major operand.
//   warps 2-5 softmax: thread = row.  tcgen05.ld the row of S, online softmax in
//             the exp2 domain, P (bf16) to swizzled shared memory, running output
//             kept in registers and updated from the per-tile P.V result in TMEM.
//
// Query heads must be 16-bit (bf16/fp16), D_qk in {64,128,192}, D_v in {64,128}.
// Causal offset: row token i of a sequence with q_len new tokens and kv_len total
// sits at position kv_len - q_len + i.  Sliding window, soft-cap and attention
// sinks are supported; LSE can be returned for later merges.
//
// Replaces flash_attn_varlen_func (vllm_metax/v1/attention/backends/flash_attn.py:1302-1322,
// mla/prefill/flash_attn.py:157-163).
#include <type_traits>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"
#include "ops.h"

namespace b200 {
using namespace ptx;


constexpr int kPfBM = 128;   // query rows per tile

template <int DQK, int DV, int BN>
struct PfSmem {
  static constexpr int kQBytes = kPfBM * DQK * 2;
  static constexpr int kKBytes = BN * DQK * 2;
  static constexpr int kVBytes = BN * DV * 2;
  static constexpr int kPBytes = kPfBM * BN * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kQBytes;            // 2 stages
  static constexpr int kV = kK + 2 * kKBytes;        // 2 stages
  static constexpr int kP = kV + 2 * kVBytes;
  static constexpr int kBar = kP + kPBytes;
  static constexpr int kNumBars = 1 + 2 + 2 + 2 + 2 + 2 + 2 + 1 + 1 + 3;   // + row-exchange barriers
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
  static constexpr int kDyn = kTotal + 1024;
};

template <typename T, int DQK, int DV, int BN>
__global__ void __launch_bounds__(320, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  using L = PfSmem<DQK, DV, BN>;
  constexpr int KC = DQK / 64;   // 64-wide chunks of the QK contraction
  constexpr int VC = DV / 64;    // 64-wide chunks of the value dim
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* o_full = bars + 14;
  uint64_t* x_bar = bars + 15;    // [3] the two threads of a row exchange max (per tile, alternating) and sum
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int hg = blockIdx.y;                    // head group index
  const int q_begin = p.query_start_loc[b];
  const int q_len = p.query_start_loc[b + 1] - q_begin;
  const int toks_per_tile = kPfBM / p.gp;
  const int num_q_tiles = (q_len + toks_per_tile - 1) / toks_per_tile;
  // heavier (later) tiles first
  const int qt = num_q_tiles - 1 - (int)blockIdx.x;
  if (qt < 0) return;
  const int kv_begin = p.paged ? 0 : p.kv_start_loc[b];
  const int kv_len = p.paged ? p.seq_lens[b] : (p.kv_start_loc[b + 1] - kv_begin);
  const int tok0 = qt * toks_per_tile;                        // first query token of the tile (in sequence)
  const int h0 = hg * p.gp;                                   // first query head of the tile
  const int hk = h0 / (p.num_q_heads / p.num_kv_heads);       // kv head
  const int pos0 = kv_len - q_len + tok0;                     // position of the first tile token
  const int last_tok = min(q_len, tok0 + toks_per_tile) - 1;
  const int kv_hi = p.causal ? min(kv_len, kv_len - q_len + last_tok + 1) : kv_len;  // exclusive
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, pos0 + 1 - p.window);
  const int tile_lo = kv_lo / BN;
  const int tile_hi = (kv_hi + BN - 1) / BN;            // exclusive
  const int n_tiles = max(0, tile_hi - tile_lo);

  constexpr uint32_t kTmemCols = 512;  // S0, S1 (128 each), O_tile (DV)
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 256);
    }
    mbar_init(p_full, 256);
    for (int i = 0; i < 3; ++i) mbar_init(&x_bar[i], 256);
    mbar_init(o_full, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S[2] = {tmem_base, tmem_base + 128};  // BN <= 128 columns each
  const uint32_t tmem_O = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(q_full, L::kQBytes);
#pragma unroll
      for (int kc = 0; kc < KC; ++kc)
        tma_load_3d(smem + L::kQ + kc * (kPfBM * 128), &tmQ, q_full, kc * 64, h0, q_begin + tok0);
      const int* btab = p.paged ? p.block_table + (int64_t)b * p.max_blocks : nullptr;
      const int pages_per_tile = p.paged ? (BN / min(p.block_size, BN)) : 1;
      const int rows_per_box = p.paged ? min(p.block_size, BN) : BN;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int t0 = (tile_lo + j) * BN;
        for (int which = 0; which < 2 && ok; ++which) {  // 0: K, 1: V
          uint64_t* full = which ? &v_full[st] : &k_full[st];
          uint64_t* empty = which ? &v_empty[st] : &k_empty[st];
          if (!mbar_wait(empty, ph ^ 1)) {
            report_status(p.status, kWaitTimeout, 30 + which, j, st);
            ok = false;
            break;
          }
          const int nch = which ? VC : KC;
          const int tile_bytes = which ? L::kVBytes : L::kKBytes;
          uint8_t* dst = smem + (which ? L::kV + st * L::kVBytes : L::kK + st * L::kKBytes);
          mbar_expect_tx(full, tile_bytes);
          for (int pg = 0; pg < pages_per_tile; ++pg) {
            const int tok = t0 + pg * rows_per_box;
            if (p.paged) {
              int page = 0, off = 0;
              if (tok < kv_len) {
                page = btab[tok / p.block_size];
                off = tok % p.block_size;
                if (page < 0 || page >= p.num_blocks) {
                  report_status(p.status, kBadIndex, 32, (int)p.num_blocks, page);
                  page = 0;
                }
              }
              for (int c = 0; c < nch; ++c)
                tma_load_4d(dst + c * (BN * 128) + pg * rows_per_box * 128, which ? &tmV : &tmK, full, c * 64, hk,
                            off, page * 2 + which);
            } else {
              for (int c = 0; c < nch; ++c)
                tma_load_3d(dst + c * (BN * 128), which ? &tmV : &tmK, full, c * 64, hk, kv_begin + tok);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc_qk = make_idesc(1, fmt, fmt, kPfBM, BN);
      // P.V: A = P (K-major), B = V (MN-major: bit 16)
      constexpr uint32_t idesc_pv = make_idesc(1, fmt, fmt, kPfBM, DV) | (1u << 16);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) report_status(p.status, kWaitTimeout, 40, 0, 0);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph) || !mbar_wait(&s_empty[st], ph ^ 1)) {
          report_status(p.status, kWaitTimeout, 41, j, st);
          return false;
        }
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(smem + L::kQ);
        const uint32_t ka = smem_u32(smem + L::kK + st * L::kKBytes);
#pragma unroll
        for (int kc = 0; kc < KC; ++kc) {
          const uint64_t dq = make_smem_desc_sw128(qa + kc * (kPfBM * 128));
          const uint64_t dk = make_smem_desc_sw128(ka + kc * (BN * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem_S[st], dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, (kc | k) != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&v_full[st], ph) || !mbar_wait(p_full, j & 1)) {
          report_status(p.status, kWaitTimeout, 42, j, st);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(smem + L::kP);
        const uint32_t va = smem_u32(smem + L::kV + st * L::kVBytes);
        // contraction over the 128 tile tokens in steps of 16
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t dp = make_smem_desc_sw128(pa + (kk >> 2) * (kPfBM * 128)) + (uint64_t)((kk & 3) * 2);
          const uint64_t dv = make_smem_desc_sw128_mn(va + kk * 16 * 128, BN * 128);
          umma_f16_ss(tmem_O, dp, dv, idesc_pv, kk != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(o_full);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / output (warps 2..9)
    // Two threads per tile row: warps 2..5 take the first half of a tile's key columns and of the value
    // dimension, warps 6..9 the second half (a warp reaches the TMEM lanes of quarter warp % 4, any columns).
    // The row maximum is exchanged through shared memory once per tile; the row sums are added at the end.
    constexpr int HC = BN / 2, HD = DV / 2;
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int c_lo = half * HC, d_lo = half * HD;
    __shared__ float s_xmax[2][2][kPfBM];
    __shared__ float s_xsum[2][kPfBM];
    const int r = quarter * 32 + lane;              // tile row
    const int tok = tok0 + r / p.gp;                // token within the sequence
    const int hq = h0 + r % p.gp;
    const bool row_valid = tok < q_len;
    const int pos = kv_len - q_len + tok;           // absolute position of this row
    const int lim = row_valid ? (p.causal ? pos + 1 : kv_len) : 0;  // sees kv < lim
    const int lo = (p.window > 0) ? max(0, lim - p.window) : 0;
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint32_t lane_base = ((uint32_t)(quarter * 32)) << 16;
    float o_reg[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o_reg[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    const float alibi2 = (p.alibi_slopes && row_valid) ? p.alibi_slopes[hq] * 1.4426950408889634f : 0.f;
    auto fx = [&](float s, int col) -> float {
      const float base = (p.softcap > 0.f) ? p.softcap * tanhf(s * p.scale / p.softcap) * 1.4426950408889634f : s * sl2;
      return base + alibi2 * (float)(col - pos);     // ALiBi bias (0 without slopes)
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph)) {
        report_status(p.status, kWaitTimeout, 50, j, st);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int t0 = (tile_lo + j) * BN;
      const bool need_mask = (t0 + BN > lim) || (t0 < lo);
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = c_lo; c < c_lo + HC; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_S[st] + lane_base + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = fx(__uint_as_float(v[i]), t0 + c + i);
          if (need_mask) {
            const int col = t0 + c + i;
            if (col >= lim || col < lo) s = -INFINITY;
          }
          mx = fmaxf(mx, s);
        }
      }
      // the other half of the row: buffers alternate per tile, so one barrier per tile is enough
      s_xmax[j & 1][half][r] = mx;
      mbar_arrive(&x_bar[j & 1]);
      if (!mbar_wait(&x_bar[j & 1], (j >> 1) & 1)) {      // bounded like every other wait
        report_status(p.status, kWaitTimeout, 53, j, half);
        ok = false;
        break;
      }
      mx = fmaxf(mx, s_xmax[j & 1][half ^ 1][r]);
      const float m_new = fmaxf(m_run, mx);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_run - m_safe);
      m_run = m_new;
      // fold the previous tile's P.V (kept separate so its MMA overlapped pass 1)
      if (j > 0) {
        if (!mbar_wait(o_full, (j - 1) & 1)) {
          report_status(p.status, kWaitTimeout, 51, j, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_O + lane_base + d_lo + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_reg[c + i] += __uint_as_float(v[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < HD; ++i) o_reg[i] *= corr;
      l_run *= corr;
      // pass 2: P = exp2(S - m) -> shared memory (bf16, K-major, 128B swizzle)
      float rs = 0.f;
#pragma unroll 1
      for (int c = c_lo; c < c_lo + HC; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_S[st] + lane_base + c, v);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = fx(__uint_as_float(v[i]), t0 + c + i);
          if (need_mask) {
            const int col = t0 + c + i;
            if (col >= lim || col < lo) s = -INFINITY;
          }
          const float e = exp2f(s - m_safe);
          // the row sum uses the value the MMA will see
          pv[i] = to_f(from_f<T>(e));
          rs += pv[i];
        }
        uint8_t* prow = smem + L::kP + (c >> 6) * (kPfBM * 128) + r * 128;
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = pv[g8 * 8 + i];
          const int chunk = ((c & 63) >> 3) + g8;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) * 16)) = pack8<T>(f);
        }
      }
      l_run += rs;
      // S buffer free for tile j+2, P ready for the MMA warp
      tc_fence_before_sync();
      fence_proxy_async();
      mbar_arrive(&s_empty[st]);
      mbar_arrive(p_full);
    }
    if (ok && n_tiles > 0) {
      if (!mbar_wait(o_full, (n_tiles - 1) & 1)) {
        report_status(p.status, kWaitTimeout, 52, n_tiles, 0);
        ok = false;
      } else {
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_O + lane_base + d_lo + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_reg[c + i] += __uint_as_float(v[i]);
        }
      }
    }
    s_xsum[half][r] = l_run;
    mbar_arrive(&x_bar[2]);
    if (ok && !mbar_wait(&x_bar[2], 0)) {
      report_status(p.status, kWaitTimeout, 54, 0, half);
      ok = false;
    }
    if (row_valid && ok) {
      float l_tot = l_run + s_xsum[half ^ 1][r];
      const float m_safe = (m_run == -INFINITY) ? 0.f : m_run;
      if (p.sinks) l_tot += exp2f(p.sinks[hq] * 1.4426950408889634f - m_safe);
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + ((int64_t)(q_begin + tok) * p.num_q_heads + hq) * DV + d_lo;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = o_reg[c + i] * inv;
        *reinterpret_cast<uint4*>(dst + c) = pack8<T>(f);
      }
      if (p.lse_out && half == 0)
        p.lse_out[(int64_t)hq * p.total_q + q_begin + tok] =
            l_tot > 0.f ? (m_safe * 0.6931471805599453f + logf(l_tot)) : -INFINITY;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int DQK, int DV, int BN>
static void launch_prefill(const PrefillParams& p, const void* q, int64_t q_stride, const void* k_src,
                           const void* v_src, int64_t kv_tok_stride_k, int64_t kv_tok_stride_v, int64_t total_kv,
                           int batch, int max_q_len, cudaStream_t stream) {
  using L = PfSmem<DQK, DV, BN>;
  static_assert(L::kDyn + 3072 <= 232448, "shared memory budget exceeded (dynamic + the static row-exchange arrays)");
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // Q: [T, Hq, DQK], box [128/gp tokens, gp heads, 64]
  uint64_t qd[3] = {(uint64_t)DQK, (uint64_t)p.num_q_heads, (uint64_t)p.total_q};
  uint64_t qs[2] = {(uint64_t)DQK * 2, (uint64_t)q_stride * 2};
  uint32_t qb[3] = {64, (uint32_t)p.gp, (uint32_t)(kPfBM / p.gp)};
  CUtensorMap tmQ = make_tmap_nd(q, dt, 3, qd, qs, qb, CU_TENSOR_MAP_SWIZZLE_128B);
  CUtensorMap tmK, tmV;
  if (p.paged) {
    // cache [num_blocks, 2, block_size, Hkv, D] -> dims [D, Hkv, block_size, 2*num_blocks]
    const uint32_t rows = (uint32_t)(p.block_size < BN ? p.block_size : BN);
    uint64_t kd[4] = {(uint64_t)DQK, (uint64_t)p.num_kv_heads, (uint64_t)p.block_size, (uint64_t)(2 * p.num_blocks)};
    uint64_t ks[3] = {(uint64_t)DQK * 2, (uint64_t)p.num_kv_heads * DQK * 2,
                      (uint64_t)p.block_size * p.num_kv_heads * DQK * 2};
    uint32_t kb[4] = {64, 1, rows, 1};
    tmK = make_tmap_nd(k_src, dt, 4, kd, ks, kb, CU_TENSOR_MAP_SWIZZLE_128B);
    tmV = tmK;
  } else {
    uint64_t kd[3] = {(uint64_t)DQK, (uint64_t)p.num_kv_heads, (uint64_t)total_kv};
    uint64_t ks[2] = {(uint64_t)DQK * 2, (uint64_t)kv_tok_stride_k * 2};
    uint32_t kb[3] = {64, 1, (uint32_t)BN};
    tmK = make_tmap_nd(k_src, dt, 3, kd, ks, kb, CU_TENSOR_MAP_SWIZZLE_128B);
    uint64_t vd[3] = {(uint64_t)DV, (uint64_t)p.num_kv_heads, (uint64_t)total_kv};
    uint64_t vs[2] = {(uint64_t)DV * 2, (uint64_t)kv_tok_stride_v * 2};
    tmV = make_tmap_nd(v_src, dt, 3, vd, vs, kb, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  auto kern = attn_prefill_kernel<T, DQK, DV, BN>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
  const int toks_per_tile = kPfBM / p.gp;
  dim3 grid(ceil_div(max_q_len, toks_per_tile), p.num_q_heads / p.gp, batch);
  kern<<<grid, 320, L::kDyn, stream>>>(tmQ, tmK, tmV, p);
}

// Returns 0 on success, -1 when the head sizes are not supported by this kernel.
int attention_prefill(const PrefillParams& p, const void* q, int64_t q_stride, const void* k_src, const void* v_src,
                      int64_t k_tok_stride, int64_t v_tok_stride, int64_t total_kv, int dqk, int dv, int dtype,
                      int batch, int max_q_len, cudaStream_t stream) {
  if (batch <= 0 || max_q_len <= 0) return 0;
#define PF(T)                                                                                                        \
  if (dqk == 128 && dv == 128)                                                                                       \
    launch_prefill<T, 128, 128, 128>(p, q, q_stride, k_src, v_src, k_tok_stride, v_tok_stride, total_kv, batch, max_q_len, stream); \
  else if (dqk == 64 && dv == 64)                                                                                    \
    launch_prefill<T, 64, 64, 128>(p, q, q_stride, k_src, v_src, k_tok_stride, v_tok_stride, total_kv, batch, max_q_len, stream);   \
  else if (dqk == 192 && dv == 128 && !p.paged)                                                                      \
    launch_prefill<T, 192, 128, 64>(p, q, q_stride, k_src, v_src, k_tok_stride, v_tok_stride, total_kv, batch, max_q_len, stream); \
  else                                                                                                               \
    return -1;
  if (dtype == 0) { PF(__nv_bfloat16) } else { PF(__half) }
#undef PF
  return 0;
}

}  // namespace b200
