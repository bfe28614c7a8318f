// Varlen (ragged) causal attention for prefill / chunked prefill on tcgen05, two query tiles per CTA:
// one CTA per (sequence, kv-head group, PAIR of 128-row query tiles).
//
//   rows      the 128 rows of a tile are (query token, head-in-group) pairs, so all the query heads that
//             share a KV head reuse the same K/V tiles (GQA packing); without packing a tile is 128 tokens
//             of one head.  Tile B holds the tokens that follow tile A's, so both walk the same K/V tiles
//             and every K/V byte is fetched once per 256 rows.
//   warp 8    TMA producer: both Q tiles once, then BN-token K and V tiles through 2-stage rings, from the
//             paged cache (4-D tensor map, one box per page) or from contiguous [T, H, D] tensors.
//   warp 9    MMA issuer, alternating between the tiles so that the tensor core works on one tile while the
//             other tile's softmax runs:  S_t = Q_t.K^T into TMEM;  O_t += P_t.V with P_t read from TMEM
//             (it overwrites the first half of S_t's columns as packed 16-bit pairs) and V used in place
//             as an MN-major shared-memory operand.  The output accumulators never leave TMEM.
//   warps 0-3 softmax of tile A, warps 4-7 softmax of tile B: thread = row.  One tcgen05.ld brings the
//             whole row of S into registers; online softmax in the exp2 domain; P goes back with
//             tcgen05.st.  The running maximum is only moved when the new row maximum exceeds it by more
//             than 2^8 (the accumulators are then rescaled in TMEM by the same thread), so after the first
//             tiles the softmax never waits for the P.V product of the previous tile.
//   The three warp groups re-balance the register file at start-up (setmaxnreg): the producer / issuer
//   group gives registers up, the softmax groups take them so that a 128-wide row of S fits.
//
// Query heads must be 16-bit (bf16/fp16); (D_qk, D_v) in {(128,128), (64,64), (192,128)}.
// Causal offset: row token i of a sequence with q_len new tokens and kv_len total sits at position
// kv_len - q_len + i.  Sliding window, soft-cap, ALiBi and attention sinks are supported; LSE can be
// returned for later merges.  TMA loads touch this GPU's memory only.
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

constexpr int kPpBM = 128;          // rows per query tile
constexpr float kPpLazy = 8.f;      // log2 of the growth of a row maximum that forces a rescale

template <int DQK, int DV, int BN>
struct PpSmem {
  static constexpr int kQBytes = kPpBM * DQK * 2;     // per tile
  static constexpr int kKBytes = BN * DQK * 2;
  static constexpr int kVBytes = BN * DV * 2;
  static constexpr int kQ = 0;                        // 2 tiles
  static constexpr int kK = kQ + 2 * kQBytes;         // 2 stages
  static constexpr int kV = kK + 2 * kKBytes;         // 2 stages
  static constexpr int kBar = kV + 2 * kVBytes;
  static constexpr int kNumBars = 1 + 2 + 2 + 2 + 2 + 2 + 2 + 2;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
  static constexpr int kDyn = kTotal + 1024;
};

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ex2.approx: one MUFU op, exp2(-inf) = 0
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T, int DQK, int DV, int BN>
__global__ void __launch_bounds__(384, 1)
attn_prefill_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  using L = PpSmem<DQK, DV, BN>;
  constexpr int KC = DQK / 64;   // 64-wide chunks of the QK contraction
  constexpr int VC = DV / 64;    // 64-wide chunks of the value dim
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2] stages
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] per query tile
  uint64_t* p_full = bars + 11;   // [2] per query tile
  uint64_t* o_done = bars + 13;   // [2] per query tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int hg = blockIdx.y;                    // head group index
  const int q_begin = p.query_start_loc[b];
  const int q_len = p.query_start_loc[b + 1] - q_begin;
  const int tpt = kPpBM / p.gp;                 // tokens per query tile
  const int num_pairs = (q_len + 2 * tpt - 1) / (2 * tpt);
  const int qp = num_pairs - 1 - (int)blockIdx.x;   // heavier (later) pairs first
  if (qp < 0) return;
  const int kv_begin = p.paged ? 0 : p.kv_start_loc[b];
  const int kv_len = p.paged ? p.seq_lens[b] : (p.kv_start_loc[b + 1] - kv_begin);
  const int tok0 = qp * 2 * tpt;                              // first query token of tile A (in sequence)
  const int h0 = hg * p.gp;                                   // first query head of the tiles
  const int hk = h0 / (p.num_q_heads / p.num_kv_heads);       // kv head
  const int pos0 = kv_len - q_len + tok0;                     // position of tile A's first token
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, pos0 + 1 - p.window);
  const int tile_lo = kv_lo / BN;
  // number of K/V tiles each query tile walks (0: the tile holds no token of this sequence)
  auto tiles_of = [&](int t) -> int {
    const int first = tok0 + t * tpt;
    const int last = min(q_len, first + tpt) - 1;
    if (last < first) return 0;
    const int kv_hi = p.causal ? min(kv_len, kv_len - q_len + last + 1) : kv_len;   // exclusive
    return max(0, (kv_hi + BN - 1) / BN - tile_lo);
  };
  const int n_a = tiles_of(0), n_b = tiles_of(1);
  const int n_all = max(n_a, n_b);

  constexpr uint32_t kTmemCols = 512;  // S_A, S_B (128 columns reserved each), O_A, O_B (DV each)
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_done[i], 1);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // (selected with ?: so that nothing is indexed through local memory)
  const uint32_t tmem_S0 = tmem_base, tmem_S1 = tmem_base + 128;
  const uint32_t tmem_O0 = tmem_base + 256, tmem_O1 = tmem_base + 256 + DV;

  // warp-group-wide register re-balancing: 2 x 128 x 224 + 128 x 56 registers = the 384 x 168 of the launch
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_all > 0) {
      const int q_tiles = n_b > 0 ? 2 : 1;
      mbar_expect_tx(q_full, q_tiles * L::kQBytes);
      for (int t = 0; t < q_tiles; ++t)
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
          tma_load_3d(smem + L::kQ + t * L::kQBytes + kc * (kPpBM * 128), &tmQ, q_full, kc * 64, h0,
                      q_begin + tok0 + t * tpt);
      const int* btab = p.paged ? p.block_table + (int64_t)b * p.max_blocks : nullptr;
      const int pages_per_tile = p.paged ? (BN / min(p.block_size, BN)) : 1;
      const int rows_per_box = p.paged ? min(p.block_size, BN) : BN;
      bool ok = true;
      for (int j = 0; j < n_all && ok; ++j) {
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
                const int bi = tok / p.block_size;
                page = bi < p.max_blocks ? btab[bi] : -1;
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
    } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_all > 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc_qk = make_idesc(1, fmt, fmt, kPpBM, BN);
      // P.V: A = P from TMEM (K-major), B = V in shared memory, MN-major (bit 16)
      constexpr uint32_t idesc_pv = make_idesc(1, fmt, fmt, kPpBM, DV) | (1u << 16);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) report_status(p.status, kWaitTimeout, 40, 0, 0);
      // tile t is the last reader of K/V tile j when it is tile B, or when tile B does not reach j
      auto last_user = [&](int t, int j) -> bool { return t == 1 || j >= n_b; };
      auto issue_qk = [&](int t, int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph)) {
          report_status(p.status, kWaitTimeout, 41, j, t);
          return false;
        }
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(smem + L::kQ + t * L::kQBytes);
        const uint32_t ka = smem_u32(smem + L::kK + st * L::kKBytes);
#pragma unroll
        for (int kc = 0; kc < KC; ++kc) {
          const uint64_t dq = make_smem_desc_sw128(qa + kc * (kPpBM * 128));
          const uint64_t dk = make_smem_desc_sw128(ka + kc * (BN * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(t ? tmem_S1 : tmem_S0, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, (kc | k) != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
        if (last_user(t, j)) umma_commit(&k_empty[st]);
        return true;
      };
      for (int t = 0; t < 2 && ok; ++t)
        if ((t ? n_b : n_a) > 0) ok = issue_qk(t, 0);
      for (int j = 0; j < n_all && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        for (int t = 0; t < 2 && ok; ++t) {
          const int n_mine = t ? n_b : n_a;
          if (j >= n_mine) continue;
          if (!mbar_wait(&v_full[st], ph) || !mbar_wait(&p_full[t], j & 1)) {
            report_status(p.status, kWaitTimeout, 42, j, t);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t va = smem_u32(smem + L::kV + st * L::kVBytes);
          // contraction over the BN tile tokens in steps of 16 (8 TMEM columns of packed pairs)
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            const uint64_t dv = make_smem_desc_sw128_mn(va + kk * 16 * 128, BN * 128);
            umma_f16_ts(t ? tmem_O1 : tmem_O0, (t ? tmem_S1 : tmem_S0) + kk * 8, dv, idesc_pv, (j | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&o_done[t]);
          if (last_user(t, j)) umma_commit(&v_empty[st]);
          // the next S of this tile may only overwrite P once the product above has read it: same issue order
          if (j + 1 < n_mine) ok = issue_qk(t, j + 1);
        }
      }
    }
    }
  } else {
    // ------------------------------------------------------------ softmax / output (warps 0..7)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int t = warp >> 2;                        // query tile of this warp group
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;              // tile row
    const int tok = tok0 + t * tpt + r / p.gp;      // token within the sequence
    const int hq = h0 + r % p.gp;
    const bool row_valid = tok < q_len;
    const int pos = kv_len - q_len + tok;           // absolute position of this row
    const int lim = row_valid ? (p.causal ? pos + 1 : kv_len) : 0;  // sees kv < lim
    const int lo = (p.window > 0) ? max(0, lim - p.window) : 0;
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint32_t lane_base = ((uint32_t)(quarter * 32)) << 16;
    const bool plain = !(p.softcap > 0.f) && p.alibi_slopes == nullptr;
    const float alibi2 = (p.alibi_slopes && row_valid) ? p.alibi_slopes[hq] * 1.4426950408889634f : 0.f;
    const float mul = plain ? sl2 : 1.f;            // scores are kept raw on the plain path
    const int n_mine = t ? n_b : n_a;
    const uint32_t tmem_St = (t ? tmem_S1 : tmem_S0) + lane_base, tmem_Ot = (t ? tmem_O1 : tmem_O0) + lane_base;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!mbar_wait(&s_full[t], j & 1)) {
        report_status(p.status, kWaitTimeout, 50, j, t);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int t0 = (tile_lo + j) * BN;
      // the whole row of S: all loads in flight, one wait, nothing reads the registers before it
      uint32_t sv[BN];
#pragma unroll
      for (int c = 0; c < BN; c += 32) tmem_ld_32x32b_x32(tmem_St + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_ld_wait();
      float s[BN];
#pragma unroll
      for (int i = 0; i < BN; ++i) s[i] = __uint_as_float(sv[i]);
      if (!plain) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const float base =
              (p.softcap > 0.f) ? p.softcap * tanhf(s[i] * p.scale / p.softcap) * 1.4426950408889634f : s[i] * sl2;
          s[i] = base + alibi2 * (float)(t0 + i - pos);
        }
      }
      if ((t0 + BN > lim) || (t0 < lo)) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int col = t0 + i;
          if (col >= lim || col < lo) s[i] = -INFINITY;
        }
      }
      float mx = s[0];
#pragma unroll
      for (int i = 1; i < BN; ++i) mx = fmaxf(mx, s[i]);
      mx *= mul;                                     // scale > 0: the maximum commutes with it
      // lazy maximum: move it only when a row outgrows the exponent range the packed P can carry
      const bool grow = mx > m_run + kPpLazy;        // also true for the first finite maximum
      float corr = 1.f;
      if (grow) {
        corr = (m_run == -INFINITY) ? 0.f : exp2f(m_run - mx);
        m_run = mx;
        l_run *= corr;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        if (!mbar_wait(&o_done[t], (j - 1) & 1)) {
          report_status(p.status, kWaitTimeout, 51, j, t);
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < DV; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_Ot + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tmem_st_32x32b_x32(tmem_Ot + c, v);
        }
      }
      const float m_off = (m_run == -INFINITY) ? 0.f : m_run;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < BN; c += 64) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e0 = fast_exp2(fmaf(s[c + 2 * i], mul, -m_off));
          const float e1 = fast_exp2(fmaf(s[c + 2 * i + 1], mul, -m_off));
          rs += e0 + e1;
          pk[i] = pack2<T>(e0, e1);
        }
        tmem_st_32x32b_x32(tmem_St + (c >> 1), pk);
      }
      l_run += rs;
      // P (and a rescaled O) visible to the MMA warp
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&p_full[t]);
    }
    float o_acc_scale = 0.f;
    float l_tot = l_run;
    const float m_safe = (m_run == -INFINITY) ? 0.f : m_run;
    if (p.sinks && row_valid) l_tot += exp2f(p.sinks[hq] * 1.4426950408889634f - m_safe);
    if (l_tot > 0.f) o_acc_scale = 1.f / l_tot;
    if (ok && n_mine > 0) {
      if (!mbar_wait(&o_done[t], (n_mine - 1) & 1)) {
        report_status(p.status, kWaitTimeout, 52, n_mine, t);
        ok = false;
      }
      tc_fence_after_sync();
    }
    if (ok && n_mine > 0) {
      T* dst = reinterpret_cast<T*>(p.out) + ((int64_t)(q_begin + tok) * p.num_q_heads + hq) * DV;
#pragma unroll 1
      for (int c = 0; c < DV; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_Ot + c, v);     // warp-collective: every lane takes part
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g8 * 8 + i]) * o_acc_scale;
            *reinterpret_cast<uint4*>(dst + c + g8 * 8) = pack8<T>(f);
          }
        }
      }
    } else if (ok && row_valid) {
      // a row whose tile sees no key at all (empty context): zeros
      T* dst = reinterpret_cast<T*>(p.out) + ((int64_t)(q_begin + tok) * p.num_q_heads + hq) * DV;
      for (int c = 0; c < DV; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
    }
    if (ok && row_valid && p.lse_out)
      p.lse_out[(int64_t)hq * p.total_q + q_begin + tok] =
          l_tot > 0.f ? (m_safe * 0.6931471805599453f + logf(l_tot)) : -INFINITY;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int DQK, int DV, int BN>
static void launch_prefill_pp(const PrefillParams& p, const void* q, int64_t q_stride, const void* k_src,
                              const void* v_src, int64_t kv_tok_stride_k, int64_t kv_tok_stride_v, int64_t total_kv,
                              int batch, int max_q_len, cudaStream_t stream) {
  using L = PpSmem<DQK, DV, BN>;
  static_assert(L::kDyn <= 232448, "shared memory budget exceeded");
  static_assert(BN == 64 || BN == 128, "a row of S is held in registers");
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // Q: [T, Hq, DQK], box [128/gp tokens, gp heads, 64]
  uint64_t qd[3] = {(uint64_t)DQK, (uint64_t)p.num_q_heads, (uint64_t)p.total_q};
  uint64_t qs[2] = {(uint64_t)DQK * 2, (uint64_t)q_stride * 2};
  uint32_t qb[3] = {64, (uint32_t)p.gp, (uint32_t)(kPpBM / p.gp)};
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
  auto kern = attn_prefill_pp_kernel<T, DQK, DV, BN>;
  // the shared-memory limit is a per-device attribute of the kernel
  static bool set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set[dev]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
    set[dev] = true;
  }
  const int tpt = kPpBM / p.gp;
  dim3 grid(ceil_div(max_q_len, 2 * tpt), p.num_q_heads / p.gp, batch);
  kern<<<grid, 384, L::kDyn, stream>>>(tmQ, tmK, tmV, p);
}

// Returns 0 on success, -1 when the head sizes are not supported by this kernel.
int attention_prefill_pp(const PrefillParams& p, const void* q, int64_t q_stride, const void* k_src, const void* v_src,
                         int64_t k_tok_stride, int64_t v_tok_stride, int64_t total_kv, int dqk, int dv, int dtype,
                         int batch, int max_q_len, cudaStream_t stream) {
  if (batch <= 0 || max_q_len <= 0) return 0;
#define PF(T)                                                                                                        \
  if (dqk == 128 && dv == 128)                                                                                       \
    launch_prefill_pp<T, 128, 128, 128>(p, q, q_stride, k_src, v_src, k_tok_stride, v_tok_stride, total_kv, batch, max_q_len, stream); \
  else if (dqk == 64 && dv == 64)                                                                                    \
    launch_prefill_pp<T, 64, 64, 128>(p, q, q_stride, k_src, v_src, k_tok_stride, v_tok_stride, total_kv, batch, max_q_len, stream);   \
  else if (dqk == 192 && dv == 128 && !p.paged)                                                                      \
    launch_prefill_pp<T, 192, 128, 64>(p, q, q_stride, k_src, v_src, k_tok_stride, v_tok_stride, total_kv, batch, max_q_len, stream); \
  else                                                                                                               \
    return -1;
  if (dtype == 0) { PF(__nv_bfloat16) } else { PF(__half) }
#undef PF
  return 0;
}

}  // namespace b200
