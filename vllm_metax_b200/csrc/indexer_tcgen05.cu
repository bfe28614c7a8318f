// Sparse-attention indexer logits on the 5th-generation tensor cores.
//
//   logits[t, n] = k_scale[n] * sum_h w[t, h] * relu(q[t, h, :] . k[n, :])     n < limit(t), else -inf
//
// q [T, heads, 128] and the cached keys are 8-bit (e4m3 -> kind::f8f6f4, or int8 -> kind::i8), so one key row and one
// (token, head) row are exactly one 128-byte swizzle atom.  One CTA owns a tile of 128 keys of one request (UMMA M, read
// once from the paged, block-planar key cache by TMA: one box per page) and streams the request's query tokens past
// it in groups of 256 / heads tokens (UMMA N = up to 256 (token, head) rows, K = 128 bytes = 4 instructions).  The
// [128 keys x 256] fp32 (s32) accumulator lives in TMEM, double-buffered; the four epilogue warps (one thread per key)
// read it back 32 columns at a time, apply ReLU and the per-(token, head) weight, sum over the heads of each token,
// scale by the key's scale and store one logit per (token, key) - so the [keys x tokens x heads] products never
// leave the SM.  Causal limits skip whole token groups that cannot see the tile; those and the tiles beyond a
// request's length are filled with -inf for the top-k pass.
//
// A CTA walks through up to 16 consecutive key tiles (two key stages), so that decode steps - one token per request,
// thousands of tiles - amortise barrier and TMEM set-up.
// Warp roles: 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2..9 = epilogue (two warps per TMEM lane quarter, which
// split the tokens of a group).  Every wait is bounded.
// Replaces deep_gemm fp8_mqa_logits / fp8_paged_mqa_logits of the reference (vllm_metax/utils/deep_gemm.py:306-401,
// registry/custom_ops/layers/sparse_attn_indexer/fp8.py:219-228, 308-370).
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {

using namespace ptx;

constexpr int kIxKeys = 128, kIxD = 128, kIxStages = 4, kIxKStages = 2;
constexpr int kIxQBytes = 256 * kIxD;              // one stage of (token, head) rows
constexpr int kIxKBytes = kIxKeys * kIxD;
constexpr int kIxEpiThreads = 256;                 // two warps per TMEM lane quarter: they split the tokens of a group

struct IxParams {
  float* logits;
  int64_t stride;                 // row stride of logits (>= padded length)
  const float* w;                 // [T, heads]
  const uint8_t* cache;           // [num_blocks, block_size * 132]
  const int* block_table;
  int max_blocks;
  const int* seq_lens;
  const int* query_start_loc;
  int tokens, batch, heads, block_size, num_blocks;
  int group_tokens;               // tokens per MMA (heads * group_tokens <= 256)
  int chunks;                     // gridDim.z: the token groups of a request are cut into this many ranges
  int tiles_per_cta;              // consecutive key tiles one CTA walks through
  int num_tiles;                  // stride / 128
  StatusWord* status;
};

struct IxSmem {
  static constexpr int kK = 0;
  static constexpr int kQ = kIxKStages * kIxKBytes;
  static constexpr int kW = kQ + kIxStages * kIxQBytes;         // 2 x 256 floats
  static constexpr int kBars = kW + 2 * 256 * 4;
  static constexpr int kTotal = kBars + 24 * 8 + 16;
};

template <bool INT8>
__global__ void __launch_bounds__(64 + kIxEpiThreads)
indexer_logits_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                         const IxParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + IxSmem::kBars);
  uint64_t* k_full = bars;
  uint64_t* k_empty = k_full + kIxKStages;
  uint64_t* q_full = k_empty + kIxKStages;
  uint64_t* q_empty = q_full + kIxStages;
  uint64_t* tmem_full = q_empty + kIxStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  float* s_w = reinterpret_cast<float*>(smem + IxSmem::kW);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y;
  const int q0 = p.query_start_loc[b], qlen = p.query_start_loc[b + 1] - q0;
  const int L = p.seq_lens[b];
  const int G = p.group_tokens, heads = p.heads;
  const int n_groups = (qlen + G - 1) / G;
  const int per_chunk = (n_groups + p.chunks - 1) / p.chunks;
  const int g_begin = blockIdx.z * per_chunk, g_end = min(n_groups, g_begin + per_chunk);
  if (qlen <= 0 || g_begin >= g_end) return;
  const int tile_begin = blockIdx.x * p.tiles_per_cta;
  const int tile_end = min(p.num_tiles, tile_begin + p.tiles_per_cta);
  // token i of the request sees keys n < L - qlen + i + 1.  For the tile that starts at key n0 the groups
  // [first_group(n0), g_end) need the tensor cores; a tile is "live" when that range is not empty.
  auto first_group = [&](int n0) { return max(g_begin, min(g_end, max(0, n0 - (L - qlen)) / G)); };
  auto live = [&](int n0) { return n0 < L && first_group(n0) < g_end; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kIxKStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < kIxStages; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], kIxEpiThreads);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int box_rows = p.block_size < kIxKeys ? p.block_size : kIxKeys;
      const int* btab = p.block_table + (int64_t)b * p.max_blocks;
      int ks = 0, stage = 0;
      uint32_t kphase = 0, phase = 0;
      bool ok = true;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        const int n0 = tile * kIxKeys;
        if (!live(n0)) continue;
        if (!mbar_wait(&k_empty[ks], kphase ^ 1)) {
          report_status(p.status, kWaitTimeout, 206, tile, ks);
          break;
        }
        // keys: one box per page (or one box of 128 rows inside a larger page)
        uint32_t bytes = 0;
        for (int r = 0; r < kIxKeys; r += box_rows)
          if (n0 + r < L) bytes += (uint32_t)box_rows * kIxD;
        mbar_expect_tx(&k_full[ks], bytes);
        for (int r = 0; r < kIxKeys; r += box_rows) {
          const int n = n0 + r;
          if (n >= L) break;
          int page = btab[n / p.block_size];
          if (page < 0 || page >= p.num_blocks) {
            report_status(p.status, kBadIndex, 200, p.num_blocks, page);
            page = 0;
          }
          tma_load_3d(smem + IxSmem::kK + ks * kIxKBytes + r * kIxD, &tmK, &k_full[ks], 0, n % p.block_size, page);
        }
        if (++ks == kIxKStages) { ks = 0; kphase ^= 1; }
        for (int g = first_group(n0); g < g_end; ++g) {
          if (!mbar_wait(&q_empty[stage], phase ^ 1)) {
            report_status(p.status, kWaitTimeout, 201, g, stage);
            ok = false;
            break;
          }
          mbar_expect_tx(&q_full[stage], (uint32_t)(G * heads * kIxD));
          tma_load_2d(smem + IxSmem::kQ + stage * kIxQBytes, &tmQ, &q_full[stage], 0, (q0 + g * G) * heads);
          if (++stage == kIxStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t N = (uint32_t)(G * heads);
      const uint32_t idesc = INT8 ? make_idesc(2, 1, 1, kIxKeys, N) : make_idesc(1, 0, 0, kIxKeys, N);
      int ks = 0, stage = 0, it = 0;
      uint32_t kphase = 0, phase = 0;
      bool ok = true;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        const int n0 = tile * kIxKeys;
        if (!live(n0)) continue;
        if (!mbar_wait(&k_full[ks], kphase)) {
          report_status(p.status, kWaitTimeout, 202, tile, b);
          break;
        }
        tc_fence_after_sync();
        const uint64_t da = make_smem_desc_sw128(smem_u32(smem + IxSmem::kK + ks * kIxKBytes));
        for (int g = first_group(n0); g < g_end; ++g, ++it) {
          const int acc = it & 1;
          if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
            report_status(p.status, kWaitTimeout, 203, g, acc);
            ok = false;
            break;
          }
          if (!mbar_wait(&q_full[stage], phase)) {
            report_status(p.status, kWaitTimeout, 204, g, stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t db = make_smem_desc_sw128(smem_u32(smem + IxSmem::kQ + stage * kIxQBytes));
          const uint32_t d_tmem = tmem_base + acc * 256;
#pragma unroll
          for (int k = 0; k < kIxD / 32; ++k) {
            if (INT8) umma_i8_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k != 0 ? 1u : 0u);
            else umma_f8_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k != 0 ? 1u : 0u);
          }
          umma_commit(&q_empty[stage]);
          umma_commit(&tmem_full[acc]);
          if (++stage == kIxStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&k_empty[ks]);             // the tile's MMAs have read the keys
        if (++ks == kIxKStages) { ks = 0; kphase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;                    // which tokens of a group this warp sums (j % 2 == half)
    const int row = quarter * 32 + lane;                 // key of this thread inside the tile
    const int et = threadIdx.x - 64;                     // 0..255 among the epilogue threads
    const int64_t w_total = (int64_t)p.tokens * heads;
    int it = 0;
    bool ok = true;
    for (int tile = tile_begin; tile < tile_end; ++tile) {
      const int n0 = tile * kIxKeys;
      const int n = n0 + row;
      const bool col_ok = n < p.stride;
      const bool is_live = live(n0);
      // groups that cannot see this tile (and whole tiles beyond the request): -inf
      const int g_fill_end = is_live ? first_group(n0) : g_end;
      for (int g = g_begin; g < g_fill_end; ++g)
        for (int j = half; j < G; j += 2) {
          const int i = g * G + j;
          if (i < qlen && col_ok) p.logits[(int64_t)(q0 + i) * p.stride + n] = -INFINITY;
        }
      if (!is_live) continue;
      float k_scale = 0.f;
      if (n < L) {
        const int page = p.block_table[(int64_t)b * p.max_blocks + n / p.block_size];
        if (page >= 0 && page < p.num_blocks)
          k_scale = *reinterpret_cast<const float*>(p.cache + (int64_t)page * p.block_size * (kIxD + 4) +
                                                    (int64_t)p.block_size * kIxD + (n % p.block_size) * 4);
      }
      for (int g = first_group(n0); g < g_end; ++g, ++it) {
        const int acc = it & 1;
        float* wbuf = s_w + acc * 256;
        const int64_t wbase = (int64_t)(q0 + g * G) * heads;
        if (et < G * heads) wbuf[et] = (wbase + et < w_total) ? p.w[wbase + et] : 0.f;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        // after a timeout every thread still walks all iterations (same named-barrier count), without waiting again
        if (ok && !mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
          report_status(p.status, kWaitTimeout, 205, g, acc);
          ok = false;
        }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
        for (int j = half; j < G && ok; j += 2) {
          float sum = 0.f;
          for (int c = 0; c < heads; c += 64) {
            // 64 columns in flight (heads is a multiple of 32; the second half may fall outside the token)
            uint32_t r0[32], r1[32];
            const bool two = c + 32 < heads;
            tmem_ld_32x32b_x32(taddr + j * heads + c, r0);
            if (two) tmem_ld_32x32b_x32(taddr + j * heads + c + 32, r1);
            tmem_ld_wait();
            const float4* wj = reinterpret_cast<const float4*>(wbuf + j * heads + c);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float4 w4 = wj[e];
              const float v0 = INT8 ? (float)max((int)r0[4 * e + 0], 0) : fmaxf(__uint_as_float(r0[4 * e + 0]), 0.f);
              const float v1 = INT8 ? (float)max((int)r0[4 * e + 1], 0) : fmaxf(__uint_as_float(r0[4 * e + 1]), 0.f);
              const float v2 = INT8 ? (float)max((int)r0[4 * e + 2], 0) : fmaxf(__uint_as_float(r0[4 * e + 2]), 0.f);
              const float v3 = INT8 ? (float)max((int)r0[4 * e + 3], 0) : fmaxf(__uint_as_float(r0[4 * e + 3]), 0.f);
              sum = fmaf(v0, w4.x, fmaf(v1, w4.y, fmaf(v2, w4.z, fmaf(v3, w4.w, sum))));
            }
            if (two) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float4 w4 = wj[8 + e];
                const float v0 = INT8 ? (float)max((int)r1[4 * e + 0], 0) : fmaxf(__uint_as_float(r1[4 * e + 0]), 0.f);
                const float v1 = INT8 ? (float)max((int)r1[4 * e + 1], 0) : fmaxf(__uint_as_float(r1[4 * e + 1]), 0.f);
                const float v2 = INT8 ? (float)max((int)r1[4 * e + 2], 0) : fmaxf(__uint_as_float(r1[4 * e + 2]), 0.f);
                const float v3 = INT8 ? (float)max((int)r1[4 * e + 3], 0) : fmaxf(__uint_as_float(r1[4 * e + 3]), 0.f);
                sum = fmaf(v0, w4.x, fmaf(v1, w4.y, fmaf(v2, w4.z, fmaf(v3, w4.w, sum))));
              }
            }
          }
          const int i = g * G + j;
          if (i < qlen && col_ok) {
            const int lim = L - qlen + i + 1;
            p.logits[(int64_t)(q0 + i) * p.stride + n] = (n < lim) ? sum * k_scale : -INFINITY;
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&tmem_empty[acc]);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Returns 0, or -1 when the shapes are not served by this kernel (the caller falls back to the mma.sync kernel).
int indexer_logits_tc(float* logits, int64_t logits_stride, const void* q, const float* w, const void* cache,
                      const int* block_table, int max_blocks, const int* seq_lens, const int* query_start_loc,
                      int tokens, int batch, int heads, int block_size, int64_t num_blocks, int max_len,
                      int max_query_len, void* status, cudaStream_t stream, int kind) {
  if (tokens <= 0 || max_len <= 0) return 0;
  if (kind != 0 && kind != 1) return -1;
  if (heads % 32 != 0 || heads > 256 || 256 % heads != 0) return -1;
  const bool bs_ok = block_size >= 8 && ((block_size <= 128 && 128 % block_size == 0) || block_size % 128 == 0);
  if (!bs_ok || (reinterpret_cast<uintptr_t>(cache) & 15) != 0 || (reinterpret_cast<uintptr_t>(q) & 15) != 0) return -1;
  if (((int64_t)block_size * (kIxD + 4)) % 16 != 0 || logits_stride % kIxKeys != 0) return -1;
  int G = 256 / heads;
  if (max_query_len > 0 && max_query_len < G) G = max_query_len;
  const int N = G * heads;
  if (N % 16 != 0 || N < 16) return -1;

  // keys: [num_blocks][block_size rows][128 bytes], pages block_size * 132 bytes apart
  const uint64_t kd[3] = {(uint64_t)kIxD, (uint64_t)block_size, (uint64_t)num_blocks};
  const uint64_t ks[2] = {(uint64_t)kIxD, (uint64_t)block_size * (kIxD + 4)};
  const uint32_t kb[3] = {(uint32_t)kIxD, (uint32_t)(block_size < kIxKeys ? block_size : kIxKeys), 1u};
  const CUtensorMap tmK = make_tmap_nd(cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, kd, ks, kb, CU_TENSOR_MAP_SWIZZLE_128B);
  const uint64_t qd[2] = {(uint64_t)kIxD, (uint64_t)tokens * heads};
  const uint64_t qs[1] = {(uint64_t)kIxD};
  const uint32_t qb[2] = {(uint32_t)kIxD, (uint32_t)N};
  const CUtensorMap tmQ = make_tmap_nd(q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, qd, qs, qb, CU_TENSOR_MAP_SWIZZLE_128B);

  IxParams p{};
  p.logits = logits; p.stride = logits_stride; p.w = w; p.cache = (const uint8_t*)cache;
  p.block_table = block_table; p.max_blocks = max_blocks; p.seq_lens = seq_lens; p.query_start_loc = query_start_loc;
  p.tokens = tokens; p.batch = batch; p.heads = heads; p.block_size = block_size; p.num_blocks = (int)num_blocks;
  p.group_tokens = G;
  const int tiles = (int)(logits_stride / kIxKeys);
  const int avg_groups = ((tokens + batch - 1) / batch + G - 1) / G;
  // token-group ranges per request when there are too few (request, tile) pairs to fill the GPU; several key tiles
  // per CTA when there are too many (decode: a CTA then amortises its set-up over up to 16 tiles)
  int chunks = (2 * 148 + tiles * batch - 1) / (tiles * batch);
  chunks = chunks < 1 ? 1 : (chunks > avg_groups ? avg_groups : chunks);
  if (chunks > 64) chunks = 64;
  int tpc = (int)(((int64_t)tiles * batch * chunks + 4 * 148 - 1) / (4 * 148));
  tpc = tpc < 1 ? 1 : (tpc > 16 ? 16 : tpc);
  p.chunks = chunks;
  p.tiles_per_cta = tpc;
  p.num_tiles = tiles;
  p.status = (StatusWord*)status;
  const dim3 grid((tiles + tpc - 1) / tpc, batch, chunks);
  constexpr int kThreads = 64 + kIxEpiThreads;
  if (kind == 1) {
    cudaFuncSetAttribute(indexer_logits_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, IxSmem::kTotal);
    indexer_logits_tc_kernel<true><<<grid, kThreads, IxSmem::kTotal, stream>>>(tmK, tmQ, p);
  } else {
    cudaFuncSetAttribute(indexer_logits_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, IxSmem::kTotal);
    indexer_logits_tc_kernel<false><<<grid, kThreads, IxSmem::kTotal, stream>>>(tmK, tmQ, p);
  }
  return 0;
}

}  // namespace b200
