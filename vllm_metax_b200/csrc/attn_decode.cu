// Paged GQA decode attention (query length 1, or a few tokens for speculative
// decoding / short chunk tails) with split-KV and in-kernel KV dequantisation.
//
// Decode is bound by streaming the KV cache from HBM, so the kernel is organised
// around keeping many independent 16-byte cp.async streams in flight, not around
// tensor-core throughput: each of the 4 warps of a CTA walks its own sequence of
// 16-token tiles through a private 4-stage shared-memory ring and runs the
// FlashAttention-2 recurrence with m16n8k16 MMAs on the (query-token x group-head)
// rows packed into one 16-row tile; the four partial states are merged through
// shared memory at the end.  grid = (kv_head * row_tiles, sequence, kv_split).
// With more than one split the normalised partial outputs and their
// log-sum-exps go to a workspace that `attn_split_reduce` folds.
//
// KV kinds: 0 = same dtype as q; 1 = int8 and 2 = e4m3 with per-(token, head) f32
// scales (dequantised on the fly: K scale multiplies the logit column, V scale is
// folded into P); 3 = e4m3 with static per-tensor scales.
//
// Cache layout [num_blocks, 2, block_size, num_kv_heads, D]; block_size % 16 == 0.
// Replaces flash_attn_with_kvcache (vllm_metax/v1/attention/backends/flash_attn.py:1339-1355)
// and the Triton unified_attention int8 path (triton_attn.py:688-725).
#include <type_traits>
#include "common.cuh"
#include "ops.h"

namespace b200 {

constexpr int kDecWarps = 4;
constexpr int kDecTile = 16;    // tokens per tile
template <int D> __host__ __device__ constexpr int dec_stages() { return 3; }  // D <= 128: ~100 KB per CTA, two CTAs per SM

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  T lo = from_f<T>(a), hi = from_f<T>(b);
  return (uint32_t)(*reinterpret_cast<uint16_t*>(&lo)) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&hi)) << 16);
}


// Eight int8 values -> eight bf16 values without the conversion unit: a byte b (as b ^ 0x80 = b + 128, unsigned)
// dropped into the mantissa of 2^23 gives the float 8388608 + b + 128; subtracting 8388736 leaves b exactly, and a
// float holding an integer of at most 8 significant bits has zero low mantissa bits, so its upper half IS the bf16.
__device__ __forceinline__ uint4 int8x8_to_bf16x8(const uint2 raw) {
  const uint32_t w[2] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u};
  uint32_t out[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      f[i] = __uint_as_float(__byte_perm(w[h], 0x4B000000u, 0x7540 + i)) - 8388736.f;
    out[2 * h] = __byte_perm(__float_as_uint(f[0]), __float_as_uint(f[1]), 0x7632);
    out[2 * h + 1] = __byte_perm(__float_as_uint(f[2]), __float_as_uint(f[3]), 0x7632);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

template <int D, int KIND>
struct DecSmem {
  static constexpr int kDecStages = dec_stages<D>();
  static constexpr int kRowBytes = D * 2;                       // converted (16-bit) row
  static constexpr int kTileBytes = kDecTile * kRowBytes;       // one K or V tile, 16-bit
  static constexpr int kRawRow = (KIND == 0) ? D * 2 : D;       // bytes per token row as stored in the cache
  static constexpr int kRawTile = kDecTile * kRawRow;
  static constexpr int kScaleBytes = (KIND == 1 || KIND == 2) ? 2 * kDecTile * 4 : 0;
  static constexpr int kStageBytes = 2 * kRawTile + kScaleBytes;
  static constexpr int kConvBytes = (KIND == 0) ? 0 : 2 * kTileBytes;  // conversion target (K,V), per warp
  static constexpr int kWarpBytes = kDecStages * kStageBytes + kConvBytes;
  static constexpr int kQBytes = 16 * kRowBytes;
  static constexpr int kMergeBytes = kDecWarps * (16 * D * 4 + 16 * 8);
  static constexpr int kMain = kQBytes + kDecWarps * kWarpBytes;
  static constexpr int kTotal = kMain > kMergeBytes ? kMain : kMergeBytes;
};

template <typename T, int D, int KIND>
__global__ void __launch_bounds__(kDecWarps * 32, (D <= 128 ? 2 : 1)) paged_decode_kernel(const DecodeParams p) {
  using S = DecSmem<D, KIND>;
  constexpr int CPR = D / 8;  // 16-byte chunks per converted row
  constexpr int kDecStages = dec_stages<D>();
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = p.num_q_heads / p.num_kv_heads;
  const int b = blockIdx.y;
  const int split = blockIdx.z;
  const int q_begin = p.query_start_loc ? p.query_start_loc[b] : b;
  const int q_len = p.query_start_loc ? p.query_start_loc[b + 1] - q_begin : 1;
  const int rows_total = q_len * g;
  const int row_tiles = gridDim.x / p.num_kv_heads;
  const int hk = blockIdx.x / row_tiles;
  const int row0 = (blockIdx.x % row_tiles) * 16;
  if (q_len <= 0 || row0 >= rows_total) return;
  int kv_len = p.seq_lens[b];
  // a length the block table cannot hold would index past its row: record it and attend to what the row covers
  const long long kv_cap = (long long)p.max_blocks * p.block_size;
  if (kv_len < 0 || kv_len > kv_cap) {
    report_status(p.status, kBadIndex, 21, (int)(kv_cap > 0x7fffffff ? 0x7fffffff : kv_cap), kv_len);
    kv_len = kv_len < 0 ? 0 : (int)kv_cap;
  }
  // tiles of this split
  const int tiles_total = (kv_len + kDecTile - 1) / kDecTile;
  const int tiles_per_split = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + tiles_per_split);

  uint8_t* q_smem = smem;
  uint8_t* wbase = smem + S::kQBytes + warp * S::kWarpBytes;
  const int* btab = p.block_table + (int64_t)b * p.max_blocks;

  // ---- stage Q rows (zero for rows beyond rows_total), swizzled 16-byte chunks
  {
    const T* qb = reinterpret_cast<const T*>(p.q);
    for (int idx = threadIdx.x; idx < 16 * CPR; idx += blockDim.x) {
      const int r = idx / CPR, c = idx % CPR;
      const int rr = row0 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (rr < rows_total) {
        const int tok = q_begin + rr / g, hq = hk * g + rr % g;
        v = *reinterpret_cast<const uint4*>(qb + (int64_t)tok * p.q_stride + (int64_t)hq * D + c * 8);
      }
      *reinterpret_cast<uint4*>(q_smem + r * S::kRowBytes + ((c ^ (r & 7)) * 16)) = v;
    }
  }
  __syncthreads();
  // Q fragments for all k-steps
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int mat = lane >> 3;
    const int r = (mat & 1) * 8 + (lane & 7);
    const int c = 2 * ks + (mat >> 1);
    ldmatrix_x4(qf[ks], q_smem + r * S::kRowBytes + ((c ^ (r & 7)) * 16));
  }

  // per-row causal limits: row r (token i = r / g) sees kv positions < limit
  const int rA = row0 + (lane >> 2), rB = rA + 8;
  auto row_limit = [&](int r) -> int {
    if (r >= rows_total) return 0;
    return p.causal ? (kv_len - q_len + r / g + 1) : kv_len;
  };
  const int limA = row_limit(rA), limB = row_limit(rB);
  const int loA = (p.window > 0) ? max(0, limA - p.window) : 0;
  const int loB = (p.window > 0) ? max(0, limB - p.window) : 0;
  // ALiBi: bias = slope[head of the row] * (kv position - query position), in log2 units like the scores
  const float alA = (p.alibi_slopes && rA < rows_total) ? p.alibi_slopes[hk * g + rA % g] * 1.4426950408889634f : 0.f;
  const float alB = (p.alibi_slopes && rB < rows_total) ? p.alibi_slopes[hk * g + rB % g] * 1.4426950408889634f : 0.f;

  const float sm_scale_log2 = p.scale * 1.4426950408889634f * ((KIND == 3) ? p.k_scale : 1.f);
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  // ---- per-warp tile pipeline
  auto issue = [&](int tile, int stage) {
    uint8_t* st = wbase + stage * S::kStageBytes;
    const bool tile_ok = tile < tile_end;
    const int tok0 = tile * kDecTile;
    int page = 0;
    if (tile_ok) {
      page = btab[tok0 / p.block_size];
      if (page < 0 || page >= p.num_blocks) {
        report_status(p.status, kBadIndex, 20, (int)p.num_blocks, page);
        page = 0;
      }
    }
    const int off0 = tok0 % p.block_size;
    constexpr int RAW_CPR = S::kRawRow / 16;
    const uint8_t* cache = reinterpret_cast<const uint8_t*>(p.kv_cache);
#pragma unroll
    for (int kv = 0; kv < 2; ++kv) {
      const int64_t row_base = (((int64_t)page * 2 + kv) * p.block_size + off0) * p.num_kv_heads + hk;
      for (int idx = lane; idx < kDecTile * RAW_CPR; idx += 32) {
        const int r = idx / RAW_CPR, c = idx % RAW_CPR;
        const bool ok = tile_ok && (tok0 + r) < kv_len;
        const uint8_t* src = cache + (row_base + (int64_t)r * p.num_kv_heads) * S::kRawRow + c * 16;
        // 16-bit tiles are stored swizzled directly; raw 8-bit tiles are stored linearly
        const int dst_c = (KIND == 0) ? (c ^ (r & 7)) : c;
        cp_async16(st + kv * S::kRawTile + r * S::kRawRow + dst_c * 16, ok ? src : cache, ok);
      }
      if constexpr (KIND == 1 || KIND == 2) {
        if (lane < kDecTile) {
          const bool ok = tile_ok && (tok0 + lane) < kv_len;
          const float* src = p.kv_scales + row_base + (int64_t)lane * p.num_kv_heads;
          cp_async4(st + 2 * S::kRawTile + (kv * kDecTile + lane) * 4, ok ? src : p.kv_scales, ok);
        }
      }
    }
  };

  int my_tile = tile_begin + warp;
#pragma unroll
  for (int s = 0; s < kDecStages - 1; ++s) {
    issue(my_tile + s * kDecWarps, s);
    cp_async_commit();
  }
  int stage = 0;
  for (int tile = my_tile; tile < tile_end; tile += kDecWarps) {
    // prefetch the tile STAGES-1 ahead into the slot consumed in the previous iteration
    issue(tile + (kDecStages - 1) * kDecWarps, (stage + kDecStages - 1) % kDecStages);
    cp_async_commit();
    cp_async_wait<kDecStages - 1>();
    __syncwarp();
    uint8_t* st = wbase + stage * S::kStageBytes;
    const uint8_t* k_tile;
    const uint8_t* v_tile;
    float ksc[4] = {1.f, 1.f, 1.f, 1.f}, vsc[4] = {1.f, 1.f, 1.f, 1.f};
    if constexpr (KIND == 0) {
      k_tile = st;
      v_tile = st + S::kRawTile;
    } else {
      // convert the raw 8-bit tiles into swizzled 16-bit tiles
      uint8_t* conv = wbase + kDecStages * S::kStageBytes;
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        for (int idx = lane; idx < kDecTile * CPR; idx += 32) {
          const int r = idx / CPR, c = idx % CPR;
          const uint2 raw = *reinterpret_cast<const uint2*>(st + kv * S::kRawTile + r * S::kRawRow + c * 8);
          uint4 packed;
          if constexpr (KIND == 1 && std::is_same<T, __nv_bfloat16>::value) {
            packed = int8x8_to_bf16x8(raw);           // integer ALU only: no conversion-unit instruction
          } else {
            const uint8_t* rb = reinterpret_cast<const uint8_t*>(&raw);
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = (KIND == 1) ? (float)(int8_t)rb[i] : fp8_e4m3_to_float(rb[i]);
            packed = pack8<T>(f);
          }
          *reinterpret_cast<uint4*>(conv + kv * S::kTileBytes + r * S::kRowBytes + ((c ^ (r & 7)) * 16)) = packed;
        }
      }
      if constexpr (KIND == 1 || KIND == 2) {
        const float* sc = reinterpret_cast<const float*>(st + 2 * S::kRawTile);
        const int c0 = 2 * (lane & 3);
        ksc[0] = sc[c0]; ksc[1] = sc[c0 + 1]; ksc[2] = sc[8 + c0]; ksc[3] = sc[8 + c0 + 1];
        vsc[0] = sc[16 + c0]; vsc[1] = sc[16 + c0 + 1]; vsc[2] = sc[24 + c0]; vsc[3] = sc[24 + c0 + 1];
      }
      __syncwarp();
      k_tile = conv;
      v_tile = conv + S::kTileBytes;
    }
    // ---- S = Q K^T  (16 rows x 16 tokens)
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t kf[4];
      const int mat = lane >> 3;
      const int r = (mat >> 1) * 8 + (lane & 7);
      const int c = 2 * ks + (mat & 1);
      ldmatrix_x4(kf, k_tile + r * S::kRowBytes + ((c ^ (r & 7)) * 16));
      mma16816<T>(s[0], qf[ks], kf[0], kf[1]);
      mma16816<T>(s[1], qf[ks], kf[2], kf[3]);
    }
    // ---- scale, soft-cap, mask
    const int tok0 = tile * kDecTile;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = tok0 + nt * 8 + 2 * (lane & 3) + (e & 1);
        const int half = e >> 1;  // 0: row A, 1: row B
        float v = s[nt][e] * ksc[nt * 2 + (e & 1)];
        if (p.softcap > 0.f) {
          v = p.softcap * tanhf(v * p.scale * ((KIND == 3) ? p.k_scale : 1.f) / p.softcap) * 1.4426950408889634f;
        } else {
          v *= sm_scale_log2;
        }
        const int lim = half ? limB : limA, lo = half ? loB : loA;
        v += (half ? alB : alA) * (float)(col - (lim - 1));
        if (col >= lim || col < lo) v = -INFINITY;
        s[nt][e] = v;
        mx[half] = fmaxf(mx[half], v);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float mnew = fmaxf(m_run[h], mx[h]);
      msafe[h] = (mnew == -INFINITY) ? 0.f : mnew;
      corr[h] = exp2f(m_run[h] - msafe[h]);  // m_run = -inf -> 0
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
          const float pe = exp2f(s[nt][e] - msafe[e >> 1]);
          rs[e >> 1] += pe;
          pv[nt][e] = pe * vsc[nt * 2 + (e & 1)];
        }
      pf[0] = pack2<T>(pv[0][0], pv[0][1]);
      pf[1] = pack2<T>(pv[0][2], pv[0][3]);
      pf[2] = pack2<T>(pv[1][0], pv[1][1]);
      pf[3] = pack2<T>(pv[1][2], pv[1][3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
      l_run[h] = l_run[h] * corr[h] + rs[h];
    }
    // ---- O = O * corr + P V  (the rescale is skipped when no row of the warp raised its max)
    const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f);
    if (rescale) {
#pragma unroll
      for (int nd = 0; nd < D / 8; ++nd) {
        o[nd][0] *= corr[0]; o[nd][1] *= corr[0]; o[nd][2] *= corr[1]; o[nd][3] *= corr[1];
      }
    }
#pragma unroll
    for (int nd = 0; nd < D / 8; nd += 2) {
      uint32_t vf[4];
      const int mat = lane >> 3;
      const int r = (mat & 1) * 8 + (lane & 7);
      const int c = nd + (mat >> 1);
      ldmatrix_x4_trans(vf, v_tile + r * S::kRowBytes + ((c ^ (r & 7)) * 16));
      mma16816<T>(o[nd], pf, vf[0], vf[1]);
      mma16816<T>(o[nd + 1], pf, vf[2], vf[3]);
    }
    __syncwarp();
    stage = (stage + 1) % kDecStages;
  }
  cp_async_wait<0>();
  __syncthreads();  // all warps done with the tile rings; shared memory is reused for the merge

  // ---- cross-warp merge
  float* mo = reinterpret_cast<float*>(smem);                 // [warps][16][D]
  float* mm = mo + kDecWarps * 16 * D;                        // [warps][16] running max (log2 domain)
  float* ml = mm + kDecWarps * 16;                            // [warps][16] running sum
  {
    const int ra = lane >> 2, rb = ra + 8;
    if ((lane & 3) == 0) {
      mm[warp * 16 + ra] = m_run[0]; mm[warp * 16 + rb] = m_run[1];
      ml[warp * 16 + ra] = l_run[0]; ml[warp * 16 + rb] = l_run[1];
    }
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd) {
      const int col = nd * 8 + 2 * (lane & 3);
      float* base = mo + warp * 16 * D;
      base[ra * D + col] = o[nd][0]; base[ra * D + col + 1] = o[nd][1];
      base[rb * D + col] = o[nd][2]; base[rb * D + col + 1] = o[nd][3];
    }
  }
  __syncthreads();
  const float out_scale = (KIND == 3) ? p.v_scale : 1.f;
  for (int idx = threadIdx.x; idx < 16 * D; idx += blockDim.x) {
    const int r = idx / D, c = idx % D;
    const int rr = row0 + r;
    if (rr >= rows_total) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, mm[w * 16 + r]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float f = exp2f(mm[w * 16 + r] - Ms);
      L += ml[w * 16 + r] * f;
      acc += mo[(w * 16 + r) * D + c] * f;
    }
    const int tok = q_begin + rr / g, hq = hk * g + rr % g;
    if (p.num_splits == 1) {
      float Lt = L;
      if (p.sinks) Lt += exp2f(p.sinks[hq] * 1.4426950408889634f - Ms);
      const float v = Lt > 0.f ? acc / Lt * out_scale : 0.f;
      reinterpret_cast<T*>(p.out)[((int64_t)tok * p.num_q_heads + hq) * D + c] = from_f<T>(v);
      if (c == 0 && p.lse_out)
        p.lse_out[(int64_t)hq * p.total_tokens + tok] = Lt > 0.f ? (Ms * 0.6931471805599453f + logf(Lt)) : -INFINITY;
    } else {
      const int64_t prow = ((int64_t)split * p.total_tokens + tok) * p.num_q_heads + hq;
      p.part_out[prow * D + c] = L > 0.f ? acc / L * out_scale : 0.f;
      if (c == 0) p.part_lse[prow] = L > 0.f ? (Ms * 0.6931471805599453f + logf(L)) : -INFINITY;
    }
  }
}

// out[t,h,:] = sum_s part_out[s,t,h,:] * exp(lse_s - LSE), LSE = logsumexp_s (+ sink)
template <typename T>
__global__ void attn_split_reduce_kernel(T* __restrict__ out, float* __restrict__ lse_out,
                                         const float* __restrict__ part_out, const float* __restrict__ part_lse,
                                         const float* __restrict__ sinks, int num_splits, int total_tokens, int heads,
                                         int D) {
  const int64_t row = blockIdx.x;  // token * heads + head
  const int hq = (int)(row % heads);
  const int64_t tok = row / heads;
  const int64_t stride = (int64_t)total_tokens * heads;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_lse[s * stride + row]);
  if (sinks) M = fmaxf(M, sinks[hq]);
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < num_splits; ++s) L += __expf(part_lse[s * stride + row] - Ms);
  const float Lk = L;
  if (sinks) L += __expf(sinks[hq] - Ms);
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s)
      acc += part_out[(s * stride + row) * D + c] * __expf(part_lse[s * stride + row] - Ms);
    out[row * D + c] = from_f<T>(L > 0.f ? acc / L : 0.f);
  }
  (void)Lk;
  if (threadIdx.x == 0 && lse_out) lse_out[(int64_t)hq * total_tokens + tok] = L > 0.f ? Ms + logf(L) : -INFINITY;
}

template <typename T, int D, int KIND>
static void launch_decode(const DecodeParams& p, int batch, int max_q_len, cudaStream_t stream) {
  using S = DecSmem<D, KIND>;
  auto kern = paged_decode_kernel<T, D, KIND>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
  const int g = p.num_q_heads / p.num_kv_heads;
  const int row_tiles = ceil_div(max_q_len * g, 16);
  dim3 grid(p.num_kv_heads * row_tiles, batch, p.num_splits);
  kern<<<grid, kDecWarps * 32, S::kTotal, stream>>>(p);
  if (p.num_splits > 1) {
    const int64_t rows = (int64_t)p.total_tokens * p.num_q_heads;
    attn_split_reduce_kernel<T><<<(unsigned)rows, D <= 128 ? 128 : 256, 0, stream>>>(
        (T*)p.out, p.lse_out, p.part_out, p.part_lse, p.sinks, p.num_splits, p.total_tokens, p.num_q_heads, D);
  }
}

template <typename T, int D>
static void decode_kind(const DecodeParams& p, int kind, int batch, int max_q_len, cudaStream_t stream) {
  switch (kind) {
    case 0: launch_decode<T, D, 0>(p, batch, max_q_len, stream); break;
    case 1: launch_decode<T, D, 1>(p, batch, max_q_len, stream); break;
    case 2: launch_decode<T, D, 2>(p, batch, max_q_len, stream); break;
    default: launch_decode<T, D, 3>(p, batch, max_q_len, stream); break;
  }
}

// Returns 0 on success, -1 for an unsupported head size.
int paged_attention_decode(const DecodeParams& p, int head_dim, int kv_kind, int dtype, int batch, int max_q_len,
                           cudaStream_t stream) {
  if (batch <= 0) return 0;
#define DISPATCH_D(T)                                                             \
  if (head_dim == 64) decode_kind<T, 64>(p, kv_kind, batch, max_q_len, stream);   \
  else if (head_dim == 128) decode_kind<T, 128>(p, kv_kind, batch, max_q_len, stream); \
  else if (head_dim == 256) decode_kind<T, 256>(p, kv_kind, batch, max_q_len, stream); \
  else return -1;
  if (dtype == 0) { DISPATCH_D(__nv_bfloat16) } else { DISPATCH_D(__half) }
#undef DISPATCH_D
  return 0;
}

}  // namespace b200
