// Weight-only quantised GEMM (W4A16 / W8A16, group scales + zero points) on tcgen05, dense and grouped:
//
//     C[m, n] = sum_k A[m, k] * ( (Q[n, k] - Z[k/g, n]) * S[k/g, n] )
//
// The packed weights never exist in 16-bit form in global memory.  Per pipeline stage
//   warp 0      TMA: packed weight tile (128 rows x 64 k = 32 or 64 bytes per row, unswizzled) and the
//               activation tile (BN tokens x 64 k, 128B-swizzled)
//   warps 2-5   dequantise: one thread per weight row turns its 64 packed values into bf16/fp16 with the
//               exponent-splice trick (0x4300|q is exactly 128+q in bf16, 0x6400|q is 1024+q in fp16),
//               subtracts the equally biased zero point, multiplies by the group scale and writes the
//               128B-swizzled K-major tile the tensor core reads
//   warp 1      one thread issues tcgen05.mma with the WEIGHT tile as the 128-row operand and the tokens
//               as the N operand (BN = 16..256), so decode batches do not waste a 128-row tile
//   warps 6-9   epilogue from TMEM (two accumulator buffers), transposed store, optional bias, optional
//               SiLU-gate over interleaved (gate, up) rows, or fp32 partials for split-K
// Split-K (gridDim.y) keeps all SMs streaming weights when tokens x N gives few tiles.
// Packed layout (made once at load by the quant methods): Q uint8 [(E,) N, K*bits/8]; within each
// 32-bit word of a 4-bit row the nibble order is e0 e2 e4 e6 e1 e3 e5 e7 so that
// (word >> 4j) & 0x000F000F yields the pair (e2j, e2j+1) in the two 16-bit halves.  S and Z are
// [(E,) K/g, N] in the activation dtype; Z holds zero_point + 128 (bf16) / + 1024 (fp16) for 4 bits and the
// plain zero point for 8 bits.
// Replaces the exllama GPTQ / AWQ GEMMs, Marlin-style kernels and the WNA16 fused-MoE kernels
// (csrc/quantization/gptq/q_gemm.cu, awq/gemm_kernels.cu, csrc/moe/moe_wna16.cu and
// model_executor/layers/fused_moe/fused_moe.py:78-310 of the reference).
#include <type_traits>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kWqBM = 128, kWqBK = 64;

template <int BN, int STAGES, int BITS>
struct WqLayout {
  static constexpr int kPackedRow = kWqBK * BITS / 8;            // 32 or 64 bytes
  static constexpr int kPackedBytes = kWqBM * kPackedRow;
  static constexpr int kABytes = kWqBM * kWqBK * 2;              // dequantised weight tile
  static constexpr int kXBytes = BN * kWqBK * 2;
  static constexpr int kStageBytes = kPackedBytes + kABytes + kXBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kDyn = kBarOffset + (3 * STAGES + 4) * 8 + 16 + 1024;
};

struct WqArgs {
  const void* scales;
  const void* zeros;
  const void* bias;
  float* partial;           // [splits, M, N] fp32 when splits > 1
  const int* block_expert;
  const int* total_padded;
  int M, N, K, ldc, group, num_experts, epi, splits;
};

template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> { using type = __nv_bfloat162; static constexpr uint32_t magic = 0x43004300u; };
template <> struct Pair16<__half> { using type = __half2; static constexpr uint32_t magic = 0x64006400u; };

template <typename T, int BN, int STAGES, int BITS, bool GROUPED>
__global__ void __launch_bounds__(320, 1)
gemm_wna16_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmX,
                  T* __restrict__ C, const WqArgs p, StatusWord* status) {
  using L = WqLayout<BN, STAGES, BITS>;
  using T2 = typename Pair16<T>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* ready_bar = full_bar + STAGES;
  uint64_t* empty_bar = ready_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = GROUPED ? *p.total_padded : p.M;
  const int num_w = ceil_div(p.N, kWqBM);
  const int num_t = ceil_div(rows, BN);
  const int num_tiles = num_w * num_t;
  const int num_k_all = ceil_div(p.K, kWqBK);
  const int k_per = ceil_div(num_k_all, p.splits);
  const int kb0 = blockIdx.y * k_per;
  const int kb1 = min(num_k_all, kb0 + k_per);
  const int num_k = max(0, kb1 - kb0);
  const int ngroups = p.K / p.group;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&ready_bar[s], 128);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto expert_of = [&](int tt) -> int {
    if (!GROUPED) return 0;
    int e = p.block_expert[tt];
    return (e < 0 || e >= p.num_experts) ? 0 : e;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tt = tile % num_t, tw = tile / num_t;   // concurrent CTAs share the weight tile
        const int e = expert_of(tt);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 120, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sq = smem + stage * L::kStageBytes;
          uint8_t* sx = sq + L::kPackedBytes + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kPackedBytes + L::kXBytes);
          if (GROUPED) tma_load_3d(sq, &tmQ, &full_bar[stage], kb * L::kPackedRow, tw * kWqBM, e);
          else tma_load_2d(sq, &tmQ, &full_bar[stage], kb * L::kPackedRow, tw * kWqBM);
          tma_load_2d(sx, &tmX, &full_bar[stage], kb * kWqBK, tt * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(1, fmt, fmt, kWqBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
          report_status(status, kWaitTimeout, 121, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase) || !mbar_wait(&ready_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 122, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes + L::kPackedBytes);
          const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kWqBK / 16; ++k)
            umma_f16_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ dequantise (128 threads, one weight row each)
    const int r = threadIdx.x - 64;
    const T* S = reinterpret_cast<const T*>(p.scales);
    const T* Z = reinterpret_cast<const T*>(p.zeros);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int tt = tile % num_t, tw = tile / num_t;
      const int e = expert_of(tt);
      const int n = min(tw * kWqBM + r, p.N - 1);
      const T* Se = S + (size_t)e * ngroups * p.N + n;
      const T* Ze = Z ? Z + (size_t)e * ngroups * p.N + n : nullptr;
      // scales / zero points of a k-step are fetched one step ahead, so their global-memory latency overlaps the
      // wait for the stage and the conversion of the previous step instead of sitting in front of the arithmetic
      T sc_cur[2], zc_cur[2], sc_nxt[2], zc_nxt[2];
      auto fetch = [&](int kb, T (&sc)[2], T (&zc)[2]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int g = min((kb * kWqBK + h * 32) / p.group, ngroups - 1);
          sc[h] = Se[(size_t)g * p.N];
          zc[h] = Ze ? Ze[(size_t)g * p.N] : from_f<T>(BITS == 4 ? (std::is_same<T, __half>::value ? 1032.f : 136.f) : 128.f);
        }
      };
      if (kb0 < kb1) fetch(kb0, sc_cur, zc_cur);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (kb + 1 < kb1) fetch(kb + 1, sc_nxt, zc_nxt);
        if (!mbar_wait(&full_bar[stage], phase)) {
          report_status(status, kWaitTimeout, 123, tile, kb);
          ok = false;
          break;
        }
        uint8_t* sq = smem + stage * L::kStageBytes;
        uint8_t* sa = sq + L::kPackedBytes + r * 128;
        const uint4* src = reinterpret_cast<const uint4*>(sq + r * L::kPackedRow);
#pragma unroll
        for (int h = 0; h < 2; ++h) {   // 32 k values per half
          const T sc = sc_cur[h];
          if constexpr (BITS == 4) {
            const T zc = zc_cur[h];
            T2 s2, z2;
            s2.x = sc; s2.y = sc; z2.x = zc; z2.y = zc;
            const uint4 q = src[h];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint32_t o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t bits = ((w[u] >> (4 * j)) & 0x000F000Fu) | Pair16<T>::magic;
                T2 v = __hmul2(__hsub2(*reinterpret_cast<T2*>(&bits), z2), s2);
                o[j] = *reinterpret_cast<uint32_t*>(&v);
              }
              const int chunk = h * 4 + u;
              *reinterpret_cast<uint4*>(sa + ((chunk ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          } else {
            const float sf = to_f(sc), zf = to_f(zc_cur[h]);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const uint4 q = src[h * 2 + u];   // 16 bytes = 16 k values = two 16-byte output chunks
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = ((float)((w[c * 2 + (i >> 2)] >> (8 * (i & 3))) & 0xFFu) - zf) * sf;
                const int chunk = h * 4 + u * 2 + c;
                *reinterpret_cast<uint4*>(sa + ((chunk ^ (r & 7)) << 4)) = pack8<T>(f);
              }
            }
          }
        }
        fence_proxy_async();          // generic-proxy stores -> visible to the tensor core's async proxy
        mbar_arrive(&ready_bar[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
#pragma unroll
        for (int h = 0; h < 2; ++h) { sc_cur[h] = sc_nxt[h]; zc_cur[h] = zc_nxt[h]; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 6..9)
    const int quarter = warp & 3;
    const T* bias = reinterpret_cast<const T*>(p.bias);
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int tt = tile % num_t, tw = tile / num_t;
      const int acc = it & 1;
      if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
        report_status(status, kWaitTimeout, 124, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const int n = tw * kWqBM + quarter * 32 + lane;
      const bool n_ok = n < p.N;
      const float bv = (bias && n_ok && blockIdx.y == 0) ? to_f(bias[n]) : 0.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < BN; c += CH) {
        uint32_t rg[32];
        if constexpr (CH == 32) {
          tmem_ld_32x32b_x32(taddr + c, rg);
        } else {
          uint32_t r16[16];
          tmem_ld_32x32b_x16(taddr + c, r16);
#pragma unroll
          for (int i = 0; i < 16; ++i) rg[i] = r16[i];
        }
        tmem_ld_wait();
        const int t0 = tt * BN + c;
        if (num_k == 0) {
#pragma unroll
          for (int i = 0; i < CH; ++i) rg[i] = 0u;
        }
        if (p.splits > 1) {
          float* dst = p.partial + (size_t)blockIdx.y * p.M * p.N;
#pragma unroll
          for (int i = 0; i < CH; ++i)
            if (n_ok && t0 + i < rows) dst[(size_t)(t0 + i) * p.N + n] = __uint_as_float(rg[i]) + bv;
        } else if (p.epi == 1) {
#pragma unroll
          for (int i = 0; i < CH; ++i) {
            const float g = to_f(from_f<T>(__uint_as_float(rg[i]) + bv));
            const float u = __shfl_down_sync(0xffffffffu, g, 1);
            if ((lane & 1) == 0 && n_ok && t0 + i < rows)
              C[(size_t)(t0 + i) * p.ldc + (n >> 1)] = from_f<T>(g / (1.f + __expf(-g)) * u);
          }
        } else {
#pragma unroll
          for (int i = 0; i < CH; ++i)
            if (n_ok && t0 + i < rows) C[(size_t)(t0 + i) * p.ldc + n] = from_f<T>(__uint_as_float(rg[i]) + bv);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[acc]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T>
__global__ void splitk_reduce_kernel(T* __restrict__ C, const float* __restrict__ partial, int M, int N, int ldc,
                                     int splits) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)M * N) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += partial[(size_t)k * M * N + i];
  C[(i / N) * ldc + (i % N)] = from_f<T>(s);
}

static int wq_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

template <typename T, int BN, int STAGES, int BITS, bool GROUPED>
static void launch_wq(const void* A, int lda, const void* Q, int E, void* C, WqArgs p, cudaStream_t stream,
                      StatusWord* status) {
  using L = WqLayout<BN, STAGES, BITS>;
  static_assert(L::kDyn <= 232448, "shared memory budget exceeded");
  const uint64_t row_bytes = (uint64_t)p.K * BITS / 8;
  CUtensorMap tmQ;
  if (GROUPED) {
    uint64_t d[3] = {row_bytes, (uint64_t)p.N, (uint64_t)E};
    uint64_t s[2] = {row_bytes, row_bytes * p.N};
    uint32_t b[3] = {(uint32_t)L::kPackedRow, (uint32_t)kWqBM, 1};
    tmQ = make_tmap_nd(Q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d, s, b, CU_TENSOR_MAP_SWIZZLE_NONE);
  } else {
    tmQ = make_tmap_2d(Q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.N, row_bytes, row_bytes, kWqBM, L::kPackedRow, false);
  }
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmX = make_tmap_2d(A, dt, 2, p.M, p.K, lda, BN, kWqBK);
  auto kern = gemm_wna16_kernel<T, BN, STAGES, BITS, GROUPED>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
  const int tiles = ceil_div(p.N, kWqBM) * ceil_div(p.M, BN);
  int gx = wq_sms() / p.splits;
  gx = gx < 1 ? 1 : gx;
  gx = tiles < gx ? tiles : gx;
  kern<<<dim3(gx, p.splits), 320, L::kDyn, stream>>>(tmQ, tmX, reinterpret_cast<T*>(C), p, status);
  if (p.splits > 1) {
    const int64_t n = (int64_t)p.M * p.N;
    splitk_reduce_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(reinterpret_cast<T*>(C), p.partial, p.M,
                                                                             p.N, p.ldc, p.splits);
  }
}

template <typename T, int BITS, bool GROUPED>
static void dispatch_wq(const void* A, int lda, const void* Q, int E, void* C, const WqArgs& p, int bn,
                        cudaStream_t stream, StatusWord* status) {
  if (bn <= 16) launch_wq<T, 16, 8, BITS, GROUPED>(A, lda, Q, E, C, p, stream, status);
  else if (bn <= 32) launch_wq<T, 32, 8, BITS, GROUPED>(A, lda, Q, E, C, p, stream, status);
  else if (bn <= 64) launch_wq<T, 64, 6, BITS, GROUPED>(A, lda, Q, E, C, p, stream, status);
  else if (bn <= 128) launch_wq<T, 128, 5, BITS, GROUPED>(A, lda, Q, E, C, p, stream, status);
  else launch_wq<T, 256, 4, BITS, GROUPED>(A, lda, Q, E, C, p, stream, status);
}

// Token tile the launcher will use for M rows (the grouped path needs moe_align's block size to equal it).
int gemm_wna16_token_tile(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256))); }

// Split count the launcher will use (callers size the fp32 workspace [splits, M, N] from it).
int gemm_wna16_splits(int M, int N, int K, int bn) {
  const int tiles = ceil_div(N, kWqBM) * ceil_div(M, bn);
  const int num_k = ceil_div(K, kWqBK);
  // as many K ranges as fill one wave of SMs (any count, not only powers of two), each at least 8 k-steps long
  int s = wq_sms() / (tiles > 0 ? tiles : 1);
  s = s < 1 ? 1 : (s > 8 ? 8 : s);
  while (s > 1 && num_k / s < 8) --s;
  return s;
}

// A [M,K] 16-bit (row pitch lda elements); Q / scales / zeros as described at the top of the file.
// bits 4 or 8; dtype 0 bf16, 1 fp16; token_tile 0 = choose; partial = fp32 workspace or null (no split-K).
void gemm_wna16(const void* A, int M, int lda, const void* Q, const void* scales, const void* zeros, int E, int N,
                int K, int group, int bits, void* C, int ldc, const void* bias, float* partial, int splits,
                const int* block_expert, const int* total_padded, int grouped, int token_tile, int epi, int dtype,
                cudaStream_t stream, void* status) {
  if (M <= 0 || N <= 0) return;
  const int bn = token_tile > 0 ? token_tile : gemm_wna16_token_tile(M);
  if (partial == nullptr || grouped || epi != 0) splits = 1;
  WqArgs p{scales, zeros, bias, partial, block_expert, total_padded, M, N, K, ldc, group, E, epi, splits < 1 ? 1 : splits};
  StatusWord* st = reinterpret_cast<StatusWord*>(status);
#define WQ_GO(T, B, G) dispatch_wq<T, B, G>(A, lda, Q, E, C, p, bn, stream, st)
  if (dtype == 0) {
    if (bits == 4) { if (grouped) WQ_GO(__nv_bfloat16, 4, true); else WQ_GO(__nv_bfloat16, 4, false); }
    else           { if (grouped) WQ_GO(__nv_bfloat16, 8, true); else WQ_GO(__nv_bfloat16, 8, false); }
  } else {
    if (bits == 4) { if (grouped) WQ_GO(__half, 4, true); else WQ_GO(__half, 4, false); }
    else           { if (grouped) WQ_GO(__half, 8, true); else WQ_GO(__half, 8, false); }
  }
#undef WQ_GO
}

}  // namespace b200
