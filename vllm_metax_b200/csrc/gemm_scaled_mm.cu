// W8A8 "scaled mm" on tcgen05, dense and grouped:
//
//   int8 :  C[m,n] = a_scale[m] * w_scale[n] * ( sum_k A8[m,k] W8[n,k]  -  azp[m] * azp_adj[n] ) + bias[n]
//   fp8  :  C[m,n] = a_scale[m] * w_scale[n] *   sum_k A8[m,k] W8[n,k]                          + bias[n]
//
// int8 uses tcgen05.mma kind::i8 (s8 x s8 -> s32 accumulators in TMEM, exact), fp8 uses
// kind::f8f6f4 (e4m3 -> f32).  a_scale is per token or per tensor, w_scale per output channel or per
// tensor; azp (per-token zero point) and azp_adj (column sums of W, already multiplied by the
// zero point when it is per tensor) implement asymmetric activations.
// Grouped mode: A is the expert-sorted 128-row-padded activation matrix, W [E,N,K], w_scale [E,N]
// (block_expert / total_padded as produced by moe_align_block_size).
// Same pipeline as the bf16 kernel: TMA producer warp, single-thread MMA issuer, four epilogue
// warps, STAGES-deep 128B-swizzled ring, two TMEM accumulator buffers, bounded waits.
// Replaces cutlass_scaled_mm / cutlass_scaled_mm_azp / cutlass_moe_mm_w8a8
// (vllm_metax/model_executor/layers/quantization/_python_api_ops.py:812-1105,
//  registry/linear_kernels/int8.py:33-79 of the reference).
#include <cstdlib>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kSmBM = 128, kSmBK = 128;   // 128 one-byte elements = one 128-byte swizzle row

template <int BN, int STAGES>
struct SmLayout {
  static constexpr int kABytes = kSmBM * kSmBK;
  static constexpr int kBBytes = BN * kSmBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kDyn = kBarOffset + (2 * STAGES + 4) * 8 + 16 + 1024;
};

struct ScaledMmArgs {
  const float* a_scale;     // [M] or [1]
  const float* w_scale;     // [(E,) N] or [1]
  const int* azp;           // [M] or null
  const int* azp_adj;       // [N] or null
  const void* bias;         // [N] of T or null
  const int* block_expert;  // grouped
  const int* total_padded;  // grouped
  int M, N, K, ldc, num_experts;
  int a_per_row, w_per_col;
};

template <typename T, int BN, int STAGES, bool INT8, bool GROUPED>
__global__ void __launch_bounds__(192, 1)
scaled_mm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                 T* __restrict__ C, const ScaledMmArgs p, StatusWord* status) {
  using L = SmLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = GROUPED ? *p.total_padded : p.M;
  const int num_mb = ceil_div(rows, kSmBM);
  const int num_n = ceil_div(p.N, BN);
  const int num_tiles = num_mb * num_n;
  const int num_k = ceil_div(p.K, kSmBK);
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto expert_of = [&](int mb) -> int {
    if (!GROUPED) return 0;
    int e = p.block_expert[mb];
    return (e < 0 || e >= p.num_experts) ? 0 : e;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mb = tile % num_mb, tn = tile / num_mb;   // neighbouring CTAs share the weight tile
        const int e = expert_of(mb);
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 110, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * kSmBK, mb * kSmBM);
          if (GROUPED) tma_load_3d(sa + L::kABytes, &tmW, &full_bar[stage], kb * kSmBK, tn * BN, e);
          else tma_load_2d(sa + L::kABytes, &tmW, &full_bar[stage], kb * kSmBK, tn * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // int8: c = s32 (2), a = b = signed 8-bit (1);  fp8: c = f32 (1), a = b = e4m3 (0)
      constexpr uint32_t idesc = INT8 ? make_idesc(2, 1, 1, kSmBM, BN) : make_idesc(1, 0, 0, kSmBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
          report_status(status, kWaitTimeout, 111, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 112, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kSmBK / 32; ++k) {
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (INT8) umma_i8_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            else umma_f8_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int it = 0;
    const T* bias = reinterpret_cast<const T*>(p.bias);
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int mb = tile % num_mb, tn = tile / num_mb;
      const int e = expert_of(mb);
      const int acc = it & 1;
      if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
        report_status(status, kWaitTimeout, 113, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const int row = mb * kSmBM + quarter * 32 + lane;
      const bool row_ok = row < rows;
      const float as = p.a_scale[(p.a_per_row && row_ok) ? row : 0];
      const int zp = (p.azp && row_ok) ? p.azp[row] : (p.azp_adj ? 1 : 0);
      const float* ws = p.w_scale + (p.w_per_col ? (size_t)e * p.N : (GROUPED ? (size_t)e : 0));
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        if (row_ok) {
          const int col0 = tn * BN + c;
          T* dst = C + (size_t)row * p.ldc + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int col = col0 + v * 8 + i;
              const bool cok = col < p.N;
              float a;
              if (INT8) {
                int x = (int)r[v * 8 + i];
                if (p.azp_adj && cok) x -= zp * p.azp_adj[col];
                a = (float)x;
              } else {
                a = __uint_as_float(r[v * 8 + i]);
              }
              const float w = p.w_per_col ? (cok ? ws[col] : 0.f) : ws[0];
              a *= as * w;
              if (bias && cok) a += to_f(bias[col]);
              f[i] = a;
            }
            const int col = col0 + v * 8;
            if (col + 8 <= p.N) {
              *reinterpret_cast<uint4*>(dst + v * 8) = pack8<T>(f);
            } else {
              for (int i = 0; i < 8; ++i)
                if (col + i < p.N) dst[v * 8 + i] = from_f<T>(f[i]);
            }
          }
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

// ---------------------------------------------------------------------------------------------- CTA pairs
// Large dense problems: two CTAs own one 256 x 256 tile (tcgen05 cta_group::2).  Per SM and k-block this halves
// the bytes pulled from L2 for the same tensor work; with one-byte operands the single-CTA tile needs 96 B/clk/SM,
// more than L2 delivers, so this is what lets the 8-bit kinds run ahead of the 16-bit rate.  Same
// synchronisation as the bf16 CTA-pair kernel: full[] on the leader, empty[] / tmem_full[] per CTA (committed to
// both), tmem_empty[] on the leader (256 epilogue threads); each CTA loads ITS halves with plain TMA loads.
constexpr int kSmPairStages = 6;
struct SmPairLayout {
  static constexpr int kABytes = 128 * kSmBK, kBBytes = 128 * kSmBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kSmPairStages * kStageBytes;
  static constexpr int kDyn = kBarOffset + (2 * kSmPairStages + 4) * 8 + 16 + 1024;
};

template <typename T, bool INT8>
__global__ void __launch_bounds__(192, 1)
scaled_mm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                      T* __restrict__ C, const ScaledMmArgs p, StatusWord* status) {
  using L = SmPairLayout;
  constexpr int BN = 256, BM = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kSmPairStages;
  uint64_t* tmem_full = empty_bar + kSmPairStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_m = ceil_div(p.M, BM), num_n = ceil_div(p.N, BN);
  const int num_tiles = num_m * num_n;
  const int num_k = ceil_div(p.K, kSmBK);
  constexpr uint32_t kTmemCols = 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSmPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 256);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmW);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int tm = tile % num_m, tn = tile / num_m;
        const int row_a = tm * BM + (int)rank * 128, row_b = tn * BN + (int)rank * 128;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 114, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          tma_load_2d_pair(sa, &tmA, &full_bar[stage], kb * kSmBK, row_a);
          tma_load_2d_pair(sa + L::kABytes, &tmW, &full_bar[stage], kb * kSmBK, row_b);
          if (++stage == kSmPairStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = INT8 ? make_idesc(2, 1, 1, BM, BN) : make_idesc(1, 0, 0, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
          report_status(status, kWaitTimeout, 115, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 116, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kSmBK / 32; ++k) {
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (INT8) umma_i8_ss_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            else umma_f8_ss_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          }
          umma_commit_pair(&empty_bar[stage], 0x3);
          if (++stage == kSmPairStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 0x3);
      }
    }
  } else {
    const int quarter = warp & 3;
    const uint32_t leader_empty0 = mapa(smem_u32(&tmem_empty[0]), 0);
    const uint32_t leader_empty1 = mapa(smem_u32(&tmem_empty[1]), 0);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    int it = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters, ++it) {
      const int tm = tile % num_m, tn = tile / num_m;
      const int acc = it & 1;
      if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
        report_status(status, kWaitTimeout, 117, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * BM + (int)rank * 128 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const float as = p.a_scale[(p.a_per_row && row_ok) ? row : 0];
      const int zp = (p.azp && row_ok) ? p.azp[row] : (p.azp_adj ? 1 : 0);
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        if (row_ok) {
          const int col0 = tn * BN + c;
          T* dst = C + (size_t)row * p.ldc + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int col = col0 + v * 8 + i;
              const bool cok = col < p.N;
              float a;
              if (INT8) {
                int x = (int)r[v * 8 + i];
                if (p.azp_adj && cok) x -= zp * p.azp_adj[col];
                a = (float)x;
              } else {
                a = __uint_as_float(r[v * 8 + i]);
              }
              const float w = p.w_per_col ? (cok ? p.w_scale[col] : 0.f) : p.w_scale[0];
              a *= as * w;
              if (bias && cok) a += to_f(bias[col]);
              f[i] = a;
            }
            const int col = col0 + v * 8;
            if (col + 8 <= p.N) {
              *reinterpret_cast<uint4*>(dst + v * 8) = pack8<T>(f);
            } else {
              for (int i = 0; i < 8; ++i)
                if (col + i < p.N) dst[v * 8 + i] = from_f<T>(f[i]);
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

static int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

template <typename T, int BN, int STAGES, bool INT8, bool GROUPED>
static void launch_sm(const void* A, int lda, const void* W, int E, void* C, const ScaledMmArgs& p,
                      cudaStream_t stream, StatusWord* status) {
  using L = SmLayout<BN, STAGES>;
  static_assert(L::kDyn <= 232448, "shared memory budget exceeded");
  CUtensorMap tmA = make_tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.M, p.K, lda, kSmBM, kSmBK);
  CUtensorMap tmW;
  if (GROUPED) {
    uint64_t wd[3] = {(uint64_t)p.K, (uint64_t)p.N, (uint64_t)E};
    uint64_t ws[2] = {(uint64_t)p.K, (uint64_t)p.N * p.K};
    uint32_t wb[3] = {(uint32_t)kSmBK, (uint32_t)BN, 1};
    tmW = make_tmap_nd(W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    tmW = make_tmap_2d(W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.N, p.K, p.K, BN, kSmBK);
  }
  auto kern = scaled_mm_kernel<T, BN, STAGES, INT8, GROUPED>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
  const int tiles = ceil_div(p.M, kSmBM) * ceil_div(p.N, BN);
  const int grid = tiles < sm_count() ? (tiles < 1 ? 1 : tiles) : sm_count();
  kern<<<grid, 192, L::kDyn, stream>>>(tmA, tmW, reinterpret_cast<T*>(C), p, status);
}

template <typename T, bool INT8, bool GROUPED>
static void dispatch_bn(const void* A, int lda, const void* W, int E, void* C, const ScaledMmArgs& p,
                        cudaStream_t stream, StatusWord* status) {
  const int mt = ceil_div(p.M, kSmBM);
  int bn = 256;
  while (bn > 64 && mt * ceil_div(p.N, bn) < sm_count()) bn >>= 1;
  if (bn == 256) launch_sm<T, 256, 4, INT8, GROUPED>(A, lda, W, E, C, p, stream, status);
  else if (bn == 128) launch_sm<T, 128, 6, INT8, GROUPED>(A, lda, W, E, C, p, stream, status);
  else launch_sm<T, 64, 8, INT8, GROUPED>(A, lda, W, E, C, p, stream, status);
}

template <typename T, bool INT8>
static void launch_sm_pair(const void* A, int lda, const void* W, void* C, const ScaledMmArgs& p, cudaStream_t stream,
                           StatusWord* status) {
  using L = SmPairLayout;
  static_assert(L::kDyn <= 232448, "shared memory budget exceeded");
  CUtensorMap tmA = make_tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.M, p.K, lda, 128, kSmBK);
  CUtensorMap tmW = make_tmap_2d(W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.N, p.K, p.K, 128, kSmBK);
  auto kern = scaled_mm_pair_kernel<T, INT8>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
  const int tiles = ceil_div(p.M, 256) * ceil_div(p.N, 256);
  int clusters = sm_count() / 2;
  if (tiles < clusters) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = L::kDyn;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, tmA, tmW, reinterpret_cast<T*>(C), p, status);
}

// A [M,K] one-byte elements (row pitch lda bytes, K % 16 == 0); W [N,K] or [E,N,K] contiguous.
// kind: 0 int8, 1 fp8 e4m3.  out_dtype: 0 bf16, 1 fp16.
void gemm_scaled_mm(const void* A, int M, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                    const float* a_scale, int a_per_row, const float* w_scale, int w_per_col, const int* azp,
                    const int* azp_adj, const void* bias, const int* block_expert, const int* total_padded,
                    int grouped, int kind, int out_dtype, cudaStream_t stream, void* status) {
  if (M <= 0 || N <= 0) return;
  ScaledMmArgs p{a_scale, w_scale, azp, azp_adj, bias, block_expert, total_padded, M, N, K, ldc, E, a_per_row, w_per_col};
  StatusWord* st = reinterpret_cast<StatusWord*>(status);
  // dense and at least one 256 x 256 tile per pair of SMs: the CTA-pair kernel (B200_GEMM_PAIR=0 switches it off)
  static const bool pair_default = [] {
    const char* e = std::getenv("B200_GEMM_PAIR");
    return e == nullptr || std::atoi(e) != 0;
  }();
  if (!grouped && pair_default && M >= 512 && (int64_t)ceil_div(M, 256) * ceil_div(N, 256) >= 64) {
    if (out_dtype == 0) {
      if (kind == 0) launch_sm_pair<__nv_bfloat16, true>(A, lda, W, C, p, stream, st);
      else launch_sm_pair<__nv_bfloat16, false>(A, lda, W, C, p, stream, st);
    } else {
      if (kind == 0) launch_sm_pair<__half, true>(A, lda, W, C, p, stream, st);
      else launch_sm_pair<__half, false>(A, lda, W, C, p, stream, st);
    }
    return;
  }
#define SM_GO(T, I8, G) dispatch_bn<T, I8, G>(A, lda, W, E, C, p, stream, st)
  if (out_dtype == 0) {
    if (kind == 0) { if (grouped) SM_GO(__nv_bfloat16, true, true); else SM_GO(__nv_bfloat16, true, false); }
    else           { if (grouped) SM_GO(__nv_bfloat16, false, true); else SM_GO(__nv_bfloat16, false, false); }
  } else {
    if (kind == 0) { if (grouped) SM_GO(__half, true, true); else SM_GO(__half, true, false); }
    else           { if (grouped) SM_GO(__half, false, true); else SM_GO(__half, false, false); }
  }
#undef SM_GO
}

}  // namespace b200
