// Split-K dense GEMM for medium M (decode batches, narrow tensor-parallel shards) on thread-block clusters:
//
//     C[M,N] = A[M,K] . W[N,K]^T (+ bias) (+ residual) | SiLU-gate epilogue
//
// When M x N gives fewer 128 x 128 tiles than the GPU has SMs, the kernel is a weight stream and its speed is
// set by how many SMs pull on it.  Here S CTAs of one CLUSTER share an output tile and each multiplies 1/S of
// the K range (TMA ring -> tcgen05.mma -> fp32 accumulators in its own TMEM).  The partial tiles are then
// reduced on chip: ranks 1..S-1 read their accumulators from TMEM and store them into the leader's shared
// memory over DSMEM (st.shared::cluster, a [column-quad][row] layout so that both the remote stores and the
// leader's reads are bank-conflict free); the leader adds its own accumulators and runs the epilogue.  No
// atomics, no fp32 round trip through global memory, no second launch.
// The leader's staging area is its own TMA ring, so remote stores start only after a cluster barrier that
// follows every CTA's last MMA; a second cluster barrier publishes the partials.  All mbarrier waits are
// bounded.
#include <type_traits>
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kSkBM = 128, kSkBN = 128, kSkBK = 64, kSkStages = 6;

struct SkSmem {
  static constexpr int kABytes = kSkBM * kSkBK * 2;
  static constexpr int kBBytes = kSkBN * kSkBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;           // 32 KB
  static constexpr int kRing = kSkStages * kStageBytes;           // 192 KB = 3 partial tiles of 64 KB
  static constexpr int kDyn = kRing + (2 * kSkStages + 2) * 8 + 16 + 1024;
};

__device__ __forceinline__ float4 ld_shared_v4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

template <typename T>
__global__ void __launch_bounds__(192, 1)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   T* __restrict__ C, const T* __restrict__ bias, const T* __restrict__ residual, int M, int N, int K,
                   int ldc, int ldr, int epi, int splits, StatusWord* status) {
  using L = SkSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kRing);
  uint64_t* empty_bar = full_bar + kSkStages;
  uint64_t* tmem_full = empty_bar + kSkStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int tile = blockIdx.x / splits;
  const int num_m = ceil_div(M, kSkBM);
  const int tm = tile % num_m, tn = tile / num_m;
  const int num_k_all = ceil_div(K, kSkBK);
  const int per = ceil_div(num_k_all, splits);
  const int kb0 = (int)rank * per, kb1 = min(num_k_all, kb0 + per);
  const int num_k = max(0, kb1 - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSkStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kSkBN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool have_acc = num_k > 0;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
          report_status(status, kWaitTimeout, 160, tile, kb);
          break;
        }
        uint8_t* sa = smem + stage * L::kStageBytes;
        mbar_expect_tx(&full_bar[stage], L::kStageBytes);
        tma_load_2d(sa, &tmA, &full_bar[stage], kb * kSkBK, tm * kSkBM);
        tma_load_2d(sa + L::kABytes, &tmB, &full_bar[stage], kb * kSkBK, tn * kSkBN);
        if (++stage == kSkStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(1, fmt, fmt, kSkBM, kSkBN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < num_k; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase)) {
          report_status(status, kWaitTimeout, 161, tile, kb);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
        const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
        for (int k = 0; k < kSkBK / 16; ++k)
          umma_f16_ss(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == kSkStages) { stage = 0; phase ^= 1; }
      }
      if (ok && num_k > 0) umma_commit(&tmem_full[0]);
      if (!ok || num_k == 0) mbar_arrive(&tmem_full[0]);      // release the epilogue; it treats the tile as zero
    }
  } else {
    // epilogue warps wait for this CTA's accumulators before the cluster may touch any ring
    if (!mbar_wait(&tmem_full[0], 0)) {
      report_status(status, kWaitTimeout, 162, tile, (int)rank);
      have_acc = false;
    }
    tc_fence_after_sync();
  }

  // ---- barrier 1: every CTA of the cluster has finished its MMAs (its ring is free)
  __syncthreads();
  if (splits > 1) cluster_sync();

  const int quarter = warp & 3;
  const int row_in_tile = quarter * 32 + lane;
  const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
  if (splits > 1 && rank != 0 && warp >= 2) {
    // push the partial tile into slot (rank - 1) of the leader's ring: element (row, 4-column group q) at
    // ((q * 128 + row) * 16) bytes
    const uint32_t slot = mapa(smem_u32(smem), 0) + (rank - 1) * (kSkBM * kSkBN * 4);
#pragma unroll 1
    for (int c = 0; c < kSkBN; c += 32) {
      uint32_t r[32];
      if (have_acc) {
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q)
        st_cluster_v4(slot + (uint32_t)((((c >> 2) + q) * kSkBM + row_in_tile) * 16), __uint_as_float(r[4 * q]),
                      __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
    }
  }
  // ---- barrier 2: partial tiles are in the leader's shared memory
  if (splits > 1) cluster_sync();

  if (rank == 0 && warp >= 2) {
    const int row = tm * kSkBM + row_in_tile;
    const uint32_t base = smem_u32(smem);
#pragma unroll 1
    for (int c = 0; c < kSkBN; c += 32) {
      uint32_t r[32];
      if (have_acc) {
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      for (int s = 1; s < splits; ++s) {
        const uint32_t slot = base + (uint32_t)(s - 1) * (kSkBM * kSkBN * 4);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 v = ld_shared_v4(slot + (uint32_t)((((c >> 2) + q) * kSkBM + row_in_tile) * 16));
          r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + v.x);
          r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + v.y);
          r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + v.z);
          r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + v.w);
        }
      }
      if (row < M) store_row_segment<T, 32>(r, row, tn * kSkBN + c, N, C, ldc, bias, residual, ldr, epi);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kSkBN);
  }
}

template <typename T>
static void launch_sk(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
                      int lda, int ldw, int ldc, int ldr, int epi, int splits, cudaStream_t stream, StatusWord* status) {
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA = make_tmap_2d(A, dt, 2, M, K, lda, kSkBM, kSkBK);
  CUtensorMap tmB = make_tmap_2d(W, dt, 2, N, K, ldw, kSkBN, kSkBK);
  auto kern = gemm_splitk_kernel<T>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SkSmem::kDyn);
  const int tiles = ceil_div(M, kSkBM) * ceil_div(N, kSkBN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * splits, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SkSmem::kDyn;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, tmA, tmB, reinterpret_cast<T*>(C), reinterpret_cast<const T*>(bias),
                     reinterpret_cast<const T*>(residual), M, N, K, ldc, ldr, epi, splits, status);
}

// Splits (1, 2 or 4) that bring the grid to about one CTA per SM without making the K ranges too short.
int gemm_splitk_choice(int M, int N, int K, int sms) {
  const int tiles = ceil_div(M, kSkBM) * ceil_div(N, kSkBN);
  if (tiles * 2 > sms + sms / 4) return 1;
  int s = 1;
  while (s < 4 && tiles * s * 2 <= sms + sms / 4 && K / (s * 2) >= 1024) s *= 2;
  return s;
}

void gemm_tn_splitk(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
                    int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int epi,
                    int splits) {
  if (M <= 0 || N <= 0) return;
  StatusWord* st = reinterpret_cast<StatusWord*>(status);
  if (dtype == 0) launch_sk<__nv_bfloat16>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, ldr, epi, splits, stream, st);
  else launch_sk<__half>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, ldr, epi, splits, stream, st);
}

}  // namespace b200
