// Grouped (per-expert) GEMM for mixture-of-experts layers on tcgen05:
//
//     C[rows of block b, :] = A_perm[rows of block b, :] . W[expert(b)]^T     for every 128-row block b
//
// A_perm is the expert-sorted, 128-row-padded activation matrix produced by moe_align +
// moe_gather; `block_expert[b]` names the expert of row block b (-1 = unused) and
// `*total_padded` (device memory) the number of valid rows, so the launch is independent of
// the routing outcome (CUDA-graph friendly).  W is [E, N, K]; its TMA map is 3-D and the expert
// index is a coordinate.  Same pipeline as the dense single-CTA kernel (TMA ring ->
// tcgen05.mma -> double-buffered TMEM -> epilogue warps); epilogue 1 applies SiLU-gate over
// row-interleaved (gate, up) weights so GEMM1 of the expert MLP writes act(gate) * up directly.
// Replaces the Triton fused_moe_kernel / vendor grouped GEMM of the reference
// (vllm_metax/model_executor/layers/fused_moe/fused_moe.py:347-650, 905-1004).
#include <type_traits>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kGgBM = 128, kGgBK = 64;

template <int BN, int STAGES>
struct GgSmem {
  static constexpr int kABytes = kGgBM * kGgBK * 2;
  static constexpr int kBBytes = BN * kGgBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kDyn = kBarOffset + (2 * STAGES + 4) * 8 + 16 + 1024;
};

template <typename T, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                    T* __restrict__ C, const int* __restrict__ block_expert, const int* __restrict__ total_padded,
                    int N, int K, int ldc, int epi, int num_experts, StatusWord* status) {
  using L = GgSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = *total_padded;
  const int num_mb = rows / kGgBM;
  const int num_n = ceil_div(N, BN);
  const int num_tiles = num_mb * num_n;
  const int num_k = ceil_div(K, kGgBK);
  constexpr uint32_t kTmemCols = 2 * BN;

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

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mb = tile / num_n, tn = tile % num_n;
        int e = block_expert[mb];
        if (e < 0 || e >= num_experts) {
          if (e >= num_experts) report_status(status, kBadIndex, 80, num_experts, e);
          e = 0;  // rows of an unused block are zero; any expert's weights give zero
        }
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 81, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * kGgBK, mb * kGgBM);
          tma_load_3d(sa + L::kABytes, &tmW, &full_bar[stage], kb * kGgBK, tn * BN, e);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(1, fmt, fmt, kGgBM, BN);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
          report_status(status, kWaitTimeout, 82, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 83, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kGgBK / 16; ++k)
            umma_f16_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int mb = tile / num_n, tn = tile % num_n;
      const int acc = it & 1;
      if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
        report_status(status, kWaitTimeout, 84, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const int row = mb * kGgBM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        if (row < rows) store_row_segment<T, 32>(r, row, tn * BN + c, N, C, ldc, nullptr, nullptr, 0, epi);
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

template <typename T, int BN, int STAGES>
static void launch_grouped(const void* A, int max_rows, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                           const int* block_expert, const int* total_padded, int epi, cudaStream_t stream,
                           StatusWord* status) {
  using L = GgSmem<BN, STAGES>;
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA = make_tmap_2d(A, dt, 2, max_rows, K, lda, kGgBM, kGgBK);
  uint64_t wd[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)E};
  uint64_t ws[2] = {(uint64_t)K * 2, (uint64_t)N * K * 2};
  uint32_t wb[3] = {(uint32_t)kGgBK, (uint32_t)BN, 1};
  CUtensorMap tmW = make_tmap_nd(W, dt, 3, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
  auto kern = gemm_grouped_kernel<T, BN, STAGES>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int max_tiles = (max_rows / kGgBM) * ceil_div(N, BN);
  const int grid = max_tiles < sms ? (max_tiles < 1 ? 1 : max_tiles) : sms;
  kern<<<grid, 192, L::kDyn, stream>>>(tmA, tmW, reinterpret_cast<T*>(C), block_expert, total_padded, N, K, ldc, epi,
                                       E, status);
}

// A [max_rows, K] (max_rows multiple of 128), W [E, N, K], C [max_rows, N] (or N/2 with epi 1).
void gemm_grouped(const void* A, int max_rows, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                  const int* block_expert, const int* total_padded, int epi, int dtype, cudaStream_t stream,
                  void* status) {
  if (max_rows <= 0 || N <= 0) return;
  StatusWord* st = reinterpret_cast<StatusWord*>(status);
  const bool wide = N >= 1024;
  if (dtype == 0) {
    if (wide) launch_grouped<__nv_bfloat16, 256, 4>(A, max_rows, lda, W, E, N, K, C, ldc, block_expert, total_padded, epi, stream, st);
    else launch_grouped<__nv_bfloat16, 128, 6>(A, max_rows, lda, W, E, N, K, C, ldc, block_expert, total_padded, epi, stream, st);
  } else {
    if (wide) launch_grouped<__half, 256, 4>(A, max_rows, lda, W, E, N, K, C, ldc, block_expert, total_padded, epi, stream, st);
    else launch_grouped<__half, 128, 6>(A, max_rows, lda, W, E, N, K, C, ldc, block_expert, total_padded, epi, stream, st);
  }
}

}  // namespace b200
