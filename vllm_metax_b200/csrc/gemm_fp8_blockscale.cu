// Block-scaled fp8 (e4m3) GEMM, dense and grouped, on tcgen05 (kind::f8f6f4):
//
//     C[m, n] = sum_kb  a_scale[m, kb] * w_scale[n / 128, kb] * ( A8[m, kb-block] . W8[n, kb-block] )
//
// i.e. DeepSeek-style checkpoints: weights e4m3 with one f32 scale per 128 x 128 block
// (`weight_scale_inv`), activations quantised on the fly 1 x 128 per token.  Because the scales
// change every 128 elements of K, each 128-wide K block is multiplied into a FRESH TMEM buffer
// (4 MMAs of K = 32) and the epilogue warps fold it into fp32 register accumulators with the
// block's scale while the tensor core works on the next block (two TMEM partial buffers).
// Tile 128 x 128, TMA ring of 128-byte-swizzled [rows x 128 B] tiles, same barrier scheme as
// the bf16 kernel plus part_full / part_empty for the partial buffers.
// Grouped mode: A is the expert-sorted padded activation matrix, W [E, N, K], w_scale
// [E, N/128, K/128]; block_expert / total_padded as in gemm_grouped_tcgen05.cu.
// Replaces cutlass_fp8_block_scaled_mm / deep_gemm fp8 grouped GEMMs
// (vllm_metax/model_executor/layers/quantization/_cutlass_ops.py:23-38,
// experts/batched_deep_gemm_moe.py:299-326).
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kF8BM = 128, kF8BN = 128, kF8BK = 128, kF8Stages = 6;

struct F8Smem {
  static constexpr int kABytes = kF8BM * kF8BK;
  static constexpr int kBBytes = kF8BN * kF8BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kF8Stages * kStageBytes;
  static constexpr int kDyn = kBarOffset + (2 * kF8Stages + 4) * 8 + 16 + 1024;
};

template <typename T, bool GROUPED>
__global__ void __launch_bounds__(192, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                T* __restrict__ C, const float* __restrict__ a_scale, const float* __restrict__ w_scale,
                const int* __restrict__ block_expert, const int* __restrict__ total_padded, int M, int N, int K,
                int ldc, int num_experts, StatusWord* status) {
  using L = F8Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kF8Stages;
  uint64_t* part_full = empty_bar + kF8Stages;
  uint64_t* part_empty = part_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = GROUPED ? *total_padded : M;
  const int num_mb = ceil_div(rows, kF8BM);
  const int num_n = ceil_div(N, kF8BN);
  const int num_tiles = num_mb * num_n;
  const int num_k = ceil_div(K, kF8BK);
  const int sk = num_k;                       // scale row length
  const int sn = ceil_div(N, 128);
  constexpr uint32_t kTmemCols = 2 * kF8BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&part_full[i], 1);
      mbar_init(&part_empty[i], 128);
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
    int e = block_expert[mb];
    if (e < 0 || e >= num_experts) e = 0;
    return e;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mb = tile / num_n, tn = tile % num_n;
        const int e = expert_of(mb);
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 90, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * kF8BK, mb * kF8BM);
          if (GROUPED) tma_load_3d(sa + L::kABytes, &tmW, &full_bar[stage], kb * kF8BK, tn * kF8BN, e);
          else tma_load_2d(sa + L::kABytes, &tmW, &full_bar[stage], kb * kF8BK, tn * kF8BN);
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // c = f32, a = b = e4m3 (format code 0)
      constexpr uint32_t idesc = make_idesc(1, 0, 0, kF8BM, kF8BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;   // running K-block count across tiles selects the partial buffer
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int pb = it & 1;
          if (!mbar_wait(&part_empty[pb], ((it >> 1) & 1) ^ 1) || !mbar_wait(&full_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 91, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kF8BK / 32; ++k)
            umma_f8_ss(tmem_base + pb * kF8BN, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          umma_commit(&part_full[pb]);
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int mb = tile / num_n, tn = tile % num_n;
      const int e = expert_of(mb);
      const int row = mb * kF8BM + quarter * 32 + lane;
      const bool row_ok = row < rows;
      const float* as = a_scale + (size_t)(row_ok ? row : 0) * sk;
      const float* ws = w_scale + ((size_t)e * sn + tn) * sk;
      float acc[kF8BN];
#pragma unroll
      for (int i = 0; i < kF8BN; ++i) acc[i] = 0.f;
      bool ok = true;
      for (int kb = 0; kb < num_k; ++kb, ++it) {
        const int pb = it & 1;
        const float sc = as[kb] * ws[kb];
        if (!mbar_wait(&part_full[pb], (it >> 1) & 1)) {
          report_status(status, kWaitTimeout, 92, tile, kb);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + pb * kF8BN;
#pragma unroll
        for (int c = 0; c < kF8BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c + i] = fmaf(__uint_as_float(r[i]), sc, acc[c + i]);
        }
        tc_fence_before_sync();
        mbar_arrive(&part_empty[pb]);
      }
      if (!ok) break;
      if (row_ok) {
        T* dst = C + (size_t)row * ldc + tn * kF8BN;
#pragma unroll
        for (int v = 0; v < kF8BN / 8; ++v) {
          const int col = tn * kF8BN + v * 8;
          if (col + 8 <= N) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = acc[v * 8 + i];
            *reinterpret_cast<uint4*>(dst + v * 8) = pack8<T>(f);
          } else {
            for (int i = 0; i < 8; ++i)
              if (col + i < N) dst[v * 8 + i] = from_f<T>(acc[v * 8 + i]);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, bool GROUPED>
static void launch_f8(const void* A, int M, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                      const float* a_scale, const float* w_scale, const int* block_expert, const int* total_padded,
                      cudaStream_t stream, StatusWord* status) {
  CUtensorMap tmA = make_tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, kF8BM, kF8BK);
  CUtensorMap tmW;
  if (GROUPED) {
    uint64_t wd[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)E};
    uint64_t ws[2] = {(uint64_t)K, (uint64_t)N * K};
    uint32_t wb[3] = {(uint32_t)kF8BK, (uint32_t)kF8BN, 1};
    tmW = make_tmap_nd(W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    tmW = make_tmap_2d(W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, kF8BN, kF8BK);
  }
  auto kern = gemm_fp8_kernel<T, GROUPED>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Smem::kDyn);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ceil_div(M, kF8BM) * ceil_div(N, kF8BN);
  const int grid = tiles < sms ? (tiles < 1 ? 1 : tiles) : sms;
  kern<<<grid, 192, F8Smem::kDyn, stream>>>(tmA, tmW, reinterpret_cast<T*>(C), a_scale, w_scale, block_expert,
                                            total_padded, M, N, K, ldc, E, status);
}

// A [M, K] e4m3 (row pitch lda bytes), a_scale [M, K/128]; W [N, K] or [E, N, K] e4m3 contiguous,
// w_scale [(E,) ceil(N/128), K/128].  K must be a multiple of 128.  out_dtype: 0 bf16, 1 fp16.
void gemm_fp8_blockscale(const void* A, int M, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                         const float* a_scale, const float* w_scale, const int* block_expert,
                         const int* total_padded, int grouped, int out_dtype, cudaStream_t stream, void* status) {
  if (M <= 0 || N <= 0) return;
  StatusWord* st = reinterpret_cast<StatusWord*>(status);
  if (out_dtype == 0) {
    if (grouped) launch_f8<__nv_bfloat16, true>(A, M, lda, W, E, N, K, C, ldc, a_scale, w_scale, block_expert, total_padded, stream, st);
    else launch_f8<__nv_bfloat16, false>(A, M, lda, W, E, N, K, C, ldc, a_scale, w_scale, block_expert, total_padded, stream, st);
  } else {
    if (grouped) launch_f8<__half, true>(A, M, lda, W, E, N, K, C, ldc, a_scale, w_scale, block_expert, total_padded, stream, st);
    else launch_f8<__half, false>(A, M, lda, W, E, N, K, C, ldc, a_scale, w_scale, block_expert, total_padded, stream, st);
  }
}

}  // namespace b200
