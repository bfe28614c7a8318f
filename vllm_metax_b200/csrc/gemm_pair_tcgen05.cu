// Large-M dense GEMM on CTA pairs (tcgen05 cta_group::2):
//
//     C[M,N] = A[M,K] . W[N,K]^T (+ bias) (+ residual) | SiLU-gate epilogue
//
// Two CTAs on neighbouring SMs (a 2-CTA cluster) own one 256 x 256 output tile.  Each CTA
// loads ITS 128 rows of A and ITS 128 rows of W per 64-wide K block into its own shared
// memory with plain TMA loads (each CTA fetches its own half - nothing is broadcast); one
// thread of the leader CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16), which
// reads both CTAs' shared memory and accumulates 128 x 256 fp32 into each CTA's TMEM.  Per SM
// this halves the W traffic from L2 of the single-CTA 128 x 256 kernel at the same MMA work
// and leaves room for a 6-stage ring.
//
// Synchronisation (all waits bounded):
//   full[s]        lives in the leader; both CTAs' TMA loads complete_tx on it (64 KB per stage)
//   empty[s]       one per CTA; the leader's tcgen05.commit arrives on both
//   tmem_full[a]   one per CTA; commit arrives on both when a tile's accumulators are done
//   tmem_empty[a]  lives in the leader; 256 epilogue threads (both CTAs) arrive on it
// Clusters are persistent (74 on a 148-SM part) and walk tiles M-fastest so that
// concurrently running pairs share W tiles in L2.
#include <cstdlib>
#include <type_traits>
#include "comm_fused.cuh"
#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kPairBM = 256;          // tile rows (128 per CTA)
constexpr int kPairBN = 256;          // tile cols (128 W rows loaded per CTA)
constexpr int kPairBK = 64;

constexpr int kPairRowPitch = kPairBN * 2 + 16;   // staged output row: 512 B + 16 B so that 8 rows hit 32 banks

// STAGES-deep operand ring; BULK adds a row-major staging tile for the bulk-store epilogue.
template <int STAGES, bool BULK>
struct PairSmem {
  static constexpr int kABytes = 128 * kPairBK * 2;
  static constexpr int kBBytes = 128 * kPairBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;             // per CTA
  static constexpr int kOutStage = STAGES * kStageBytes;
  static constexpr int kBarOffset = kOutStage + (BULK ? 128 * kPairRowPitch : 0);
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16;
  static constexpr int kDyn = kTotal + 1024;
};

// 1-D bulk copy shared -> global (16-byte aligned, size a multiple of 16); completion tracked by bulk groups.
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}

// BULK epilogue (used with the row scatter): a thread converts its output row of the tile into shared memory and
// sends it as ONE bulk copy of up to 512 bytes, so rows that cross NVLink travel as large writes instead of
// 16-byte stores.
template <typename T, int STAGES, bool BULK>
__global__ void __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 T* __restrict__ C, const T* __restrict__ bias, const T* __restrict__ residual, int M, int N, int K,
                 int ldc, int ldr, int epi, StatusWord* status, const __grid_constant__ RowScatter sc) {
  using L = PairSmem<STAGES, BULK>;
  constexpr int kPairStages = STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kPairStages;
  uint64_t* tmem_full = empty_bar + kPairStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int num_m = ceil_div(M, kPairBM), num_n = ceil_div(N, kPairBN);
  const int num_tiles = num_m * num_n;
  const int num_k = ceil_div(K, kPairBK);
  constexpr uint32_t kTmemCols = 512;            // two 256-column accumulator buffers

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 256);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();                                // both CTAs' barriers exist before any remote arrive
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int tm = tile % num_m, tn = tile / num_m;
        const int row_a = tm * kPairBM + (int)rank * 128;
        const int row_b = tn * kPairBN + (int)rank * 128;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 60, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          tma_load_2d_pair(sa, &tmA, &full_bar[stage], kb * kPairBK, row_a);
          tma_load_2d_pair(sb, &tmB, &full_bar[stage], kb * kPairBK, row_b);
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(1, fmt, fmt, kPairBM, kPairBN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          report_status(status, kWaitTimeout, 61, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 62, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kPairBK / 16; ++k)
            umma_f16_ss_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage], 0x3);
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 0x3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    const uint32_t leader_empty0 = mapa(smem_u32(&tmem_empty[0]), 0);
    const uint32_t leader_empty1 = mapa(smem_u32(&tmem_empty[1]), 0);
    int it = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters, ++it) {
      const int tm = tile % num_m, tn = tile / num_m;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase)) {
        report_status(status, kWaitTimeout, 63, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * kPairBM + (int)rank * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kPairBN;
      if constexpr (BULK) {
        uint8_t* my_row = smem + L::kOutStage + (quarter * 32 + lane) * kPairRowPitch;
        tma_store_wait_read<0>();                  // this thread's previous row has left shared memory
#pragma unroll 1
        for (int c = 0; c < kPairBN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
            if (bias && tn * kPairBN + c + v * 8 + 8 <= N) {
              float b[8];
              unpack8<T>(*reinterpret_cast<const uint4*>(bias + tn * kPairBN + c + v * 8), b);
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] += b[i];
            }
            *reinterpret_cast<uint4*>(my_row + (c + v * 8) * 2) = pack8<T>(f);
          }
        }
        // accumulators are in shared memory: the tensor core may reuse the buffer while the row travels
        tc_fence_before_sync();
        mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
        const int col0 = tn * kPairBN;
        const int ncols = min(kPairBN, N - col0);
        if (row < M && ncols > 0) {
          T* drow;
          if (sc.tp > 0) {
            const int owner = row / sc.rows_per_rank;
            drow = reinterpret_cast<T*>(sc.recv[owner]) +
                   (size_t)(sc.src_rank * sc.rows_cap + (row - owner * sc.rows_per_rank)) * ldc;
          } else {
            drow = C + (size_t)row * ldc;
          }
          fence_proxy_async();                     // my generic-proxy writes are visible to the bulk copy
          bulk_store_1d(drow + col0, my_row, (uint32_t)ncols * 2);
        }
        tma_store_commit();
      } else {
#pragma unroll 1
      for (int c = 0; c < kPairBN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        if (row < M) {
          if (sc.tp > 0) {
            // the row goes to the receive slot of the rank that owns it (a peer store over NVLink for d != me)
            const int owner = row / sc.rows_per_rank;
            store_row_segment<T, 32>(r, sc.src_rank * sc.rows_cap + (row - owner * sc.rows_per_rank),
                                     tn * kPairBN + c, N, reinterpret_cast<T*>(sc.recv[owner]), ldc, bias, nullptr, 0,
                                     epi);
          } else {
            store_row_segment<T, 32>(r, row, tn * kPairBN + c, N, C, ldc, bias, residual, ldr, epi);
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
      }
    }
  }

  if constexpr (BULK) {
    if (warp >= 2) tma_store_wait<0>();          // every row of this thread has been written out
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();                                // no CTA leaves while its peer may still touch it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (sc.tp > 0 && threadIdx.x == 0) {
    // every store of this CTA is ordered before the fence by the barrier above; the last CTA of the launch
    // tells every owner that this source's rows have landed
    __threadfence_system();
    const uint32_t ticket = atomicAdd(&sc.local_sync[0], 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence_system();
      const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(sc.local_sync + 1) + 1u;
      for (int d = 0; d < sc.tp; ++d) st_release_sys(sc.flag[d] + sc.src_rank, epoch);
      sc.local_sync[0] = 0;
      sc.local_sync[1] = epoch;
    }
  }
}

template <typename T, int STAGES, bool BULK>
static void launch_pair(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N,
                        int K, int lda, int ldw, int ldc, int ldr, int epi, cudaStream_t stream, StatusWord* status,
                        const RowScatter& sc) {
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA = make_tmap_2d(A, dt, 2, M, K, lda, 128, kPairBK);
  CUtensorMap tmB = make_tmap_2d(W, dt, 2, N, K, ldw, 128, kPairBK);
  using L = PairSmem<STAGES, BULK>;
  static_assert(L::kDyn <= 232448, "shared memory budget exceeded");
  auto kern = gemm_pair_kernel<T, STAGES, BULK>;
  // kernel attributes and SM counts are per device
  static bool set[64] = {};
  static int sms_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev = dev < 0 || dev >= 64 ? 0 : dev;
  if (!set[dev]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
    set[dev] = true;
  }
  if (sms_dev[dev] == 0) cudaDeviceGetAttribute(&sms_dev[dev], cudaDevAttrMultiProcessorCount, dev);
  const int sms = sms_dev[dev];
  const int tiles = ceil_div(M, kPairBM) * ceil_div(N, kPairBN);
  int clusters = sms / 2;
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
  cudaLaunchKernelEx(&cfg, kern, tmA, tmB, reinterpret_cast<T*>(C), reinterpret_cast<const T*>(bias),
                     reinterpret_cast<const T*>(residual), M, N, K, ldc, ldr, epi, status, sc);
}

void gemm_tn_pair(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
                  int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int epi,
                  const RowScatter* scatter) {
  if (M <= 0 || N <= 0) return;
  RowScatter sc{};
  if (scatter) sc = *scatter;
  StatusWord* st = reinterpret_cast<StatusWord*>(status);
  // scattered rows leave as bulk copies (B200_SCATTER_BULK=0: plain 16-byte stores, for comparison)
  static const bool bulk_default = [] {
    const char* e = std::getenv("B200_SCATTER_BULK");
    return e == nullptr || std::atoi(e) != 0;
  }();
  const bool bulk = sc.tp > 0 && bulk_default && epi == 0 && residual == nullptr && N % 8 == 0 && ldc % 8 == 0;
#define B200_PAIR(T)                                                                                              \
  do {                                                                                                            \
    if (bulk) launch_pair<T, 4, true>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, ldr, epi, stream, st, sc);  \
    else launch_pair<T, 6, false>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, ldr, epi, stream, st, sc);      \
  } while (0)
  if (dtype == 0) B200_PAIR(__nv_bfloat16);
  else B200_PAIR(__half);
#undef B200_PAIR
}

}  // namespace b200
