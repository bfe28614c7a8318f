// All-gather -> column-parallel GEMM in ONE kernel:
//
//     C[tp*R, N] = concat_r(X_r[R, K]) . W[N, K]^T          X_r lives on rank r (symmetric memory)
//
// The activations are sharded by rows over the tensor-parallel ranks (sequence parallel); every rank needs
// all rows against its own weight shard.  Instead of an NCCL all-gather followed by a GEMM, one persistent
// grid does both:
//   CTAs [0, NC)   "copiers": one thread per CTA streams remote 128-row blocks over NVLink with TMA
//                  (peer memory -> shared ring -> this GPU's gathered buffer, 16 KB per copy, 8 copies in
//                  flight per CTA) so every remote byte crosses NVLink exactly once, and publishes a
//                  per-row-block ready flag;
//   CTAs [NC, G)   GEMM CTAs (TMA producer warp, tcgen05 issuer, 4 epilogue warps, two TMEM accumulators)
//                  walk the row blocks starting with the LOCAL shard, so the tensor cores are busy from the
//                  first microsecond and only wait (bounded) for a remote block that has not landed yet.
// Handshakes (system-scope flags in symmetric memory): "my shard is ready" before a peer pulls, and
// "I have pulled your shard" so the producer of the next step may overwrite it when this kernel ends.
// The grid never exceeds the SM count (one CTA per SM by shared memory), so flag producers and consumers
// are co-resident; every wait is bounded and reports to the status word.
// Replaces tensor_model_parallel_all_gather + the library GEMM of a column-parallel layer
// (collective call site C3 of the reference: vllm ColumnParallelLinear / sequence-parallel MoE input).
#include <type_traits>
#include "comm_fused.cuh"
#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kAgBM = 128, kAgBK = 64;
constexpr int kAgCopyStages = 12, kAgCopyLag = 8;
constexpr int kAgChunkBytes = kAgBM * kAgBK * 2;     // 16 KB

struct AgMaps {
  CUtensorMap peer[kMaxRanks];   // X shard of every rank, box 128 x 64, no swizzle (copier loads)
  CUtensorMap gath_st;           // gathered buffer, same box (copier stores)
  CUtensorMap gath_ld;           // gathered buffer, 128B swizzle (GEMM loads)
  CUtensorMap local_ld;          // own shard, 128B swizzle (GEMM loads)
  CUtensorMap w;                 // weight shard [N, K], box BN x 64, 128B swizzle
};

template <int BN, int STAGES>
struct AgSmem {
  static constexpr int kABytes = kAgBM * kAgBK * 2;
  static constexpr int kBBytes = BN * kAgBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kGemmBytes = STAGES * kStageBytes;
  static constexpr int kCopyBytes = kAgCopyStages * kAgChunkBytes;
  static constexpr int kData = kGemmBytes > kCopyBytes ? kGemmBytes : kCopyBytes;
  static constexpr int kDyn = kData + (2 * STAGES + 4 + kAgCopyStages) * 8 + 16 + 1024;
};

template <typename T, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
ag_gemm_kernel(const __grid_constant__ AgMaps maps, const AgGemmParams p, T* __restrict__ C,
               const T* __restrict__ bias, int num_copiers) {
  using L = AgSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kData);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t epoch = p.sync[0] + 1;
  // pulls of my shard that must have completed when this call ends (the copier count varies per call)
  const uint32_t done_want = p.sync[2] + (uint32_t)((p.tp - 1) * num_copiers);
  const int blocks_per_rank = p.rows_per_rank / kAgBM;
  const int num_mb = blocks_per_rank * p.tp;
  const int num_k = ceil_div(p.K, kAgBK);
  const int first_local = p.rank * blocks_per_rank;

  if ((int)blockIdx.x < num_copiers) {
    // =============================================================== copier CTA
    uint64_t* full = bars;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kAgCopyStages; ++s) mbar_init(&full[s], 1);
      fence_mbar_init();
    }
    __syncthreads();
    if (blockIdx.x == 0 && (int)threadIdx.x < p.tp && (int)threadIdx.x != p.rank)
      st_release_sys(&p.xready[threadIdx.x][p.rank], epoch);          // my shard may be pulled
    if (threadIdx.x == 0) {
      uint32_t it = 0;            // chunks loaded so far (ring position / phase)
      bool ok = true;
      int ready_src = -1;
      const int remote_blocks = num_mb - blocks_per_rank;
      for (int j = blockIdx.x; j < remote_blocks && ok; j += num_copiers) {
        const int mb = (first_local + blocks_per_rank + j) % num_mb;
        const int src = mb / blocks_per_rank;
        if (src != ready_src) {
          uint32_t seen = 0;
          if (!wait_flag_ge(&p.xready[p.rank][src], epoch, p.wait_cycles, &seen)) {
            report_status(p.status, kWaitTimeout, 150, epoch, seen);
            ok = false;
            break;
          }
          ready_src = src;
        }
        const int row_in_shard = (mb - src * blocks_per_rank) * kAgBM;
        const uint32_t base = it;
        for (int i = 0; i < num_k + kAgCopyLag && ok; ++i) {
          if (i < num_k) {
            const uint32_t c = base + i;
            const int s = c % kAgCopyStages;
            tma_store_wait_read<kAgCopyStages - kAgCopyLag - 1>();      // the store that last used this slot has read it
            mbar_expect_tx(&full[s], kAgChunkBytes);
            tma_load_2d(smem + s * kAgChunkBytes, &maps.peer[src], &full[s], i * kAgBK, row_in_shard);
          }
          if (i >= kAgCopyLag) {
            const uint32_t c = base + (i - kAgCopyLag);
            const int s = c % kAgCopyStages;
            if (!mbar_wait(&full[s], (c / kAgCopyStages) & 1)) {
              report_status(p.status, kWaitTimeout, 151, mb, i);
              ok = false;
              break;
            }
            tma_store_2d(&maps.gath_st, smem + s * kAgChunkBytes, (i - kAgCopyLag) * kAgBK, mb * kAgBM);
            tma_store_commit();
          }
        }
        it = base + num_k;
        if (!ok) break;
        tma_store_wait<0>();              // the block is in this GPU's memory
        fence_proxy_async();
        __threadfence();
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ready + mb), "r"(epoch) : "memory");
      }
      tma_store_wait<0>();
      // tell every source that this CTA will not read its shard again in this step
      for (int r = 0; r < p.tp; ++r)
        if (r != p.rank) red_add_release_sys(p.done[r], 1u);
      if (blockIdx.x == 0) {
        uint32_t seen = 0;
        if (p.tp > 1 && !wait_flag_ge(p.done[p.rank], done_want, p.wait_cycles, &seen))
          report_status(p.status, kWaitTimeout, 152, done_want, seen);
      }
    }
  } else {
    // =============================================================== GEMM CTA
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full = empty_bar + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    const int num_n = ceil_div(p.N, BN);
    const int num_tiles = num_mb * num_n;
    const int cta = blockIdx.x - num_copiers, ctas = gridDim.x - num_copiers;
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
        for (int tile = cta; tile < num_tiles && ok; tile += ctas) {
          const int j = tile / num_n, tn = tile % num_n;
          const int mb = (first_local + j) % num_mb;
          const bool local = j < blocks_per_rank;
          if (!local) {
            uint32_t seen = 0;
            const long long t0 = clock64();
            for (;;) {
              uint32_t v;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.ready + mb) : "memory");
              if ((int32_t)(v - epoch) >= 0) break;
              if (clock64() - t0 > p.wait_cycles) { seen = v; ok = false; break; }
              __nanosleep(100);
            }
            if (!ok) {
              report_status(p.status, kWaitTimeout, 153, mb, seen);
              break;
            }
            fence_proxy_async();
          }
          const CUtensorMap* am = local ? &maps.local_ld : &maps.gath_ld;
          const int arow = local ? (mb - first_local) * kAgBM : mb * kAgBM;
          for (int kb = 0; kb < num_k; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
              report_status(p.status, kWaitTimeout, 154, tile, kb);
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * L::kStageBytes;
            mbar_expect_tx(&full_bar[stage], L::kStageBytes);
            tma_load_2d(sa, am, &full_bar[stage], kb * kAgBK, arow);
            tma_load_2d(sa + L::kABytes, &maps.w, &full_bar[stage], kb * kAgBK, tn * BN);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
        constexpr uint32_t idesc = make_idesc(1, fmt, fmt, kAgBM, BN);
        int stage = 0;
        uint32_t phase = 0;
        int it = 0;
        bool ok = true;
        for (int tile = cta; tile < num_tiles && ok; tile += ctas, ++it) {
          const int acc = it & 1;
          if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
            report_status(p.status, kWaitTimeout, 155, tile, acc);
            break;
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int kb = 0; kb < num_k; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase)) {
              report_status(p.status, kWaitTimeout, 156, tile, kb);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
            const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
            for (int k = 0; k < kAgBK / 16; ++k)
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
      for (int tile = cta; tile < num_tiles; tile += ctas, ++it) {
        const int j = tile / num_n, tn = tile % num_n;
        const int mb = (first_local + j) % num_mb;
        const int acc = it & 1;
        if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
          report_status(p.status, kWaitTimeout, 157, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const int row = mb * kAgBM + quarter * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          store_row_segment<T, 32>(r, row, tn * BN + c, p.N, C, p.ldc, bias, nullptr, 0, 0);
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
  // ---- the last CTA to leave advances the epoch (every CTA read it on entry)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(&p.sync[1], 1u);
    if (done == gridDim.x - 1) {
      p.sync[1] = 0;
      p.sync[2] = done_want;
      p.sync[0] = epoch;
    }
  }
}

template <typename T, int BN, int STAGES>
static void launch_ag(const AgGemmParams& p, const void* W, int ldw, void* C, const void* bias, cudaStream_t stream) {
  using L = AgSmem<BN, STAGES>;
  static_assert(L::kDyn <= 232448, "shared memory budget exceeded");
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  AgMaps m;
  const int rows_all = p.rows_per_rank * p.tp;
  for (int r = 0; r < kMaxRanks; ++r)
    m.peer[r] = make_tmap_2d(p.x_shard[r < p.tp ? r : p.rank], dt, 2, p.rows_per_rank, p.K, p.K, kAgBM, kAgBK, false);
  m.gath_st = make_tmap_2d(p.gathered, dt, 2, rows_all, p.K, p.K, kAgBM, kAgBK, false);
  m.gath_ld = make_tmap_2d(p.gathered, dt, 2, rows_all, p.K, p.K, kAgBM, kAgBK, true);
  m.local_ld = make_tmap_2d(p.x_shard[p.rank], dt, 2, p.rows_per_rank, p.K, p.K, kAgBM, kAgBK, true);
  m.w = make_tmap_2d(W, dt, 2, p.N, p.K, ldw, BN, kAgBK, true);
  auto kern = ag_gemm_kernel<T, BN, STAGES>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDyn);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = (rows_all / kAgBM) * ceil_div(p.N, BN);
  const int remote_blocks = (rows_all - p.rows_per_rank) / kAgBM;
  int nc = p.tp > 1 ? (remote_blocks < 16 ? remote_blocks : 16) : 0;
  if (p.tp > 1 && nc < 1) nc = 1;
  int gemm_ctas = tiles < sms - nc ? tiles : sms - nc;
  kern<<<nc + gemm_ctas, 192, L::kDyn, stream>>>(m, p, reinterpret_cast<T*>(C), reinterpret_cast<const T*>(bias), nc);
}

// Number of copier CTAs the launcher uses (the "done" handshake counts them, all ranks must agree).
int ag_gemm_copiers(int tp, int rows_per_rank) {
  if (tp <= 1) return 0;
  const int remote_blocks = (tp - 1) * rows_per_rank / kAgBM;
  return remote_blocks < 16 ? (remote_blocks < 1 ? 1 : remote_blocks) : 16;
}

// rows_per_rank must be a multiple of 128 and K of 64; x_shard rows are contiguous [rows_per_rank, K].
int ag_gemm(const AgGemmParams& p, const void* W, int ldw, void* C, const void* bias, int dtype, cudaStream_t stream) {
  if (p.rows_per_rank % kAgBM != 0 || p.K % 8 != 0) return 1;
  const int tiles256 = (p.rows_per_rank * p.tp / kAgBM) * ceil_div(p.N, 256);
  const bool wide = p.N >= 256 && tiles256 >= 100;
  if (dtype == 0) {
    if (wide) launch_ag<__nv_bfloat16, 256, 4>(p, W, ldw, C, bias, stream);
    else launch_ag<__nv_bfloat16, 128, 6>(p, W, ldw, C, bias, stream);
  } else {
    if (wide) launch_ag<__half, 256, 4>(p, W, ldw, C, bias, stream);
    else launch_ag<__half, 128, 6>(p, W, ldw, C, bias, stream);
  }
  return 0;
}

}  // namespace b200
