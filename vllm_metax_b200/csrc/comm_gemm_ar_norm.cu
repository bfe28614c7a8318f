// ONE kernel for the tensor-parallel row-parallel linear and everything that follows it:
//
//   partial_r = A_r . W_r^T            tcgen05 GEMM on this rank's K shard (128 x 256 tiles)
//   push      each finished tile goes from TMEM to the receive buffer of the rank that OWNS those rows over
//             NVLink, then one release-add on that owner's per-row-block arrival counter
//   reduce    the owner sums the tp partial rows in fp32, adds its shard of the residual stream, writes the new
//             residual, RMS-normalises
//   gather    and stores the normalised rows into EVERY rank's output buffer (all-gather)
//   barrier   epoch flags between the ranks close the call
//
// i.e. GEMM -> reduce-scatter -> +residual -> RMSNorm -> all-gather, replacing o_proj/down_proj GEMM + NCCL
// all-reduce + fused_add_rms_norm (three kernels and two extra passes over the activations).  The residual stream
// stays sharded by rows between calls.
//
// Overlap: every rank walks the row blocks in the SAME order, so row block b has all of its partials shortly after
// the ranks pass it, and its reduction runs while later blocks are still being multiplied.  The reduction is done by
// the four epilogue warps of every CTA in the gaps between tiles (they are idle while the tensor core works on
// the next tile): a CTA owns every grid-th row of this rank's shard, polls the block's counter without blocking,
// and its 128 epilogue threads reduce a ready row together, each issuing all of its loads before using any (one
// memory round trip per row instead of one per vector); what is left when the CTA runs out of tiles is finished
// with bounded waits.  Measured on this part, one SM pushes 27 (plain stores) to 46 GB/s (bulk stores) into a
// peer and the pair link saturates near 610 GB/s, so the all-gather stores are spread over all SMs.
//
// Push path: when every 128-row block has a single owner (rows_per_rank % 128 == 0) a finished tile is converted
// into a 128B-swizzled shared-memory stage, 128 columns at a time, and leaves as TMA tensor stores (large NVLink
// writes); the arrival counter of tile i is bumped once its bulk groups have completed, which is checked after
// the first group of tile i+1 has been issued, so the round trip stays off the critical path.  Otherwise (small
// or ragged T) rows are pushed with plain 16-byte stores.
// CTAs never wait on another CTA of their own grid (grid = number of SMs, 1 CTA / SM); every wait is bounded.
#include <cstdlib>
#include <type_traits>

#include "comm_fused.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kArBM = 128, kArBN = 256, kArBK = 64, kArStages = 4;   // 48 KB per stage

struct ArPushMaps {
  CUtensorMap recv[kMaxRanks];   // every owner's receive buffer as [tp * rows_cap, H] rows, box 128 x 64, SW128
};

struct ArSmem {
  static constexpr int kABytes = kArBM * kArBK * 2;
  static constexpr int kBBytes = kArBN * kArBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kRing = kArStages * kStageBytes;
  static constexpr int kPushStage = kRing;                        // 128 x 128 16-bit half tile for the TMA push
  static constexpr int kBarOffset = kRing + kArBM * 128 * 2;
  static constexpr int kTotal = kBarOffset + (2 * kArStages + 4) * 8 + 64;
  static constexpr int kDyn = kTotal + 1024;
};

template <typename T, bool TMA_PUSH>
__global__ void __launch_bounds__(192, 1)
gemm_ar_norm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ ArPushMaps push, const FusedArParams p) {
  using L = ArSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kArStages;
  uint64_t* tmem_full = empty_bar + kArStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_rb = ceil_div(p.T, kArBM);
  const int num_n = ceil_div(p.H, kArBN);
  const int num_tiles = num_rb * num_n;
  const int num_k = ceil_div(p.K, kArBK);
  // Split-K for small token counts: a work unit is (tile, K range); every range lands in a receive slot of its
  // own, so the owner's row reduction sums tp * ksplit partials instead of tp.
  const int num_units = num_tiles * p.ksplit;
  const int k_per = ceil_div(num_k, p.ksplit);
  constexpr uint32_t kTmemCols = 2 * kArBN;
  // The call's epoch lives in device memory (local_sync[1] holds the last finished epoch) so that a
  // CUDA-graph replay of this launch still advances it; every rank issues the same call sequence.
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 1) + 1u;
  const int parity = (int)(epoch & 1u);
  uint32_t* my_counters = p.counters[p.rank] + (size_t)parity * p.rb_cap;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kArStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
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
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int tile = unit / p.ksplit, ks = unit - tile * p.ksplit;
        const int rb = tile / num_n, tn = tile % num_n;     // row-block-major, the same order on every rank
        const int kb1 = min(num_k, (ks + 1) * k_per);
        for (int kb = ks * k_per; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(p.status, kWaitTimeout, 70, unit, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * kArBK, rb * kArBM);
          tma_load_2d(sa + L::kABytes, &tmB, &full_bar[stage], kb * kArBK, tn * kArBN);
          if (++stage == kArStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(1, fmt, fmt, kArBM, kArBN);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
          report_status(p.status, kWaitTimeout, 71, unit, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kArBN;
        const int ks = unit % p.ksplit, kb0 = ks * k_per, kb1 = min(num_k, kb0 + k_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(p.status, kWaitTimeout, 72, unit, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kArBK / 16; ++k)
            umma_f16_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kArStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps: push tiles, reduce rows
    const int quarter = warp & 3;
    const int etid = threadIdx.x - 64;  // 0..127 within the epilogue group
    const int my_row0 = p.rank * p.rows_per_rank;
    const int my_rows = max(0, min(p.rows_per_rank, p.T - my_row0));
    const uint32_t expected = (uint32_t)(p.tp * num_n * p.ksplit);
    const int num_src = p.tp * p.ksplit;
    const T* recv_mine = reinterpret_cast<const T*>(p.recv[p.rank]);
    T* residual = reinterpret_cast<T*>(p.residual);
    const T* nw = reinterpret_cast<const T*>(p.norm_weight);
    const int nvec = p.H >> 3;
    // Rows of this CTA: lr = cta + k * grid.  The 128 epilogue threads reduce a row together: every thread issues
    // all of its loads (up to 4 vectors x 4 sources) before using any, so a row costs about one memory round trip.
    __shared__ float s_part[4];
    __shared__ int s_go;
    const int row_stride = (int)gridDim.x;
    int next_lr = (int)blockIdx.x, ready_rb = -1;
    bool gave_up = false;

    auto reduce_rows = [&](int max_rows, bool blocking) {
      while (max_rows-- > 0 && next_lr < my_rows && !gave_up) {
        const int lr = next_lr, gr = my_row0 + lr;
        const int rb = gr / kArBM;
        if (rb != ready_rb) {
          if (etid == 0) {
            int ok;
            if (blocking) {
              uint32_t seen = 0;
              ok = wait_flag_ge(my_counters + rb, expected, p.wait_cycles, &seen) ? 1 : -1;
              if (ok < 0) report_status(p.status, kWaitTimeout, 74, (int)expected, (int)seen);
            } else {
              ok = (int32_t)(ld_acquire_sys(my_counters + rb) - expected) >= 0 ? 1 : 0;
            }
            s_go = ok;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int ok = s_go;
          asm volatile("bar.sync 1, 128;" ::: "memory");   // s_go may be rewritten by the next check
          if (ok < 0) { gave_up = true; return; }   // the data will not come; the closing barrier still runs
          if (ok == 0) return;
          ready_rb = rb;
        }
        T* res_row = residual + (size_t)lr * p.H;
        for (int v0 = 0; v0 < nvec; v0 += 512) {   // 512 vectors (4096 elements) per pass of the 128 threads
          float acc[4][8];
          bool live[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            live[j] = v0 + j * 128 + etid < nvec;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
          }
          for (int s0 = 0; s0 < num_src; s0 += 4) {
            uint4 raw[4][4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (s0 + q < num_src && live[j])
                  raw[q][j] = __ldcg(reinterpret_cast<const uint4*>(recv_mine + ((size_t)(s0 + q) * p.slot_rows + lr) * p.H) +
                                     v0 + j * 128 + etid);
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (s0 + q < num_src && live[j]) {
                  float f[8];
                  unpack8<T>(raw[q][j], f);
#pragma unroll
                  for (int i = 0; i < 8; ++i) acc[j][i] += f[i];
                }
          }
          float ss = 0.f;
          uint4 keep[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (!live[j]) continue;
            const int v = v0 + j * 128 + etid;
            if (p.add_residual) {
              float f[8];
              unpack8<T>(reinterpret_cast<const uint4*>(res_row)[v], f);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[j][i] += f[i];
            }
            keep[j] = pack8<T>(acc[j]);
            reinterpret_cast<uint4*>(res_row)[v] = keep[j];
            float f[8];
            unpack8<T>(keep[j], f);  // the norm sees the rounded residual
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
          }
          // H <= 4096: one pass covers the row and the values stay in registers; longer rows are re-read below
          if (nvec <= 512) {
            ss = warp_sum(ss);
            if (lane == 0) s_part[warp - 2] = ss;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const float inv = rsqrtf((s_part[0] + s_part[1] + s_part[2] + s_part[3]) / (float)p.H + p.eps);
            asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (!live[j]) continue;
              const int v = v0 + j * 128 + etid;
              float f[8], w[8];
              unpack8<T>(keep[j], f);
              unpack8<T>(reinterpret_cast<const uint4*>(nw)[v], w);
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * w[i];
              const uint4 packed = pack8<T>(f);
              for (int dst = 0; dst < p.tp; ++dst) {
                const int o = (p.rank + dst) % p.tp;   // start with the local copy, then walk the peers
                reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out[o]) + (size_t)gr * p.H)[v] = packed;
              }
            }
          } else {
            ss = warp_sum(ss);
            if (lane == 0) atomicAdd(&s_part[0], ss);   // accumulated over the passes (zeroed below)
          }
        }
        if (nvec > 512) {
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const float inv = rsqrtf(s_part[0] / (float)p.H + p.eps);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (etid == 0) s_part[0] = 0.f;
          for (int v = etid; v < nvec; v += 128) {
            float f[8], w[8];
            unpack8<T>(reinterpret_cast<const uint4*>(res_row)[v], f);
            unpack8<T>(reinterpret_cast<const uint4*>(nw)[v], w);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * w[i];
            const uint4 packed = pack8<T>(f);
            for (int dst = 0; dst < p.tp; ++dst) {
              const int o = (p.rank + dst) % p.tp;
              reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out[o]) + (size_t)gr * p.H)[v] = packed;
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        next_lr += row_stride;
      }
    };
    if (etid == 0) s_part[0] = 0.f;
    asm volatile("bar.sync 1, 128;" ::: "memory");

    int it = 0;
    int prev_rb = -1, prev_owner = 0;   // TMA push: the tile whose arrival is not yet published
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++it) {
      const int tile = unit / p.ksplit;
      const int slot = p.rank * p.ksplit + (unit - tile * p.ksplit);   // receive slot of this (source, K range)
      const int rb = tile / num_n, tn = tile % num_n;
      const int acc = it & 1;
      if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
        report_status(p.status, kWaitTimeout, 73, unit, acc);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kArBN;
      if constexpr (TMA_PUSH) {
        const int row = quarter * 32 + lane;                   // row inside the tile
        uint8_t* stg = smem + L::kPushStage;
        const int owner = (rb * kArBM) / p.rows_per_rank;
        const int lr0 = slot * p.slot_rows + rb * kArBM - owner * p.rows_per_rank;   // row in the owner's buffer
#pragma unroll 1
        for (int h = 0; h < kArBN / 128; ++h) {                // the tile leaves in 128-column halves
          if (etid == 0) tma_store_wait_read<0>();              // earlier stores have read the stage
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + h * 128 + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
              const int chunk = ((c & 63) >> 3) + v;            // 16-byte chunk inside the 64-column box
              uint8_t* box = stg + (c >> 6) * (kArBM * 128);
              *reinterpret_cast<uint4*>(box + row * 128 + ((chunk ^ (row & 7)) << 4)) = pack8<T>(f);
            }
          }
          if (h == kArBN / 128 - 1) {
            tc_fence_before_sync();
            mbar_arrive(&tmem_empty[acc]);
          }
          fence_proxy_async();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (etid == 0) {
            tma_store_2d(&push.recv[owner], stg, tn * kArBN + h * 128, lr0);
            tma_store_2d(&push.recv[owner], stg + kArBM * 128, tn * kArBN + h * 128 + 64, lr0);
            tma_store_commit();
            if (h == 0 && prev_rb >= 0) {                       // every group of tile i-1 has landed: publish it
              tma_store_wait<1>();
              fence_proxy_async();
              __threadfence_system();
              red_add_release_sys(p.counters[prev_owner] + (size_t)parity * p.rb_cap + prev_rb, 1u);
            }
          }
        }
        if (etid == 0) {
          prev_rb = rb;
          prev_owner = owner;
        }
      } else {
        const int gr = rb * kArBM + quarter * 32 + lane;         // global row of this thread
        const bool row_ok = gr < p.T;
        const int owner = row_ok ? gr / p.rows_per_rank : 0;
        const int lr = gr - owner * p.rows_per_rank;
        T* dst_row = reinterpret_cast<T*>(p.recv[owner]) + ((size_t)slot * p.slot_rows + lr) * p.H;
#pragma unroll 1
        for (int c = 0; c < kArBN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          const int col0 = tn * kArBN + c;
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 + 8 <= p.H) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
                *reinterpret_cast<uint4*>(dst_row + col0 + v * 8) = pack8<T>(f);
              }
            }
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&tmem_empty[acc]);
        // publish: every thread's peer stores are ordered before the counter bump
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (etid == 0) {
          const int r0 = rb * kArBM, r1 = min(p.T, r0 + kArBM) - 1;
          for (int o = r0 / p.rows_per_rank; o <= r1 / p.rows_per_rank; ++o)
            red_add_release_sys(p.counters[o] + (size_t)parity * p.rb_cap + rb, 1u);
        }
      }
      // the tensor core is busy with the next tile: reduce rows whose partials have all arrived
      reduce_rows(p.rows_per_gap, false);
    }
    if (TMA_PUSH && etid == 0 && prev_rb >= 0) {               // the last tile of this CTA
      tma_store_wait<0>();
      fence_proxy_async();
      __threadfence_system();
      red_add_release_sys(p.counters[prev_owner] + (size_t)parity * p.rb_cap + prev_rb, 1u);
    }
    reduce_rows(1 << 30, true);                                // whatever is left, with bounded waits
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }

  // ================================================================== close the call
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&p.local_sync[0], 1u);
    if (prev == gridDim.x - 1) {
      // every CTA of this rank has pushed and fenced: tell the peers, then wait for theirs
      __threadfence_system();
      for (int o = 0; o < p.tp; ++o) st_release_sys(p.flags[o] + p.rank, epoch);
      for (int src = 0; src < p.tp; ++src) {
        uint32_t seen = 0;
        if (!wait_flag_ge(p.flags[p.rank] + src, epoch, p.wait_cycles, &seen))
          report_status(p.status, kWaitTimeout, 75, (int)epoch, (int)seen);
      }
      // counters of this parity are next used two calls from now
      for (int i = 0; i < num_rb; ++i) my_counters[i] = 0;
      p.local_sync[0] = 0;
      p.local_sync[1] = epoch;
      __threadfence_system();
    }
  }
}

template <typename T>
static void launch_ar(const FusedArParams& p, const void* A, int lda, const void* W, int ldw, cudaStream_t stream) {
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA = make_tmap_2d(A, dt, 2, p.T, p.K, lda, kArBM, kArBK);
  CUtensorMap tmB = make_tmap_2d(W, dt, 2, p.H, p.K, ldw, kArBN, kArBK);
  // tuning knobs (read once): B200_AR_TMA_PUSH=0 forces plain-store pushes, B200_AR_ROWS_PER_GAP=n rows a warp
  // may reduce between two tiles
  static const int env_push = [] { const char* e = std::getenv("B200_AR_TMA_PUSH"); return e ? std::atoi(e) : 1; }();
  static const int env_gap = [] { const char* e = std::getenv("B200_AR_ROWS_PER_GAP"); return e ? std::atoi(e) : 4; }();
  static const int env_split = [] { const char* e = std::getenv("B200_AR_KSPLIT"); return e ? std::atoi(e) : 0; }();
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // Split-K while the tiles alone leave SMs idle: every K range keeps >= 4 k-blocks, no range is empty, and the
  // tp * ksplit receive slots fit the buffer sized for tp sources of rows_cap rows.
  const int num_tiles = ((p.T + kArBM - 1) / kArBM) * ((p.H + kArBN - 1) / kArBN);
  const int num_k = (p.K + kArBK - 1) / kArBK;
  auto split_ok = [&](int s) {
    const int per = (num_k + s - 1) / s;
    return per * (s - 1) < num_k && ((p.rows_cap / s) & ~7) >= p.rows_per_rank;
  };
  int ksplit = 1;
  if (env_split > 0) {
    ksplit = env_split;
  } else {
    while (ksplit < 8 && num_tiles * ksplit * 2 <= sms && num_k / (ksplit * 2) >= 4) ksplit *= 2;
  }
  while (ksplit > 1 && !split_ok(ksplit)) --ksplit;
  // TMA tensor stores push whole 128-row boxes: every box must stay inside one owner's slot
  const bool tma_push = env_push != 0 && p.rows_per_rank % kArBM == 0 && p.H % 64 == 0;
  ArPushMaps maps;
  for (int r = 0; r < kMaxRanks; ++r) {
    const int o = r < p.tp ? r : p.rank;
    maps.recv[r] = make_tmap_2d(p.recv[o], dt, 2, tma_push ? (uint64_t)p.tp * p.rows_cap : 8, p.H, p.H,
                                tma_push ? kArBM : 8, 64);
  }
  auto kern = tma_push ? gemm_ar_norm_kernel<T, true> : gemm_ar_norm_kernel<T, false>;
  static bool set[2] = {false, false};
  if (!set[tma_push]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ArSmem::kDyn);
    set[tma_push] = true;
  }
  FusedArParams q = p;
  q.rows_per_gap = env_gap;
  q.ksplit = ksplit;
  q.slot_rows = ksplit == 1 ? p.rows_cap : ((p.rows_cap / ksplit) & ~7);
  // the whole grid must be co-resident (CTAs wait on peers, never on each other)
  kern<<<sms, 192, ArSmem::kDyn, stream>>>(tmA, tmB, maps, q);
}

// Returns 0, or -1 when H is not a multiple of 8.
int gemm_ar_norm(const FusedArParams& p, const void* A, int lda, const void* W, int ldw, int dtype,
                 cudaStream_t stream) {
  if (p.T <= 0) return 0;
  if ((p.H & 7) != 0) return -1;
  if (dtype == 0) launch_ar<__nv_bfloat16>(p, A, lda, W, ldw, stream);
  else launch_ar<__half>(p, A, lda, W, ldw, stream);
  return 0;
}

}  // namespace b200
