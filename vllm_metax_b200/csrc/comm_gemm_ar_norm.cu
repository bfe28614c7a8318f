// ONE kernel for the tensor-parallel row-parallel linear and everything that follows it:
//
//   partial_r = A_r . W_r^T            tcgen05 GEMM on this rank's K shard          (phase A)
//   push      each finished 128 x 128 tile goes straight from TMEM to the receive buffer of the
//             rank that OWNS those rows (peer stores over NVLink), then one release-add on that
//             owner's per-row-block arrival counter
//   reduce    the owner sums the tp partial rows in fp32, adds its shard of the residual
//             stream, writes the new residual, RMS-normalises                      (phase B)
//   gather    and pushes the normalised rows into EVERY rank's output buffer (all-gather),
//   barrier   epoch flags between the ranks close the call                         (phase C)
//
// i.e. GEMM -> reduce-scatter -> +residual -> RMSNorm -> all-gather, replacing
// o_proj/down_proj GEMM + NCCL all-reduce + fused_add_rms_norm (three kernels and two extra
// passes over the activations).  The residual stream stays sharded by rows between calls.
//
// Phase A reuses the single-CTA GEMM pipeline (TMA ring -> tcgen05.mma -> double-buffered
// TMEM).  Tiles are walked row-block-major starting at the NEXT rank's rows, so that at any
// moment the ranks push to different owners and an owner's row blocks complete early.
// Phase B starts on a CTA as soon as its own tiles are done; it only ever waits on counters,
// never on another CTA of its own grid being scheduled (grid <= number of SMs, 1 CTA/SM).
#include <type_traits>

#include "comm_fused.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {
using namespace ptx;

constexpr int kArBM = 128, kArBN = 128, kArBK = 64, kArStages = 6;

struct ArSmem {
  static constexpr int kABytes = kArBM * kArBK * 2;
  static constexpr int kBBytes = kArBN * kArBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kRing = kArStages * kStageBytes;          // reused as the fp32 row stage in phase B
  static constexpr int kBarOffset = kRing;
  static constexpr int kTotal = kBarOffset + (2 * kArStages + 4) * 8 + 64;
  static constexpr int kDyn = kTotal + 1024;
};

template <typename T>
__global__ void __launch_bounds__(192, 1)
gemm_ar_norm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const FusedArParams p) {
  using L = ArSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kArStages;
  uint64_t* tmem_full = empty_bar + kArStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  __shared__ float red[32];
  __shared__ int s_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_rb = ceil_div(p.T, kArBM);
  const int num_n = ceil_div(p.H, kArBN);
  const int num_tiles = num_rb * num_n;
  const int num_k = ceil_div(p.K, kArBK);
  constexpr uint32_t kTmemCols = 2 * kArBN;
  // first row block this rank produces: the one holding the next rank's first row
  const int rb_start = (int)(((int64_t)((p.rank + 1) % p.tp) * p.rows_per_rank) / kArBM) % num_rb;
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

  // ================================================================== phase A: GEMM + push
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int rb = (tile / num_n + rb_start) % num_rb, tn = tile % num_n;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(p.status, kWaitTimeout, 70, tile, kb);
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
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(1, fmt, fmt, kArBM, kArBN);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
          report_status(p.status, kWaitTimeout, 71, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kArBN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(p.status, kWaitTimeout, 72, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kArBK / 16; ++k)
            umma_f16_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kArStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int etid = threadIdx.x - 64;  // 0..127 within the epilogue group
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int rb = (tile / num_n + rb_start) % num_rb, tn = tile % num_n;
      const int acc = it & 1;
      if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1)) {
        report_status(p.status, kWaitTimeout, 73, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const int gr = rb * kArBM + quarter * 32 + lane;         // global row of this thread
      const bool row_ok = gr < p.T;
      const int owner = row_ok ? gr / p.rows_per_rank : 0;
      const int lr = gr - owner * p.rows_per_rank;
      T* dst_row = reinterpret_cast<T*>(p.recv[owner]) + ((size_t)p.rank * p.rows_cap + lr) * p.H;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kArBN;
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
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }

  // ================================================================== phase B: reduce + norm + gather
  const int my_row0 = p.rank * p.rows_per_rank;
  const int my_rows = max(0, min(p.rows_per_rank, p.T - my_row0));
  const uint32_t expected = (uint32_t)(p.tp * num_n);
  float* stage_row = reinterpret_cast<float*>(smem);                 // H floats (H * 4 <= ring bytes)
  const T* recv_mine = reinterpret_cast<const T*>(p.recv[p.rank]);
  T* residual = reinterpret_cast<T*>(p.residual);
  const T* nw = reinterpret_cast<const T*>(p.norm_weight);
  const int nvec = p.H >> 3;
  int ready_rb = -1;
  for (int lr = blockIdx.x; lr < my_rows; lr += gridDim.x) {
    const int gr = my_row0 + lr;
    const int rb = gr / kArBM;
    if (rb != ready_rb) {
      if (threadIdx.x == 0) {
        uint32_t seen = 0;
        const bool ok = wait_flag_ge(my_counters + rb, expected, p.wait_cycles, &seen);
        if (!ok) report_status(p.status, kWaitTimeout, 74, (int)expected, (int)seen);
        s_flag = ok ? 1 : 0;
      }
      __syncthreads();
      ready_rb = rb;
      if (!s_flag) break;  // give up on the data; phase C still runs so that peers are not left waiting
    }
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int src = 0; src < p.tp; ++src) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(recv_mine + ((size_t)src * p.rows_cap + lr) * p.H) + v);
        float f[8];
        unpack8<T>(raw, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      if (p.add_residual) {
        float f[8];
        unpack8<T>(reinterpret_cast<const uint4*>(residual + (size_t)lr * p.H)[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      const uint4 packed = pack8<T>(acc);
      reinterpret_cast<uint4*>(residual + (size_t)lr * p.H)[v] = packed;
      unpack8<T>(packed, acc);  // the norm sees the rounded residual
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        stage_row[v * 8 + i] = acc[i];
        ss += acc[i] * acc[i];
      }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)p.H + p.eps);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8], w[8];
      unpack8<T>(reinterpret_cast<const uint4*>(nw)[v], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = stage_row[v * 8 + i] * inv * w[i];
      const uint4 packed = pack8<T>(f);
      for (int dst = 0; dst < p.tp; ++dst) {
        const int o = (p.rank + dst) % p.tp;   // start with the local copy, then walk the peers
        reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out[o]) + (size_t)gr * p.H)[v] = packed;
      }
    }
    __syncthreads();  // stage_row is reused by the next row
  }

  // ================================================================== phase C: close the call
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
  auto kern = gemm_ar_norm_kernel<T>;
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ArSmem::kDyn);
    set = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // the whole grid must be co-resident (CTAs wait on peers, never on each other)
  kern<<<sms, 192, ArSmem::kDyn, stream>>>(tmA, tmB, p);
}

// Returns 0, or -1 when H does not fit the phase-B row stage.
int gemm_ar_norm(const FusedArParams& p, const void* A, int lda, const void* W, int ldw, int dtype,
                 cudaStream_t stream) {
  if (p.T <= 0) return 0;
  if ((size_t)p.H * 4 > (size_t)ArSmem::kRing || (p.H & 7) != 0) return -1;
  if (dtype == 0) launch_ar<__nv_bfloat16>(p, A, lda, W, ldw, stream);
  else launch_ar<__half>(p, A, lda, W, ldw, stream);
  return 0;
}

}  // namespace b200
