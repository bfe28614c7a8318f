// Stream-K dense GEMM for skinny problems (decode batches, narrow tensor-parallel shards) on CTA pairs:
//
//     C[M,N] = A[M,K] . W[N,K]^T (+ bias) (+ residual) | SiLU-gate epilogue,      M <= a few hundred tokens
//
// With few tokens the GEMM is a weight stream: its speed is set by how many SMs pull on W and by how often the
// activations are re-read.  Here
//   * the WEIGHT is the 256-row operand of tcgen05.mma.cta_group::2 (128 rows per CTA) and the tokens are the
//     N operand (TN <= 256 columns, each CTA of the pair loads half of them), so every W byte is fetched once
//     and an activation tile is shared by 256 output features;
//   * the (tile, k-block) iteration space is cut into equal contiguous ranges, one per persistent CTA pair
//     (stream-K): all SMs stream for the same time whatever N and K are.  A pair whose range covers a whole
//     tile writes it directly; otherwise it stores its fp32 partial in a scratch slot of its own and bumps the
//     tile's arrival counter - the pair that arrives LAST adds the partials in pair order (a fixed order, so
//     results are bit-reproducible) and runs the epilogue.  Nobody waits for anybody: no spin, no atomics on
//     data, and the counter is back at zero when the kernel ends.
//
// Scratch: `ws` holds 2 slots per pair of 256 x 256 floats, `counters` one int per (tile, CTA of the pair).
// All mbarrier waits are bounded.  Replaces the library GEMM behind every unquantised linear layer at decode
// batch sizes (torch.nn.functional.linear in the reference's model files).
#include <type_traits>
#include "comm_fused.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"
#include "ops.h"

namespace b200 {
using namespace ptx;

constexpr int kStkBW = 256;           // weight rows per pair tile (128 per CTA)
constexpr int kStkBT = 256;           // tokens per tile at most
constexpr int kStkBK = 64;
constexpr int kStkStages = 6;
constexpr int kStkMaxContrib = 8;      // partials that may meet in one tile (host plan keeps to it)
constexpr int kStkSlotFloats = 2 * kStkBT * 128;   // one partial tile: [cta][token column][128 lanes]

struct StkSmem {
  static constexpr int kWBytes = 128 * kStkBK * 2;
  static constexpr int kTBytes = 128 * kStkBK * 2;                // room for TN/2 <= 128 token rows
  static constexpr int kStageBytes = kWBytes + kTBytes;
  static constexpr int kBarOffset = kStkStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + (2 * kStkStages + 4) * 8 + 32;
  static constexpr int kDyn = kTotal + 1024;
};

struct StkShape {
  int M, N, K;          // tokens, output features, contraction
  int TN;               // token columns per tile (multiple of 16, <= 256)
  int num_t, num_w;     // token tiles, weight tiles
  int num_k;            // k blocks per tile
  int clusters;         // CTA pairs that share the unit space
};

// Unit u = tile * num_k + kb.  Pair c owns [unit_start(c), unit_start(c + 1)).
__host__ __device__ __forceinline__ long long stk_unit_start(long long units, int clusters, int c) {
  return units * c / clusters;
}
// The pair whose range holds `unit`: the largest c with unit_start(c) <= unit.
__host__ __device__ __forceinline__ int stk_cluster_of(long long units, int clusters, long long unit) {
  return (int)(((unit + 1) * clusters - 1) / units);
}

__device__ __forceinline__ void stk_bar_epilogue() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename T>
__global__ void __launch_bounds__(192, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    T* __restrict__ C, const T* __restrict__ bias, const T* __restrict__ residual, const StkShape sh,
                    int ldc, int ldr, int epi, float* __restrict__ ws, int* __restrict__ counters,
                    StatusWord* status, const __grid_constant__ RowScatter sc) {
  using L = StkSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStkStages;
  uint64_t* tmem_full = empty_bar + kStkStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* arrival = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_k = sh.num_k;
  const long long units = (long long)sh.num_t * sh.num_w * num_k;
  const long long u_begin = stk_unit_start(units, sh.clusters, cluster_id);
  const long long u_end = stk_unit_start(units, sh.clusters, cluster_id + 1);
  const int half_tn = sh.TN >> 1;
  const uint32_t cta_bytes = (uint32_t)(L::kWBytes + half_tn * 128);
  constexpr uint32_t kTmemCols = 512;            // two accumulator buffers of up to 256 token columns

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStkStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 256);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
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
      for (long long u = u_begin; u < u_end && ok;) {
        const int tile = (int)(u / num_k), k0 = (int)(u % num_k);
        const int k1 = (int)min((long long)num_k, k0 + (u_end - u));
        const int tw = tile / sh.num_t, tt = tile % sh.num_t;
        const int row_w = tw * kStkBW + (int)rank * 128;
        const int row_x = tt * kStkBT + (int)rank * half_tn;
        for (int kb = k0; kb < k1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 170, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sw = smem + stage * L::kStageBytes;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * cta_bytes);
          tma_load_2d_pair(sw, &tmW, &full_bar[stage], kb * kStkBK, row_w);
          tma_load_2d_pair(sw + L::kWBytes, &tmX, &full_bar[stage], kb * kStkBK, row_x);
          if (++stage == kStkStages) { stage = 0; phase ^= 1; }
        }
        u += k1 - k0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      const uint32_t idesc = make_idesc(1, fmt, fmt, kStkBW, (uint32_t)sh.TN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (long long u = u_begin; u < u_end && ok; ++it) {
        const int tile = (int)(u / num_k), k0 = (int)(u % num_k);
        const int k1 = (int)min((long long)num_k, k0 + (u_end - u));
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          report_status(status, kWaitTimeout, 171, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kStkBT;
        for (int kb = k0; kb < k1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 172, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sw = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t dw = make_smem_desc_sw128(sw);
          const uint64_t dx = make_smem_desc_sw128(sw + L::kWBytes);
#pragma unroll
          for (int k = 0; k < kStkBK / 16; ++k)
            umma_f16_ss_pair(d_tmem, dw + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc,
                             (kb != k0 || k != 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage], 0x3);
          if (++stage == kStkStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 0x3);
        u += k1 - k0;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                     // TMEM lane = weight row within this CTA's half
    const int epi_tid = (int)threadIdx.x - 64;
    const uint32_t leader_empty0 = mapa(smem_u32(&tmem_empty[0]), 0);
    const uint32_t leader_empty1 = mapa(smem_u32(&tmem_empty[1]), 0);
    int it = 0;
    for (long long u = u_begin; u < u_end; ++it) {
      const int tile = (int)(u / num_k), k0 = (int)(u % num_k);
      const int k1 = (int)min((long long)num_k, k0 + (u_end - u));
      u += k1 - k0;
      const int tw = tile / sh.num_t, tt = tile % sh.num_t;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase)) {
        report_status(status, kWaitTimeout, 173, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kStkBT;
      const bool complete = (k0 == 0 && k1 == num_k);
      const long long tile_u0 = (long long)tile * num_k;
      int c_first = cluster_id, c_last = cluster_id;
      bool finish = true;
      if (!complete) {
        // park this pair's partial: head partial (the tile began in an earlier pair) in slot 0, tail in slot 1
        const int which = k0 > 0 ? 0 : 1;
        float* dst = ws + (size_t)(cluster_id * 2 + which) * kStkSlotFloats + (size_t)rank * (kStkBT * 128) + row;
#pragma unroll 1
        for (int c = 0; c < sh.TN; c += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) dst[(c + i) * 128] = __uint_as_float(r[i]);
        }
        __threadfence();
        stk_bar_epilogue();
        if (epi_tid == 0) *arrival = atomicAdd(&counters[tile * 2 + (int)rank], 1);
        stk_bar_epilogue();
        c_first = stk_cluster_of(units, sh.clusters, tile_u0);
        c_last = stk_cluster_of(units, sh.clusters, tile_u0 + num_k - 1);
        finish = (*arrival == c_last - c_first);             // every other contributor has already arrived
        if (finish) {
          __threadfence();
          if (epi_tid == 0) counters[tile * 2 + (int)rank] = 0;   // ready for the next launch
        }
      }
      if (finish && !complete) {
        // Every partial of this tile half (this pair's own included) sits in scratch as [token column][lane].
        // The 128 epilogue threads walk it flat, four lanes (= four output features) per float4, with the loads
        // of every contributor and of four units in flight together; contributors are added in pair order, so
        // the result does not depend on who arrived last.
        const int n = min(c_last - c_first + 1, kStkMaxContrib);
        if (c_last - c_first + 1 > kStkMaxContrib) report_status(status, kBadIndex, 174, kStkMaxContrib, c_last - c_first + 1);
        const float* src[kStkMaxContrib];
#pragma unroll
        for (int k = 0; k < kStkMaxContrib; ++k) {
          const int cc = c_first + (k < n ? k : 0);
          const int which = stk_unit_start(units, sh.clusters, cc) > tile_u0 ? 0 : 1;
          src[k] = ws + (size_t)(cc * 2 + which) * kStkSlotFloats + (size_t)rank * (kStkBT * 128);
        }
        const int units4 = sh.TN * 32;                       // float4 units of this CTA's half tile
        const int feat0 = tw * kStkBW + (int)rank * 128;
#pragma unroll 1
        for (int u0 = epi_tid; u0 < units4; u0 += 4 * 128) {
          float4 v[kStkMaxContrib][4];
#pragma unroll
          for (int k = 0; k < kStkMaxContrib; ++k)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int u = u0 + q * 128;
              v[k][q] = (k < n && u < units4) ? __ldcg(reinterpret_cast<const float4*>(src[k]) + u)
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int u = u0 + q * 128;
            if (u >= units4) break;
            float4 a = v[0][q];
#pragma unroll
            for (int k = 1; k < kStkMaxContrib; ++k) {
              if (k < n) { a.x += v[k][q].x; a.y += v[k][q].y; a.z += v[k][q].z; a.w += v[k][q].w; }
            }
            const int col = u >> 5, l4 = (u & 31) << 2;
            const int tok = tt * kStkBT + col, ra = feat0 + l4;
            if (tok >= sh.M || ra >= sh.N) continue;
            float f[4] = {a.x, a.y, a.z, a.w};
            if (bias) {
#pragma unroll
              for (int e = 0; e < 4; ++e) if (ra + e < sh.N) f[e] += to_f(bias[ra + e]);
            }
            T* crow;
            if (sc.tp > 0) {
              const int owner = tok / sc.rows_per_rank;
              crow = reinterpret_cast<T*>(sc.recv[owner]) +
                     (size_t)(sc.src_rank * sc.rows_cap + tok - owner * sc.rows_per_rank) * ldc;
            } else {
              crow = C + (size_t)tok * ldc;
            }
            if (epi == 1) {
              // interleaved (gate, up) features: two outputs per four lanes
              T o2[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const float g = to_f(from_f<T>(f[2 * e])), up = to_f(from_f<T>(f[2 * e + 1]));
                o2[e] = from_f<T>(g / (1.f + __expf(-g)) * up);
              }
              if (ra + 3 < sh.N) *reinterpret_cast<uint32_t*>(crow + (ra >> 1)) = *reinterpret_cast<const uint32_t*>(o2);
              else if (ra + 1 < sh.N) crow[ra >> 1] = o2[0];
            } else {
              if (residual && sc.tp == 0) {
#pragma unroll
                for (int e = 0; e < 4; ++e) if (ra + e < sh.N) f[e] += to_f(residual[(size_t)tok * ldr + ra + e]);
              }
              if (ra + 3 < sh.N) {
                T o4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) o4[e] = from_f<T>(f[e]);
                *reinterpret_cast<uint2*>(crow + ra) = *reinterpret_cast<const uint2*>(o4);
              } else {
                for (int e = 0; e < 4 && ra + e < sh.N; ++e) crow[ra + e] = from_f<T>(f[e]);
              }
            }
          }
        }
      } else if (finish) {
        const int ra = tw * kStkBW + (int)rank * 128 + row;  // output feature of this lane
        const bool ra_ok = ra < sh.N;
        const float bv = (bias && ra_ok) ? to_f(bias[ra]) : 0.f;
#pragma unroll 1
        for (int c = 0; c < sh.TN; c += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr + c, r);
          tmem_ld_wait();
          float a[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = __uint_as_float(r[i]);
          const int tok0 = tt * kStkBT + c;
          if (epi == 1) {
            // lanes hold interleaved (gate, up) features: even lane = gate, odd lane = up
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g = to_f(from_f<T>(a[i] + bv));
              const float up = __shfl_down_sync(0xffffffffu, g, 1);
              if ((lane & 1) == 0 && ra_ok && tok0 + i < sh.M)
                C[(size_t)(tok0 + i) * ldc + (ra >> 1)] = from_f<T>(g / (1.f + __expf(-g)) * up);
            }
          } else if (ra_ok) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int tok = tok0 + i;
              if (tok < sh.M) {
                float f = a[i] + bv;
                if (sc.tp > 0) {
                  // the token's row lives in the receive slot of the rank that owns it
                  const int owner = tok / sc.rows_per_rank;
                  reinterpret_cast<T*>(sc.recv[owner])[(size_t)(sc.src_rank * sc.rows_cap + tok -
                                                                 owner * sc.rows_per_rank) * ldc + ra] = from_f<T>(f);
                } else {
                  if (residual) f += to_f(residual[(size_t)tok * ldr + ra]);
                  C[(size_t)tok * ldc + ra] = from_f<T>(f);
                }
              }
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
  cluster_sync();                                // no CTA leaves while its peer may still touch it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (sc.tp > 0 && threadIdx.x == 0) {
    // the last CTA of the launch tells every owner that this source's rows have landed
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

// How the (tile, k-block) space is shared out for a problem; clusters == 0: not a stream-K shape.
static StkShape stk_plan(int M, int N, int K, int sms) {
  StkShape sh{};
  sh.M = M; sh.N = N; sh.K = K;
  sh.TN = M >= kStkBT ? kStkBT : ((M + 15) / 16) * 16;
  sh.num_t = ceil_div(M, kStkBT);
  sh.num_w = ceil_div(N, kStkBW);
  sh.num_k = ceil_div(K, kStkBK);
  const long long tiles = (long long)sh.num_t * sh.num_w;
  const long long units = tiles * sh.num_k;
  long long c = sms / 2;
  if (c > 6 * tiles) c = 6 * tiles;          // keeps the partials that meet in one tile within kStkMaxContrib
  if (c > units / 4) c = units / 4;          // at least 4 k-blocks per pair
  if (c < 1) c = 1;
  sh.clusters = (int)c;
  return sh;
}

size_t gemm_streamk_workspace_bytes(int sms) { return (size_t)(sms / 2) * 2 * kStkSlotFloats * sizeof(float); }
int gemm_streamk_max_tiles() { return 8192; }

template <typename T>
static void launch_stk(const void* A, const void* W, void* C, const void* bias, const void* residual,
                       const StkShape& sh, int lda, int ldw, int ldc, int ldr, int epi, float* ws, int* counters,
                       cudaStream_t stream, StatusWord* status, const RowScatter& sc) {
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmW = make_tmap_2d(W, dt, 2, sh.N, sh.K, ldw, 128, kStkBK);
  CUtensorMap tmX = make_tmap_2d(A, dt, 2, sh.M, sh.K, lda, sh.TN / 2, kStkBK);
  auto kern = gemm_streamk_kernel<T>;
  static bool set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set[dev]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, StkSmem::kDyn);
    set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sh.clusters, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = StkSmem::kDyn;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, tmW, tmX, reinterpret_cast<T*>(C), reinterpret_cast<const T*>(bias),
                     reinterpret_cast<const T*>(residual), sh, ldc, ldr, epi, ws, counters, status, sc);
}

// Returns 0 when launched, -1 when the shape is outside what the scratch buffers cover.
// `ws` must hold gemm_streamk_workspace_bytes(sms) bytes, `counters` 2 * gemm_streamk_max_tiles() zeroed ints.
int gemm_tn_streamk(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
                    int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int epi,
                    float* ws, int* counters, int sms, const RowScatter* scatter) {
  if (M <= 0 || N <= 0) return 0;
  RowScatter sc{};
  if (scatter) sc = *scatter;
  const StkShape sh = stk_plan(M, N, K, sms);
  if ((long long)sh.num_t * sh.num_w > gemm_streamk_max_tiles() || K <= 0) return -1;
  StatusWord* st = reinterpret_cast<StatusWord*>(status);
  if (dtype == 0)
    launch_stk<__nv_bfloat16>(A, W, C, bias, residual, sh, lda, ldw, ldc, ldr, epi, ws, counters, stream, st, sc);
  else
    launch_stk<__half>(A, W, C, bias, residual, sh, lda, ldw, ldc, ldr, epi, ws, counters, stream, st, sc);
  return 0;
}

}  // namespace b200
