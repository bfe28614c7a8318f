// Dense bf16/fp16 GEMM on the 5th-generation tensor cores:
//
//     C[M,N] = A[M,K] . W[N,K]^T  (+ bias[N]) (+ residual[M,N])
//
// (the nn.Linear contraction; replaces the library GEMM the reference reaches
// through torch.nn.functional.linear for every unquantised linear layer).
//
// Design (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: 128B-swizzled K-major tiles of A (128 x 64) and W
//               (BN x 64) into a STAGES-deep shared-memory ring, mbarrier tx-count.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma
//               (cta_group::1, kind::f16, M=128, N=BN, K=16) into one of two
//               TMEM accumulator buffers; tcgen05.commit releases ring slots and
//               publishes finished accumulators.
//   warps 2-5   epilogue: tcgen05.ld (32 lanes x 32 columns), bias / residual add,
//               bf16 convert, 64-byte row segments to global.  Runs concurrently
//               with the next tile's main loop thanks to the second TMEM buffer.
//
// SWAP variant (small M, decode): the weight is the 128-row MMA operand and the
// activations are the N operand (BN = 16/32/64 tokens), so a handful of tokens do
// not waste a 128-row tile; the epilogue writes the transposed tile.
//
// All mbarrier waits are bounded; a timeout is recorded in the status word and
// the CTA drains and frees its TMEM.
#include <type_traits>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"

namespace b200 {

using namespace ptx;

constexpr int kBM = 128;
constexpr int kBK = 64;  // 64 x 16-bit = 128 bytes = one swizzle row

template <int BN, int STAGES>
struct GemmSmemLayout {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16;
  static constexpr int kDynSmem = kTotal + 1024;  // slack for 1024-byte alignment
};

template <typename T, int BN, int STAGES, bool SWAP>
__global__ void __launch_bounds__(192, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA,   // 128-row operand
               const __grid_constant__ CUtensorMap tmB,   // BN-row operand
               T* __restrict__ C, const T* __restrict__ bias, const T* __restrict__ residual,
               int rows_a, int rows_b, int K, int ldc, int ldr, int epi, StatusWord* status) {
  using L = GemmSmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_a = ceil_div(rows_a, kBM);
  const int num_b = ceil_div(rows_b, BN);
  const int num_tiles = num_a * num_b;
  const int num_k = ceil_div(K, kBK);
  constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;

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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        // consecutive CTAs share the BN-row operand tile (same tb) and walk the 128-row operand
        const int ta = tile % num_a, tb = tile / num_a;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_status(status, kWaitTimeout, 1, tile, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * kBK, ta * kBM);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * kBK, tb * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;  // 0 = f16, 1 = bf16
      constexpr uint32_t idesc = make_idesc(/*c=f32*/ 1, fmt, fmt, kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          report_status(status, kWaitTimeout, 2, tile, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_status(status, kWaitTimeout, 3, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // advance 16 elements (32 bytes) along K inside the swizzled row: +2 in 16-byte units
            umma_f16_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // slot reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int ta = tile % num_a, tb = tile / num_a;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase)) {
        report_status(status, kWaitTimeout, 4, tile, acc);
        break;
      }
      tc_fence_after_sync();
      const int ra = ta * kBM + quarter * 32 + lane;  // row index in the 128-row operand
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      constexpr int CH = (BN >= 32) ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < BN; c += CH) {
        uint32_t r[32];
        if constexpr (CH == 32) {
          tmem_ld_32x32b_x32(taddr + c, r);
        } else {
          uint32_t r16[16];
          tmem_ld_32x32b_x16(taddr + c, r16);
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = r16[i];
        }
        tmem_ld_wait();
        const int cb0 = tb * BN + c;  // first index in the BN-row operand
        if constexpr (!SWAP) {
          // row = token (ra), columns = output features cb0..cb0+CH
          if (ra < rows_a && epi == 1) {
            // columns hold interleaved (gate, up) pairs: out[:, j] = silu(gate_j) * up_j
            T* dst = C + (size_t)ra * ldc + (cb0 >> 1);
#pragma unroll
            for (int v = 0; v < CH / 8; ++v) {
              const int col = cb0 + v * 8;
              if (col + 8 <= rows_b) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
                if (bias) {
                  float b[8];
                  unpack8<T>(*reinterpret_cast<const uint4*>(bias + col), b);
#pragma unroll
                  for (int i = 0; i < 8; ++i) f[i] += b[i];
                }
                T o4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float g = to_f(from_f<T>(f[2 * i])), u = to_f(from_f<T>(f[2 * i + 1]));
                  o4[i] = from_f<T>(g / (1.f + __expf(-g)) * u);
                }
                *reinterpret_cast<uint2*>(dst + v * 4) = *reinterpret_cast<const uint2*>(o4);
              }
            }
          } else if (ra < rows_a) {
            T* dst = C + (size_t)ra * ldc + cb0;
            const T* res = residual ? residual + (size_t)ra * ldr + cb0 : nullptr;
#pragma unroll
            for (int v = 0; v < CH / 8; ++v) {
              const int col = cb0 + v * 8;
              if (col + 8 <= rows_b) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
                if (bias) {
                  float b[8];
                  unpack8<T>(*reinterpret_cast<const uint4*>(bias + col), b);
#pragma unroll
                  for (int i = 0; i < 8; ++i) f[i] += b[i];
                }
                if (res) {
                  float b[8];
                  unpack8<T>(*reinterpret_cast<const uint4*>(res + v * 8), b);
#pragma unroll
                  for (int i = 0; i < 8; ++i) f[i] += b[i];
                }
                *reinterpret_cast<uint4*>(dst + v * 8) = pack8<T>(f);
              } else {
                for (int i = 0; i < 8; ++i) {
                  if (col + i < rows_b) {
                    float f = __uint_as_float(r[v * 8 + i]);
                    if (bias) f += to_f(bias[col + i]);
                    if (res) f += to_f(res[v * 8 + i]);
                    dst[v * 8 + i] = from_f<T>(f);
                  }
                }
              }
            }
          }
        } else {
          // row = output feature (ra), columns = tokens cb0..cb0+CH; C is [tokens, features]
          const float bv = (bias && ra < rows_a) ? to_f(bias[ra]) : 0.f;
          if (epi == 1) {
            // lanes hold interleaved (gate, up) features: even lane = gate, odd lane = up
#pragma unroll
            for (int i = 0; i < CH; ++i) {
              const int tok = cb0 + i;
              const float g = to_f(from_f<T>(__uint_as_float(r[i]) + bv));
              const float u = __shfl_down_sync(0xffffffffu, g, 1);
              if ((lane & 1) == 0 && ra < rows_a && tok < rows_b)
                C[(size_t)tok * ldc + (ra >> 1)] = from_f<T>(g / (1.f + __expf(-g)) * u);
            }
          } else if (ra < rows_a) {
#pragma unroll
            for (int i = 0; i < CH; ++i) {
              const int tok = cb0 + i;
              if (tok < rows_b) {
                float f = __uint_as_float(r[i]) + bv;
                if (residual) f += to_f(residual[(size_t)tok * ldr + ra]);
                C[(size_t)tok * ldc + ra] = from_f<T>(f);
              }
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

// ------------------------------------------------------------------ host side
static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <typename T, int BN, int STAGES, bool SWAP>
static void launch_cfg(const void* a_op, int rows_a, int lda, const void* b_op, int rows_b, int ldb, void* C,
                       const void* bias, const void* residual, int K, int ldc, int ldr, int epi, cudaStream_t stream,
                       StatusWord* status) {
  using L = GemmSmemLayout<BN, STAGES>;
  static_assert(L::kDynSmem <= 232448, "shared memory budget exceeded");
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA = make_tmap_2d(a_op, dt, 2, rows_a, K, lda, kBM, kBK);
  CUtensorMap tmB = make_tmap_2d(b_op, dt, 2, rows_b, K, ldb, BN, kBK);
  auto kern = gemm_tn_kernel<T, BN, STAGES, SWAP>;
  // a per-device attribute of the kernel: set on every launch (cheap) rather than once per process
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynSmem);
  const int tiles = ceil_div(rows_a, kBM) * ceil_div(rows_b, BN);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  kern<<<grid, 192, L::kDynSmem, stream>>>(tmA, tmB, reinterpret_cast<T*>(C), reinterpret_cast<const T*>(bias),
                                           reinterpret_cast<const T*>(residual), rows_a, rows_b, K, ldc, ldr, epi, status);
}

template <typename T>
static void gemm_dispatch(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N,
                          int K, int lda, int ldw, int ldc, int ldr, int epi, cudaStream_t stream, StatusWord* status,
                          int force_bn) {
  const int sms = num_sms();
  if (M <= 64 && force_bn <= 0 || force_bn < 0) {
    // swap-AB: weight rows on the 128-row MMA operand, tokens on the N operand
    const int bn = (force_bn < 0) ? -force_bn : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
    if (bn == 16)
      launch_cfg<T, 16, 8, true>(W, N, ldw, A, M, lda, C, bias, residual, K, ldc, ldr, epi, stream, status);
    else if (bn == 32)
      launch_cfg<T, 32, 8, true>(W, N, ldw, A, M, lda, C, bias, residual, K, ldc, ldr, epi, stream, status);
    else
      launch_cfg<T, 64, 8, true>(W, N, ldw, A, M, lda, C, bias, residual, K, ldc, ldr, epi, stream, status);
    return;
  }
  int bn = force_bn;
  if (bn <= 0) {
    // Every N tile re-reads the whole A panel from L2, so narrow tiles only pay off while the
    // grid would otherwise leave most SMs idle; 128 is the floor once M spans a full tile.
    const int mt = ceil_div(M, kBM);
    bn = 256;
    while (bn > 128 && mt * ceil_div(N, bn) < sms) bn >>= 1;
    while (bn > 32 && mt * ceil_div(N, bn) < sms / 4) bn >>= 1;
  }
  if (bn >= 256)
    launch_cfg<T, 256, 4, false>(A, M, lda, W, N, ldw, C, bias, residual, K, ldc, ldr, epi, stream, status);
  else if (bn == 128)
    launch_cfg<T, 128, 6, false>(A, M, lda, W, N, ldw, C, bias, residual, K, ldc, ldr, epi, stream, status);
  else if (bn == 64)
    launch_cfg<T, 64, 8, false>(A, M, lda, W, N, ldw, C, bias, residual, K, ldc, ldr, epi, stream, status);
  else
    launch_cfg<T, 32, 8, false>(A, M, lda, W, N, ldw, C, bias, residual, K, ldc, ldr, epi, stream, status);
}

// epi: 0 = plain, 1 = SiLU-gate epilogue over interleaved (gate, up) output features (C is [M, N/2]).
// dtype: 0 = bf16, 1 = fp16.  force_bn: 0 = heuristic, >0 = that BN without swap, <0 = swap with |BN| tokens.
void gemm_tn(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
             int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int force_bn, int epi) {
  if (M <= 0 || N <= 0) return;
  if (dtype == 0)
    gemm_dispatch<__nv_bfloat16>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, ldr, epi, stream,
                                 reinterpret_cast<StatusWord*>(status), force_bn);
  else
    gemm_dispatch<__half>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, ldr, epi, stream,
                          reinterpret_cast<StatusWord*>(status), force_bn);
}

}  // namespace b200
