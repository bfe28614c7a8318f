// Min-latency GEMM for a handful of tokens (M <= 32) against a skinny weight:
//
//     C[M, N] = A[M, K] . W[N, K]^T        (DeepSeek fused_qkv_a_proj 7168 -> 2112, router 7168/6144/3072 ->
//                                           256/384/128 experts with fp32 logits)
//
// At these sizes the op is a weight stream (a few MB) whose latency is set by how many SMs pull on it,
// so the grid is (N / 8 column groups) x (S K-splits) and the S CTAs of one column group form a
// THREAD-BLOCK CLUSTER: each CTA multiplies its K range on the tensor cores (mma.sync m16n8k16, tokens on
// the M side, both operands loaded straight from global memory with 16-byte loads under a shared
// K permutation), reduces its 4 warps through shared memory, and the cluster's rank-0 CTA sums the S
// partial tiles over distributed shared memory (DSMEM) and writes the result - no atomics, no second
// launch, no zero-fill.
// Replaces fused_a_gemm_kernel (csrc/dsv3_fused_a_gemm.cu:577-700) and the router GEMMs
// (csrc/moe/dsv3_router_gemm_*_out.cu:51, fp32_router_gemm.cu:78) of the reference.
#include <cooperative_groups.h>
#include <type_traits>
#include "common.cuh"

namespace b200 {
namespace cg = cooperative_groups;

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2], bool bf16) {
  if (bf16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// T: operand type (bf16 / fp16); OutT: float, bf16 or fp16.  MT = number of 16-token tiles (1 or 2).
template <typename T, typename OutT, int MT>
__global__ void __launch_bounds__(128)
small_gemm_kernel(OutT* __restrict__ C, const T* __restrict__ A, const T* __restrict__ W, const T* __restrict__ bias,
                  int M, int N, int K, int lda, int ldw, int ldc) {
  cg::cluster_group cluster = cg::this_cluster();
  const int splits = cluster.num_blocks();
  const int split = cluster.block_rank();
  const int n0 = blockIdx.x * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  __shared__ float part[4][MT][16][8];      // per-warp partial tiles; warp 0's slot ends up holding the CTA sum

  // K range of this CTA in 32-wide chunks, warps interleave chunks
  const int chunks = K / 32;
  const int per = (chunks + splits - 1) / splits;
  const int c0 = split * per, c1 = min(chunks, c0 + per);
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;
  const int wn = min(n0 + g, N - 1);
  const T* wrow = W + (size_t)wn * ldw + t * 8;
  const T* arow[MT][2];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    arow[m][0] = A + (size_t)min(m * 16 + g, M - 1) * lda + t * 8;
    arow[m][1] = A + (size_t)min(m * 16 + g + 8, M - 1) * lda + t * 8;
  }
#pragma unroll 2
  for (int c = c0 + warp; c < c1; c += 4) {
    const int k = c * 32;
    const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
    uint4 av[MT][2];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      av[m][0] = *reinterpret_cast<const uint4*>(arow[m][0] + k);
      av[m][1] = *reinterpret_cast<const uint4*>(arow[m][1] + k);
    }
    // thread t holds k-values [8t, 8t+8) of the chunk; the same permutation on A and W keeps the dot product
    const uint32_t b_lo[2] = {wv.x, wv.y}, b_hi[2] = {wv.z, wv.w};
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const uint32_t a_lo[4] = {av[m][0].x, av[m][1].x, av[m][0].y, av[m][1].y};
      const uint32_t a_hi[4] = {av[m][0].z, av[m][1].z, av[m][0].w, av[m][1].w};
      mma_16816(acc[m], a_lo, b_lo, kBf16);
      mma_16816(acc[m], a_hi, b_hi, kBf16);
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    part[warp][m][g][2 * t] = acc[m][0];
    part[warp][m][g][2 * t + 1] = acc[m][1];
    part[warp][m][g + 8][2 * t] = acc[m][2];
    part[warp][m][g + 8][2 * t + 1] = acc[m][3];
  }
  __syncthreads();
  float* flat = &part[0][0][0][0];
  constexpr int kTile = MT * 16 * 8;
  for (int i = threadIdx.x; i < kTile; i += blockDim.x)
    flat[i] = flat[i] + flat[kTile + i] + flat[2 * kTile + i] + flat[3 * kTile + i];
  cluster.sync();                                   // every CTA's partial tile is complete
  if (split == 0) {
    for (int i = threadIdx.x; i < kTile; i += blockDim.x) {
      float s = flat[i];
      for (int r = 1; r < splits; ++r) s += cluster.map_shared_rank(flat, r)[i];
      const int row = i / 8, col = n0 + (i & 7);
      if (row < M && col < N) {
        if (bias) s += to_f(bias[col]);
        if constexpr (sizeof(OutT) == 4) C[(size_t)row * ldc + col] = s;
        else C[(size_t)row * ldc + col] = from_f<OutT>(s);
      }
    }
  }
  cluster.sync();                                   // keep remote shared memory alive until rank 0 has read it
}

template <typename T, typename OutT, int MT>
static int launch_small(void* C, const void* A, const void* W, const void* bias, int M, int N, int K, int lda, int ldw,
                        int ldc, int splits, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + 7) / 8, splits, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = splits;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  auto kern = small_gemm_kernel<T, OutT, MT>;
  return cudaLaunchKernelEx(&cfg, kern, (OutT*)C, (const T*)A, (const T*)W, (const T*)bias, M, N, K, lda, ldw, ldc) ==
                 cudaSuccess ? 0 : 2;
}

// K-splits (= cluster size, a power of two <= 8) chosen so that the grid covers the GPU a few times over.
int small_gemm_splits(int N, int K) {
  const int groups = (N + 7) / 8;
  int s = 1;
  while (s < 8 && groups * s < 592 && K / (s * 2) >= 512) s *= 2;
  return s;
}

// M <= 32, K % 32 == 0, rows 16-byte aligned.  dtype: 0 bf16, 1 fp16; out_kind: 0 = same as input, 1 = fp32.
int small_gemm(void* C, const void* A, const void* W, const void* bias, int M, int N, int K, int lda, int ldw, int ldc,
               int dtype, int out_kind, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32 || K % 32 != 0 || lda % 8 != 0 || ldw % 8 != 0) return 1;
  const int s = small_gemm_splits(N, K);
#define SG(T, O)                                                                                          \
  (M <= 16 ? launch_small<T, O, 1>(C, A, W, bias, M, N, K, lda, ldw, ldc, s, stream)                      \
           : launch_small<T, O, 2>(C, A, W, bias, M, N, K, lda, ldw, ldc, s, stream))
  if (dtype == 0) return out_kind == 1 ? SG(__nv_bfloat16, float) : SG(__nv_bfloat16, __nv_bfloat16);
  return out_kind == 1 ? SG(__half, float) : SG(__half, __half);
#undef SG
}

}  // namespace b200
