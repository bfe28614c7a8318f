// Second half of the tensor-parallel row-parallel linear: the GEMM before it (gemm_pair_tcgen05.cu for prefill
// chunks, gemm_streamk_tcgen05.cu for decode batches) has already pushed every output row, tile by tile while it was
// still multiplying, into the receive slot of the rank that owns the row.  This kernel is everything that
// follows, in ONE launch per rank and with no library collective:
//
//   wait     flag1[me][s] == epoch for every source s: s's rows have landed (bounded)
//   reduce   my rows: sum of the tp partial rows in rank order (bit-identical on every rank whoever computes it),
//            + my shard of the residual stream -> new residual (kept sharded by rows between calls)
//   norm     RMSNorm of the row
//   gather   the normalised row is stored into EVERY rank's output buffer: one multimem.st per 16 bytes when the
//            buffers are mapped as an NVLink multicast object (the switch replicates it: 1/tp of the bytes leave
//            the GPU), else one peer store per rank
//   close    the last CTA raises flag2[d][me] on every rank d and waits (bounded) for flag2[me][o] of every owner
//            o, so when the kernel has finished on a rank, that rank's output buffer is complete and every peer
//            has finished reading the receive slots of this call.
//
// i.e. reduce-scatter -> +residual -> RMSNorm -> all-gather around the partial rows, replacing all-reduce +
// fused_add_rms_norm (the reference's tensor_model_parallel_all_reduce after every o_proj / down_proj,
// vllm_metax/models/deepseek_v2.py:1026-1033, followed by csrc/layernorm_kernels.cu:100, and its fused special
// case csrc/minimax_reduce_rms_kernel.cu:237-320).  Per GPU 2 (tp-1)/tp payloads cross NVLink, half of them inside
// the GEMM.  Epochs live in device memory so that CUDA-graph replays advance them.
#include "comm_fused.cuh"
#include "ops.h"

namespace b200 {

// One 16-byte store that the NVSwitch replicates into every rank's copy of a multicast-mapped buffer.
__device__ __forceinline__ void multimem_st_u4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// every source's pushes for this call have landed (bounded); returns false after a timeout
__device__ __forceinline__ bool arn_wait_pushes(const ArNormParams& p, uint32_t epoch, int* s_ok) {
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.tp) {
    uint32_t seen = 0;
    if (!wait_flag_ge(p.flag1[p.rank] + threadIdx.x, epoch, p.wait_cycles, &seen)) {
      report_status(p.status, kWaitTimeout, 180, (int)epoch, (int)seen);
      *s_ok = 0;
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

// close: the last CTA publishes "my rows are in your output buffer" and waits for every owner's
__device__ __forceinline__ void arn_close(const ArNormParams& p, uint32_t epoch, int* s_ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t ticket = atomicAdd(&p.local_sync[2], 1u);
    *s_ok = (ticket == gridDim.x - 1) ? 2 : 0;
  }
  __syncthreads();
  if (*s_ok == 2) {
    if ((int)threadIdx.x < p.tp) {
      __threadfence_system();
      st_release_sys(p.flag2[threadIdx.x] + p.rank, epoch);
      uint32_t seen = 0;
      if (!wait_flag_ge(p.flag2[p.rank] + threadIdx.x, epoch, p.wait_cycles, &seen))
        report_status(p.status, kWaitTimeout, 181, (int)epoch, (int)seen);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      p.local_sync[2] = 0;
      p.local_sync[3] = epoch;
    }
  }
}

// General widths: the summed row is staged in shared memory between the two passes.
template <typename T>
__global__ void __launch_bounds__(256)
ar_norm_gather_kernel(const ArNormParams p) {
  extern __shared__ __align__(16) uint8_t smem_row[];
  __shared__ float red[32];
  __shared__ int s_ok;
  T* row = reinterpret_cast<T*>(smem_row);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 3) + 1u;
  const int my_rows = max(0, min(p.rows_per_rank, p.T - p.rank * p.rows_per_rank));
  const int nvec = p.H >> 3;
  const bool ok = arn_wait_pushes(p, epoch, &s_ok);

  const char* mine = static_cast<const char*>(p.recv[p.rank]);
  const size_t slot_bytes = (size_t)p.rows_cap * p.H * sizeof(T);
  for (int r = blockIdx.x; r < my_rows && ok; r += gridDim.x) {
    const size_t row_off = (size_t)r * p.H * sizeof(T);
    uint4* res = reinterpret_cast<uint4*>(static_cast<T*>(p.residual) + (size_t)r * p.H);
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < p.tp; ++s) {
        float f[8];
        unpack8<T>(__ldcg(reinterpret_cast<const uint4*>(mine + s * slot_bytes + row_off) + v), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      if (p.add_residual) {
        float f[8];
        unpack8<T>(res[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      const uint4 packed = pack8<T>(acc);
      res[v] = packed;
      reinterpret_cast<uint4*>(row)[v] = packed;
      unpack8<T>(packed, acc);                       // the norm sees the rounded residual
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += acc[i] * acc[i];
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)p.H + p.eps);
    const size_t grow = (size_t)(p.rank * p.rows_per_rank + r) * p.H;   // element offset of the row in `out`
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8], w[8];
      unpack8<T>(reinterpret_cast<const uint4*>(row)[v], f);
      unpack8<T>(reinterpret_cast<const uint4*>(p.norm_weight)[v], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * w[i];
      const uint4 y = pack8<T>(f);
      if (p.out_mc) {
        multimem_st_u4(reinterpret_cast<uint4*>(static_cast<T*>(p.out_mc) + grow) + v, y);
      } else {
        for (int d = 0; d < p.tp; ++d) {
          const int dst = (p.rank + d) % p.tp;       // start with the local copy, spread the peers
          reinterpret_cast<uint4*>(static_cast<T*>(p.out[dst]) + grow)[v] = y;
        }
      }
    }
    __syncthreads();                                 // `row` and `red` are rewritten by the next row
  }
  arn_close(p, epoch, &s_ok);
}

// Rows of 128 * VPT vectors (H = 1024 * VPT): 128 threads per row, every load of the row - all sources and the
// residual - in flight before the first use, the summed row kept in registers between the two passes.
template <typename T, int VPT>
__global__ void __launch_bounds__(128)
ar_norm_gather_reg_kernel(const ArNormParams p) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 3) + 1u;
  const int my_rows = max(0, min(p.rows_per_rank, p.T - p.rank * p.rows_per_rank));
  const bool ok = arn_wait_pushes(p, epoch, &s_ok);

  const char* mine = static_cast<const char*>(p.recv[p.rank]);
  const size_t slot_bytes = (size_t)p.rows_cap * p.H * sizeof(T);
  for (int r = blockIdx.x; r < my_rows && ok; r += gridDim.x) {
    const size_t row_off = (size_t)r * p.H * sizeof(T);
    uint4* res = reinterpret_cast<uint4*>(static_cast<T*>(p.residual) + (size_t)r * p.H);
    uint4 part[kMaxRanks][VPT], rv[VPT];
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s)
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        part[s][i] = s < p.tp ? __ldcg(reinterpret_cast<const uint4*>(mine + s * slot_bytes + row_off) + threadIdx.x + i * 128)
                              : make_uint4(0, 0, 0, 0);
    if (p.add_residual) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) rv[i] = res[threadIdx.x + i * 128];
    }
    float f[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[i][e] = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < p.tp) {                              // rank order: the same bits whoever owns the row
          float g[8];
          unpack8<T>(part[s][i], g);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[i][e] += g[e];
        }
      }
      if (p.add_residual) {
        float g[8];
        unpack8<T>(rv[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[i][e] += g[e];
      }
      const uint4 packed = pack8<T>(f[i]);
      res[threadIdx.x + i * 128] = packed;
      unpack8<T>(packed, f[i]);                      // the norm sees the rounded residual
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[i][e] * f[i][e];
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)p.H + p.eps);
    const size_t grow = (size_t)(p.rank * p.rows_per_rank + r) * p.H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float w[8];
      unpack8<T>(reinterpret_cast<const uint4*>(p.norm_weight)[threadIdx.x + i * 128], w);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[i][e] = f[i][e] * inv * w[e];
      const uint4 y = pack8<T>(f[i]);
      if (p.out_mc) {
        multimem_st_u4(reinterpret_cast<uint4*>(static_cast<T*>(p.out_mc) + grow) + threadIdx.x + i * 128, y);
      } else {
        for (int d = 0; d < p.tp; ++d) {
          const int dst = (p.rank + d) % p.tp;
          reinterpret_cast<uint4*>(static_cast<T*>(p.out[dst]) + grow)[threadIdx.x + i * 128] = y;
        }
      }
    }
  }
  arn_close(p, epoch, &s_ok);
}

// Returns 0, -1 (H not a multiple of 8 / too wide for the row stage), -2 (bad dtype).
int ar_norm_gather(const ArNormParams& p, int dtype, cudaStream_t stream) {
  if (p.T <= 0) return 0;
  if ((p.H & 7) != 0 || (size_t)p.H * 2 > 96 * 1024) return -1;
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -1;
  if (sms[dev] == 0) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  const int my_rows_max = p.rows_per_rank;
  int grid = my_rows_max < 8 * sms[dev] ? my_rows_max : 8 * sms[dev];
  grid = grid < 1 ? 1 : grid;
  const size_t sm = (size_t)p.H * 2;
  const int vpt = p.H % 1024 == 0 ? p.H / 1024 : 0;
#define B200_ARN(T)                                                                                               \
  do {                                                                                                            \
    if (vpt == 1) ar_norm_gather_reg_kernel<T, 1><<<grid, 128, 0, stream>>>(p);                                   \
    else if (vpt == 2) ar_norm_gather_reg_kernel<T, 2><<<grid, 128, 0, stream>>>(p);                              \
    else if (vpt == 4) ar_norm_gather_reg_kernel<T, 4><<<grid, 128, 0, stream>>>(p);                              \
    else {                                                                                                        \
      if (sm > 48 * 1024)                                                                                         \
        cudaFuncSetAttribute(ar_norm_gather_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);     \
      ar_norm_gather_kernel<T><<<grid, 256, sm, stream>>>(p);                                                     \
    }                                                                                                             \
  } while (0)
  if (dtype == 0) B200_ARN(__nv_bfloat16);
  else if (dtype == 1) B200_ARN(__half);
  else return -2;
#undef B200_ARN
  return 0;
}

}  // namespace b200
