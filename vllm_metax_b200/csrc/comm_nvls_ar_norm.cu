// All-reduce + residual + RMSNorm of a row-parallel linear's partial sums through the NVSwitch (NVLS), one launch
// per rank, for the step sizes where latency and not bandwidth sets the time (decode batches).
//
// The GEMM before it is an ordinary local GEMM whose output buffer, `partial [T, H]`, lives in symmetric memory that
// all ranks have bound to ONE NVLink multicast address.  This kernel then is
//
//   arrive    multimem.red.add on the multicast flag word: one instruction raises the counter on every rank
//   wait      every CTA polls its LOCAL copy of the counter until all tp ranks of this call arrived (bounded)
//   reduce    for the rows this rank owns: multimem.ld_reduce - the switch fetches the 16 bytes from all tp copies
//             and adds them (fp32 accumulation) on the way; + this rank's shard of the residual -> new residual
//   norm      RMSNorm of the row
//   gather    multimem.st of the normalised row: the switch writes it into every rank's output buffer
//   close     last CTA: multimem.red.add on the second flag word, then waits for all tp arrivals, so that when the
//             kernel has finished on a rank its output buffer is complete and nobody still reads its partial sums.
//
// Against the peer-store path (comm_ar_norm.cu after a scatter GEMM) the reduction costs one switch round trip
// instead of tp - 1 pushed copies per row, the GEMM runs its plain local epilogue, and both barriers are one
// instruction each.  It replaces tensor_model_parallel_all_reduce + fused_add_rms_norm of the reference
// (vllm_metax/models/deepseek_v2.py:1026-1033 + csrc/layernorm_kernels.cu:100).  Counters only grow (call n waits for
// n * tp); the call number lives in device memory so that CUDA-graph replays advance it.
#include "comm_fused.cuh"
#include "ops.h"

namespace b200 {

__device__ __forceinline__ void multimem_red_add_u32(uint32_t* mc_addr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}

template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce_16(const void* mc_addr);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_16<__nv_bfloat16>(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_16<__half>(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

__device__ __forceinline__ void nvls_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// arrive (once per rank: the GEMM that filled `partial` finished before this launch started) and wait for all ranks
__device__ __forceinline__ bool nvls_open(const NvlsArNormParams& p, uint32_t want, int* s_ok) {
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      multimem_red_add_u32(p.flag_mc + 0, 1u);
    }
    uint32_t seen = 0;
    *s_ok = 1;
    if (!wait_flag_ge(p.flag_local + 0, want, p.wait_cycles, &seen)) {
      report_status(p.status, kWaitTimeout, 190, (int)want, (int)seen);
      *s_ok = 0;
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

// last CTA: "my rows are in everybody's output buffer, and I no longer read anybody's partial sums"
__device__ __forceinline__ void nvls_close(const NvlsArNormParams& p, uint32_t call, uint32_t want, bool ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t ticket = atomicAdd(&p.local_sync[0], 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence_system();
      multimem_red_add_u32(p.flag_mc + 1, 1u);
      uint32_t seen = 0;
      if (ok && !wait_flag_ge(p.flag_local + 1, want, p.wait_cycles, &seen))
        report_status(p.status, kWaitTimeout, 191, (int)want, (int)seen);
      p.local_sync[0] = 0;
      p.local_sync[1] = call;
    }
  }
}

// Any H that is a multiple of 8: vectors of a row are taken 128 at a time.
template <typename T>
__global__ void __launch_bounds__(128)
nvls_ar_norm_kernel(const NvlsArNormParams p) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 1) + 1u;
  const uint32_t want = call * (uint32_t)p.tp;
  const int my_rows = max(0, min(p.rows_per_rank, p.T - p.rank * p.rows_per_rank));
  const int nvec = p.H >> 3;
  const bool ok = nvls_open(p, want, &s_ok);

  for (int r = blockIdx.x; r < my_rows && ok; r += gridDim.x) {
    const size_t grow = (size_t)(p.rank * p.rows_per_rank + r) * p.H;       // element offset of the row
    const T* part = static_cast<const T*>(p.partial_mc) + grow;
    uint4* res = reinterpret_cast<uint4*>(static_cast<T*>(p.residual) + (size_t)r * p.H);
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8<T>(multimem_ld_reduce_16<T>(reinterpret_cast<const uint4*>(part) + v), f);
      if (p.add_residual) {
        float g[8];
        unpack8<T>(res[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
      }
      const uint4 packed = pack8<T>(f);
      res[v] = packed;
      unpack8<T>(packed, f);                          // the norm sees the rounded residual
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)p.H + p.eps);
    T* dst = static_cast<T*>(p.out_mc) + grow;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8], w[8];
      unpack8<T>(res[v], f);                          // written by this same thread above
      unpack8<T>(reinterpret_cast<const uint4*>(p.norm_weight)[v], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * w[i];
      nvls_st_16(reinterpret_cast<uint4*>(dst) + v, pack8<T>(f));
    }
    __syncthreads();                                  // `red` is reused by the next row
  }
  nvls_close(p, call, want, ok);
}

// H = 1024 * VPT: every switch round trip of the row (and the residual loads) is in flight before the first use, and
// the row stays in registers between the two passes.
template <typename T, int VPT>
__global__ void __launch_bounds__(128)
nvls_ar_norm_reg_kernel(const NvlsArNormParams p) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 1) + 1u;
  const uint32_t want = call * (uint32_t)p.tp;
  const int my_rows = max(0, min(p.rows_per_rank, p.T - p.rank * p.rows_per_rank));
  const bool ok = nvls_open(p, want, &s_ok);

  for (int r = blockIdx.x; r < my_rows && ok; r += gridDim.x) {
    const size_t grow = (size_t)(p.rank * p.rows_per_rank + r) * p.H;
    const uint4* part = reinterpret_cast<const uint4*>(static_cast<const T*>(p.partial_mc) + grow);
    uint4* res = reinterpret_cast<uint4*>(static_cast<T*>(p.residual) + (size_t)r * p.H);
    uint4 sum[VPT], rv[VPT], wv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) sum[i] = multimem_ld_reduce_16<T>(part + threadIdx.x + i * 128);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      rv[i] = p.add_residual ? res[threadIdx.x + i * 128] : make_uint4(0, 0, 0, 0);
      wv[i] = reinterpret_cast<const uint4*>(p.norm_weight)[threadIdx.x + i * 128];
    }
    float f[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      unpack8<T>(sum[i], f[i]);
      if (p.add_residual) {
        float g[8];
        unpack8<T>(rv[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[i][e] += g[e];
      }
      const uint4 packed = pack8<T>(f[i]);
      res[threadIdx.x + i * 128] = packed;
      unpack8<T>(packed, f[i]);                       // the norm sees the rounded residual
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[i][e] * f[i][e];
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)p.H + p.eps);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.out_mc) + grow);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float w[8];
      unpack8<T>(wv[i], w);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[i][e] = f[i][e] * inv * w[e];
      nvls_st_16(dst + threadIdx.x + i * 128, pack8<T>(f[i]));
    }
  }
  nvls_close(p, call, want, ok);
}

// Returns 0, -1 (H not a multiple of 8), -2 (bad dtype).
int nvls_ar_norm(const NvlsArNormParams& p, int dtype, cudaStream_t stream) {
  if (p.T <= 0) return 0;
  if ((p.H & 7) != 0) return -1;
  int grid = p.rows_per_rank < 1 ? 1 : p.rows_per_rank;
  if (grid > 1184) grid = 1184;                       // 8 CTAs of 128 threads on each of 148 SMs
  const int vpt = p.H % 1024 == 0 ? p.H / 1024 : 0;
#define B200_NVLS(T)                                                                      \
  do {                                                                                    \
    if (vpt == 1) nvls_ar_norm_reg_kernel<T, 1><<<grid, 128, 0, stream>>>(p);             \
    else if (vpt == 2) nvls_ar_norm_reg_kernel<T, 2><<<grid, 128, 0, stream>>>(p);        \
    else if (vpt == 4) nvls_ar_norm_reg_kernel<T, 4><<<grid, 128, 0, stream>>>(p);        \
    else if (vpt == 8) nvls_ar_norm_reg_kernel<T, 8><<<grid, 128, 0, stream>>>(p);        \
    else nvls_ar_norm_kernel<T><<<grid, 128, 0, stream>>>(p);                             \
  } while (0)
  if (dtype == 0) B200_NVLS(__nv_bfloat16);
  else if (dtype == 1) B200_NVLS(__half);
  else return -2;
#undef B200_NVLS
  return 0;
}

}  // namespace b200
