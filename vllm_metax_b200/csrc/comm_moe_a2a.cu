// Expert-parallel all-to-all over NVLink peer memory: dispatch (+ optional fp8 1x128 quantisation)
// and combine (+ sum over ranks), written as plain peer stores into symmetric buffers.
//
// A token crosses NVLink ONCE per destination rank, however many of its top-k experts live there, and one
// partial sum per (token, rank) comes back - top-k / ranks-hit times less traffic than one row per (token, expert).
//
//   dispatch       one warp per (token, destination rank): if any of the token's experts is on that rank the row
//                  is pushed to recv_x[dst][rank*cap + slot] together with its top-k list rewritten for the
//                  destination (local expert id or -1) and the weights, i.e. exactly the input of the local
//                  fused-MoE path.  Slots come from a local per-destination counter, so no remote atomics.
//                  The last CTA publishes the counts, raises this rank's flag on every destination
//                  (st.release.sys) and waits - bounded - for the flags of all sources, so when the
//                  kernel ends the receive buffers of this step are complete.
//   combine_send   the weighted partial sum of every received token travels back to comb_x[src][rank][t];
//                  consumed receive slots are reset to "empty"; the last CTA raises the combine flags.
//   combine_reduce waits (bounded) for the flags of all ranks, then out[t] = sum over the ranks that own one of
//                  t's experts of comb_x[r][t] (+ shared-expert output).
// No kernel waits on a CTA of its own grid that may not be resident: the only cross-CTA dependency is
// the "last CTA" ticket.  A wait that runs out records the site in the status word and the kernel
// returns; the host raises.  Epochs live in device memory so CUDA-graph replays advance them.
// Replaces deep_ep low_latency_dispatch / low_latency_combine and the all-gather / reduce-scatter
// manager (vllm_metax/distributed/device_communicators/all2all.py:20-218,
// model_executor/layers/fused_moe/prepare_finalize/deepep_ll.py:24-145).
#include "comm_fused.cuh"

namespace b200 {

// Bit r set when one of the token's experts lives on rank r (lanes >= topk contribute nothing).
__device__ __forceinline__ uint32_t rank_mask(const int* ids, int topk, int experts_per_rank, int ep, int lane) {
  uint32_t m = 0;
  for (int k = lane; k < topk; k += 32) {
    const int e = ids[k];
    if (e >= 0 && e / experts_per_rank < ep) m |= 1u << (e / experts_per_rank);
  }
  return __reduce_or_sync(0xffffffffu, m);
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_a2a_dispatch_kernel(const MoeA2aParams p, const T* __restrict__ x, const int* __restrict__ topk_ids,
                        const float* __restrict__ topk_w) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  const int total_warps = gridDim.x * warps_per_cta;
  uint32_t* send_count = p.local_sync + 8;
  const int nvec = p.H >> 3;

  for (int item = gw; item < p.T * p.ep; item += total_warps) {
    const int t = item / p.ep, dst = (item % p.ep + p.rank) % p.ep;    // ranks start on different destinations
    const int* ids = topk_ids + (size_t)t * p.topk;
    if (!((rank_mask(ids, p.topk, p.experts_per_rank, p.ep, lane) >> dst) & 1u)) continue;
    int slot = 0;
    if (lane == 0) slot = (int)atomicAdd(&send_count[dst], 1u);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= p.cap) {
      if (lane == 0) report_status(p.status, kWaitTimeout, 140, slot, p.cap);   // receive region overflow
      continue;
    }
    const size_t idx = (size_t)p.rank * p.cap + slot;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * p.H);
    if (!p.quant) {
      uint4* dstrow = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.recv_x[dst]) + idx * p.H);
      for (int v0 = 0; v0 < nvec; v0 += 128) {               // four loads in flight per lane before the stores
        uint4 r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (v0 + j * 32 + lane < nvec) r[j] = src[v0 + j * 32 + lane];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (v0 + j * 32 + lane < nvec) dstrow[v0 + j * 32 + lane] = r[j];
      }
    } else {
      uint2* dstrow = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(p.recv_x[dst]) + idx * p.H);
      float* sc = p.recv_scale[dst] + idx * (p.H >> 7);
      for (int v0 = 0; v0 < nvec; v0 += 32) {           // 16 lanes x 8 elements = one 128-wide group
        const int v = v0 + lane;
        float f[8];
        float m = 0.f;
        if (v < nvec) {
          unpack8<T>(src[v], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(f[i]));
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float s = fmaxf(m, 1e-10f) / 448.f;
        if (v < nvec) {
          const float inv = 1.f / s;
          uint32_t lo = 0, hi = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) lo |= (uint32_t)float_to_fp8_e4m3(f[i] * inv) << (8 * i);
#pragma unroll
          for (int i = 0; i < 4; ++i) hi |= (uint32_t)float_to_fp8_e4m3(f[4 + i] * inv) << (8 * i);
          dstrow[v] = make_uint2(lo, hi);
          if ((lane & 15) == 0) sc[v >> 4] = s;
        }
      }
    }
    for (int k = lane; k < p.topk; k += 32) {              // the token's top-k list as the destination sees it
      const int e = ids[k];
      const bool here = e >= 0 && e / p.experts_per_rank == dst;
      p.recv_ids[dst][idx * p.topk + k] = here ? e - dst * p.experts_per_rank : -1;
      p.recv_w[dst][idx * p.topk + k] = here ? topk_w[(size_t)t * p.topk + k] : 0.f;
    }
    if (lane == 0) p.recv_src[dst][idx] = t;
  }

  // ---- completion: the last CTA publishes counts + flags, then waits for every source
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t ticket = atomicAdd(&p.local_sync[0], 1u);
    is_last = ticket == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  const uint32_t epoch = p.local_sync[1] + 1;
  if ((int)threadIdx.x < p.ep) {
    const int r = threadIdx.x;
    const uint32_t cnt = *reinterpret_cast<volatile uint32_t*>(&send_count[r]);
    p.recv_count[r][p.rank] = cnt < (uint32_t)p.cap ? cnt : (uint32_t)p.cap;
    st_release_sys(&p.disp_flag[r][p.rank], epoch);
    send_count[r] = 0;
    uint32_t seen = 0;
    if (!wait_flag_ge(&p.disp_flag[p.rank][r], epoch, p.wait_cycles, &seen))
      report_status(p.status, kWaitTimeout, 141, epoch, seen);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    p.local_sync[0] = 0;
    p.local_sync[1] = epoch;
  }
}

// y [ep*cap, H]: partial sums of the received tokens (row = receive slot).
template <typename T>
__global__ void __launch_bounds__(256)
moe_a2a_combine_send_kernel(const MoeA2aParams p, const T* __restrict__ y) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  const int total_warps = gridDim.x * warps_per_cta;
  const int nvec = p.H >> 3;
  const int slots = p.ep * p.cap;
  for (int i = gw; i < slots; i += total_warps) {
    const int src = i / p.cap;
    if ((uint32_t)(i - src * p.cap) >= p.recv_count[p.rank][src]) continue;
    const int t = p.recv_src[p.rank][i];
    const uint4* s = reinterpret_cast<const uint4*>(y + (size_t)i * p.H);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.comb_x[src]) + ((size_t)p.rank * p.cap + t) * p.H);
    for (int v0 = 0; v0 < nvec; v0 += 128) {
      uint4 r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v0 + j * 32 + lane < nvec) r[j] = s[v0 + j * 32 + lane];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v0 + j * 32 + lane < nvec) d[v0 + j * 32 + lane] = r[j];
    }
    for (int k = lane; k < p.topk; k += 32) p.recv_ids[p.rank][(size_t)i * p.topk + k] = -1;   // slot is free again
  }
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t ticket = atomicAdd(&p.local_sync[0], 1u);
    is_last = ticket == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  const uint32_t epoch = p.local_sync[2] + 1;
  if ((int)threadIdx.x < p.ep) st_release_sys(&p.comb_flag[threadIdx.x][p.rank], epoch);
  __syncthreads();
  if (threadIdx.x == 0) {
    p.local_sync[0] = 0;
    p.local_sync[2] = epoch;
  }
}

// Runs after combine_send in stream order, so local_sync[2] already holds this step's epoch.
template <typename T>
__global__ void __launch_bounds__(256)
moe_a2a_combine_reduce_kernel(const MoeA2aParams p, T* __restrict__ out, const int* __restrict__ topk_ids,
                              const T* __restrict__ shared_out) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  const uint32_t epoch = p.local_sync[2];
  if ((int)threadIdx.x < p.ep) {
    uint32_t seen = 0;
    if (!wait_flag_ge(&p.comb_flag[p.rank][threadIdx.x], epoch, p.wait_cycles, &seen)) {
      report_status(p.status, kWaitTimeout, 142, epoch, seen);
      ok = 0;
    }
  }
  __syncthreads();
  if (!ok) return;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  const int total_warps = gridDim.x * warps_per_cta;
  const int nvec = p.H >> 3;
  const T* cx = reinterpret_cast<const T*>(p.comb_x[p.rank]);
  for (int t = gw; t < p.T; t += total_warps) {
    const uint32_t mask = rank_mask(topk_ids + (size_t)t * p.topk, p.topk, p.experts_per_rank, p.ep, lane);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8];
      if (shared_out) {
        unpack8<T>(reinterpret_cast<const uint4*>(shared_out + (size_t)t * p.H)[v], acc);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      }
      for (int r = 0; r < p.ep; ++r) {
        if (!((mask >> r) & 1u)) continue;
        float f[8];
        unpack8<T>(__ldcg(reinterpret_cast<const uint4*>(cx + ((size_t)r * p.cap + t) * p.H) + v), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      reinterpret_cast<uint4*>(out + (size_t)t * p.H)[v] = pack8<T>(acc);
    }
  }
}

// Gather rows of `row_bytes` (multiple of 16) bytes: dst[i] = src[idx[i] / div] for i < *count; idx outside
// [0, limit * div) -> zeros.
__global__ void gather_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, const int* __restrict__ idx,
                                   const int* __restrict__ count, int limit, int row_vec, int div) {
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int total_warps = (gridDim.x * blockDim.x) >> 5;
  const int n = *count;
  for (int i = gw; i < n; i += total_warps) {
    const int s = idx[i] >= 0 ? idx[i] / div : -1;
    for (int v = lane; v < row_vec; v += 32)
      dst[(size_t)i * row_vec + v] = (s >= 0 && s < limit) ? src[(size_t)s * row_vec + v] : make_uint4(0, 0, 0, 0);
  }
}

static int a2a_grid(int work_warps) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  int g = (work_warps + 7) / 8;
  g = g < 1 ? 1 : g;
  return g > 2 * sms ? 2 * sms : g;
}

void moe_a2a_dispatch(const MoeA2aParams& p, const void* x, const int* topk_ids, const float* topk_w, int dtype,
                      cudaStream_t stream) {
  const int grid = a2a_grid(p.T * p.ep);
  if (dtype == 0)
    moe_a2a_dispatch_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p, (const __nv_bfloat16*)x, topk_ids, topk_w);
  else
    moe_a2a_dispatch_kernel<__half><<<grid, 256, 0, stream>>>(p, (const __half*)x, topk_ids, topk_w);
}

void moe_a2a_combine(const MoeA2aParams& p, const void* y, void* out, const int* topk_ids, const void* shared_out,
                     int dtype, cudaStream_t stream) {
  const int g1 = a2a_grid(p.ep * p.cap), g2 = a2a_grid(p.T);
  if (dtype == 0) {
    moe_a2a_combine_send_kernel<__nv_bfloat16><<<g1, 256, 0, stream>>>(p, (const __nv_bfloat16*)y);
    moe_a2a_combine_reduce_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>(p, (__nv_bfloat16*)out, topk_ids,
                                                                        (const __nv_bfloat16*)shared_out);
  } else {
    moe_a2a_combine_send_kernel<__half><<<g1, 256, 0, stream>>>(p, (const __half*)y);
    moe_a2a_combine_reduce_kernel<__half><<<g2, 256, 0, stream>>>(p, (__half*)out, topk_ids, (const __half*)shared_out);
  }
}

void gather_rows(void* dst, const void* src, const int* idx, const int* count, int max_rows, int limit, int row_bytes,
                 int div, cudaStream_t stream) {
  if (max_rows <= 0) return;
  gather_rows_kernel<<<a2a_grid(max_rows), 256, 0, stream>>>((uint4*)dst, (const uint4*)src, idx, count, limit,
                                                             row_bytes / 16, div < 1 ? 1 : div);
}

}  // namespace b200
