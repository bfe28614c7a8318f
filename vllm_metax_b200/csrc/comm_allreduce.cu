// Stand-alone collectives over NVLink peer memory for the places where no GEMM precedes the reduction
// (MoE outputs, logits pieces, small decode messages) and the cross-rank RMSNorm of a split hidden dimension.
//
//   allreduce one-shot   CTA b pushes chunk b of its input into EVERY rank's receive slot, raises flag1[dst][rank][b],
//                        waits (bounded) for chunk b of every source and sums the tp slots in rank order, so all
//                        ranks get bit-identical results.  One NVLink crossing, tp-1 copies of the payload: the
//                        latency path for small messages.
//   allreduce two-shot   the payload is cut into tp segments.  CTA b pushes sub-chunk b of segment d to owner d,
//                        the owner sums and writes the reduced sub-chunk into every rank's gather buffer
//                        (flag2), every rank copies the gathered result out.  2 (tp-1)/tp payloads per rank.
//   reduce_rms           y = x * rsqrt(sum_over_ranks(sum x^2) / (H_local * tp) + eps) * w for one or two tensors
//                        (q and k).  The per-token partial sums are written straight into every peer's slot array;
//                        a slot holding -0.0 has not been written yet, so the value is its own flag and a token
//                        costs one 4-byte store per peer.  Three slot arrays rotate: call n uses n % 3 and clears
//                        the one call n - 1 used, which no peer touches again before call n + 2.
//
// Chunk b of every rank is handled by CTA b of that rank, so the only waits are on peers, never on a CTA of
// the same grid.  Receive buffers alternate by call parity: a rank can enter call n + 2 only after every peer
// has pushed for call n + 1, i.e. after the peer finished reading call n's slots.  Every wait is bounded and
// reports {site, expected, observed} through the status word.
// Covers the reference's quick all-reduce (csrc/quickreduce/quick_reduce_impl.cuh:540-694, without the integer
// wire codecs) and its Lamport reduce-RMS kernels (csrc/minimax_reduce_rms_kernel.cu:237-599).
#include "comm_fused.cuh"

namespace b200 {

__device__ __forceinline__ uint4 ld_cg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

template <typename T>
__device__ __forceinline__ void acc_add(float (&acc)[8], const uint4& raw) {
  float f[8];
  unpack8<T>(raw, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] += f[i];
}
// fp32 payloads: a 16-byte vector is four floats
struct F32Tag {};
template <>
__device__ __forceinline__ void acc_add<F32Tag>(float (&acc)[8], const uint4& raw) {
  acc[0] += __uint_as_float(raw.x);
  acc[1] += __uint_as_float(raw.y);
  acc[2] += __uint_as_float(raw.z);
  acc[3] += __uint_as_float(raw.w);
}
template <typename T>
__device__ __forceinline__ uint4 acc_pack(const float (&acc)[8]) { return pack8<T>(acc); }
template <>
__device__ __forceinline__ uint4 acc_pack<F32Tag>(const float (&acc)[8]) {
  return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
}

// Raise this CTA's flag on every rank (after all threads' peer stores), then wait for the same CTA of every source.
__device__ __forceinline__ bool flag_exchange(uint32_t* const* flags, const CustomArParams& p, uint32_t epoch, int site) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok = 1;
    __threadfence_system();
  }
  __syncthreads();
  if ((int)threadIdx.x < p.tp) {
    const int r = threadIdx.x;
    st_release_sys(flags[r] + (size_t)p.rank * p.max_ctas + blockIdx.x, epoch);
    uint32_t seen = 0;
    if (!wait_flag_ge(flags[p.rank] + (size_t)r * p.max_ctas + blockIdx.x, epoch, p.wait_cycles, &seen)) {
      report_status(p.status, kWaitTimeout, site, (int)epoch, (int)seen);
      s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ void close_call(const CustomArParams& p, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(&p.local_sync[0], 1u);
    if (ticket == gridDim.x - 1) {
      p.local_sync[0] = 0;
      p.local_sync[1] = epoch;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(const CustomArParams p, const uint4* __restrict__ in, uint4* __restrict__ out) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 1) + 1u;
  const size_t parity_off = (size_t)(epoch & 1u) * p.tp * p.cap_bytes;
  const long long nvec = p.n_bytes >> 4;
  const long long per = (nvec + gridDim.x - 1) / gridDim.x;
  const long long v0 = per * blockIdx.x, v1 = min(nvec, v0 + per);

  for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    const uint4 val = in[v];
    for (int d = 0; d < p.tp; ++d) {
      const int dst = (p.rank + d) % p.tp;
      reinterpret_cast<uint4*>(static_cast<char*>(p.recv[dst]) + parity_off + (size_t)p.rank * p.cap_bytes)[v] = val;
    }
  }
  const bool ok = flag_exchange(p.flag1, p, epoch, 150);
  if (ok) {
    const char* mine = static_cast<const char*>(p.recv[p.rank]) + parity_off;
    for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < p.tp; ++s) acc_add<T>(acc, ld_cg_u4(mine + (size_t)s * p.cap_bytes + (v << 4)));
      out[v] = acc_pack<T>(acc);
    }
  }
  close_call(p, epoch);
}

template <typename T>
__global__ void __launch_bounds__(512)
allreduce_twoshot_kernel(const CustomArParams p, const uint4* __restrict__ in, uint4* __restrict__ out) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 1) + 1u;
  const size_t parity = epoch & 1u;
  const size_t recv_off = parity * p.tp * p.cap_bytes, gather_off = parity * p.cap_bytes;
  const long long nvec = p.n_bytes >> 4;
  const long long seg = (nvec + p.tp - 1) / p.tp;             // vectors per segment
  const long long per = (seg + gridDim.x - 1) / gridDim.x;
  const long long s0 = per * blockIdx.x, s1 = min(seg, s0 + per);

  // scatter: sub-chunk [s0, s1) of every segment goes to the segment's owner
  for (int d = 0; d < p.tp; ++d) {
    const int dst = (p.rank + d) % p.tp;
    uint4* slot = reinterpret_cast<uint4*>(static_cast<char*>(p.recv[dst]) + recv_off + (size_t)p.rank * p.cap_bytes);
    for (long long v = s0 + threadIdx.x; v < s1; v += blockDim.x) {
      const long long gv = dst * seg + v;
      if (gv < nvec) slot[v] = in[gv];
    }
  }
  bool ok = flag_exchange(p.flag1, p, epoch, 151);
  // reduce my segment, broadcast the result
  if (ok) {
    const char* mine = static_cast<const char*>(p.recv[p.rank]) + recv_off;
    for (long long v = s0 + threadIdx.x; v < s1; v += blockDim.x) {
      const long long gv = p.rank * seg + v;
      if (gv >= nvec) continue;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < p.tp; ++s) acc_add<T>(acc, ld_cg_u4(mine + (size_t)s * p.cap_bytes + (v << 4)));
      const uint4 r = acc_pack<T>(acc);
      out[gv] = r;
      for (int d = 1; d < p.tp; ++d) {
        const int dst = (p.rank + d) % p.tp;
        reinterpret_cast<uint4*>(static_cast<char*>(p.gather[dst]) + gather_off)[gv] = r;
      }
    }
  }
  ok = flag_exchange(p.flag2, p, epoch, 152) && ok;
  if (ok) {
    const char* g = static_cast<const char*>(p.gather[p.rank]) + gather_off;
    for (int d = 1; d < p.tp; ++d) {
      const int src = (p.rank + d) % p.tp;
      for (long long v = s0 + threadIdx.x; v < s1; v += blockDim.x) {
        const long long gv = src * seg + v;
        if (gv < nvec) out[gv] = ld_cg_u4(g + (gv << 4));
      }
    }
  }
  close_call(p, epoch);
}

// mode: 0 = choose by size, 1 = one-shot, 2 = two-shot.  dtype: 0 bf16, 1 fp16, 2 fp32.
// Returns 0, -1 (payload not a multiple of 16 bytes or larger than the buffers), -2 (bad dtype).
int custom_allreduce(const CustomArParams& p, const void* in, void* out, int dtype, int mode, cudaStream_t stream) {
  if (p.n_bytes == 0) return 0;
  if ((p.n_bytes & 15) != 0 || p.n_bytes > p.cap_bytes) return -1;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // one crossing beats two while the (tp - 1)-fold payload is small; with two ranks the traffic is the same
  const long long one_shot_max = p.tp <= 2 ? (1ll << 40) : p.tp <= 4 ? (512 << 10) : (256 << 10);
  const bool one = mode == 1 || (mode == 0 && p.n_bytes <= one_shot_max);
  const long long nvec = p.n_bytes >> 4;
  const long long work = one ? nvec : (nvec + p.tp - 1) / p.tp;
  int grid = (int)((work + 1023) / 1024);                     // >= 2 vectors per thread before another CTA is added
  grid = grid < 1 ? 1 : grid;
  const int cap = p.max_ctas < sms ? p.max_ctas : sms;         // all CTAs resident: peers wait on CTA b, not on a queue
  grid = grid > cap ? cap : grid;
  const uint4* i4 = static_cast<const uint4*>(in);
  uint4* o4 = static_cast<uint4*>(out);
#define B200_AR_LAUNCH(T)                                                          \
  do {                                                                             \
    if (one) allreduce_oneshot_kernel<T><<<grid, 512, 0, stream>>>(p, i4, o4);     \
    else allreduce_twoshot_kernel<T><<<grid, 512, 0, stream>>>(p, i4, o4);         \
  } while (0)
  if (dtype == 0) B200_AR_LAUNCH(__nv_bfloat16);
  else if (dtype == 1) B200_AR_LAUNCH(__half);
  else if (dtype == 2) B200_AR_LAUNCH(F32Tag);
  else return -2;
#undef B200_AR_LAUNCH
  return 0;
}

// ------------------------------------------------------------------------------------------ reduce_rms
constexpr uint32_t kNotWritten = 0x80000000u;   // -0.0f: a sum of squares is never negative zero

template <typename T>
__global__ void __launch_bounds__(256)
reduce_rms_kernel(const ReduceRmsParams p) {
  const int which = blockIdx.y;
  const int H = p.H[which], ld = p.ld[which];
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(p.local_sync + 1);
  const int buf = (int)(call % 3u), clr = (int)((call + 2u) % 3u);
  const size_t buf_stride = (size_t)2 * p.tp * p.t_cap;
  const size_t base = (size_t)which * p.tp * p.t_cap;
  __shared__ float s_warp[8];
  __shared__ float s_src[kMaxRanks];
  __shared__ int s_ok;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = H >> 3;
  const T* w = static_cast<const T*>(p.w[which]);

  // slots of the array that the previous call used are free again: no peer writes it before call + 2
  // (both tensor halves, whatever this call's tensor count is)
  if (blockIdx.y == 0 && (int)threadIdx.x < 2 * p.tp) {
    const int t_prev = (int)p.local_sync[2 + clr];
    volatile uint32_t* mine = reinterpret_cast<volatile uint32_t*>(p.slots[p.rank] + clr * buf_stride);
    for (int t = blockIdx.x; t < t_prev; t += gridDim.x) mine[(size_t)threadIdx.x * p.t_cap + t] = kNotWritten;
  }

  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    const uint4* row = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x[which]) + (size_t)t * ld);
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8<T>(row[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    if (lane == 0) s_warp[warp] = ss;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < p.tp) {
      float tot = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += s_warp[i];
      tot = fabsf(tot);                                            // +0.0 at worst, never the sentinel
      const int r = threadIdx.x;
      // my partial into rank r's slot [buf][which][source = me][t]
      reinterpret_cast<volatile float*>(p.slots[r] + buf * buf_stride + base)[(size_t)p.rank * p.t_cap + t] = tot;
      // rank r's partial from my own array
      const volatile uint32_t* slot =
          reinterpret_cast<volatile uint32_t*>(p.slots[p.rank] + buf * buf_stride + base) + (size_t)r * p.t_cap + t;
      const long long t0 = clock64();
      uint32_t bits = *slot;
      while (bits == kNotWritten) {
        if (clock64() - t0 > p.wait_cycles) {
          report_status(p.status, kWaitTimeout, 153, t, r);
          s_ok = 0;
          bits = 0u;
          break;
        }
        __nanosleep(32);
        bits = *slot;
      }
      s_src[r] = __uint_as_float(bits);
    }
    __syncthreads();
    float total = 0.f;
    for (int r = 0; r < p.tp; ++r) total += s_src[r];             // rank order: identical on every rank
    const float inv = rsqrtf(total / ((float)H * (float)p.tp) + p.eps);
    uint4* orow = reinterpret_cast<uint4*>(static_cast<T*>(p.out[which]) + (size_t)t * ld);
    if (s_ok) {
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8], g[8];
        unpack8<T>(row[v], f);
        unpack8<T>(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * g[i];
        orow[v] = pack8<T>(f);
      }
    }
    __syncthreads();   // s_warp / s_src are rewritten by the next token
  }

  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(&p.local_sync[0], 1u);
    if (ticket == gridDim.x * gridDim.y - 1) {
      p.local_sync[0] = 0;
      p.local_sync[2 + buf] = (uint32_t)p.T;
      p.local_sync[1] = call + 1u;
    }
  }
}

// Returns 0, -1 (width not a multiple of 8 or T above the slot capacity).
int reduce_rms(const ReduceRmsParams& p, int dtype, cudaStream_t stream) {
  if (p.T <= 0) return 0;
  if (p.T > p.t_cap || p.n_tensors < 1 || p.n_tensors > 2) return -1;
  for (int i = 0; i < p.n_tensors; ++i)
    if ((p.H[i] & 7) != 0 || (p.ld[i] & 7) != 0) return -1;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // all CTAs resident (8 x 256 threads fit an SM): a CTA waits on peers only, but peers wait on its stores
  const int gx = p.T < sms * 4 / p.n_tensors ? p.T : sms * 4 / p.n_tensors;
  const dim3 grid(gx, p.n_tensors);
  if (dtype == 0) reduce_rms_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else reduce_rms_kernel<__half><<<grid, 256, 0, stream>>>(p);
  return 0;
}

}  // namespace b200
