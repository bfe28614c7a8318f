// Mamba-1 selective scan forward:
//
//     h_t = exp(dt_t * A) * h_{t-1} + dt_t * B_t * u_t ;   y_t = <h_t, C_t> + D * u_t ;   y_t *= silu(z_t)
//
// u / delta / z are [dim, total_tokens] (variable-length batch, query_start_loc) or [batch, dim, L];
// B / C are [groups, dstate, total_tokens] (or [batch, groups, dstate, L]); the recurrent state
// [slots, dim, dstate] lives in a paged cache addressed by cache_indices and is read when
// has_initial_state[b] is set (chunked prefill / decode) and always written back.
// A channel's dstate values are spread over LANES = dstate / 4 lanes (4 states per lane in registers); a warp therefore advances 32 / LANES
// channels in lock step through time, reducing <h, C> with shuffles inside each lane group.  Time is
// the only sequential dimension; (sequence, channel) pairs fill the GPU.
// Parity: csrc/mamba/selective_scan_fwd.cu:69 (+ selective_scan.h) of the reference.
#include "common.cuh"
#include "ops.h"

namespace b200 {


template <typename T, int LANES>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const ScanParams p) {
  constexpr int CPW = 32 / LANES;                    // channels per warp
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LANES, cw = lane / LANES;
  const int b = blockIdx.y;
  const int d = (blockIdx.x * 4 + warp) * CPW + cw;
  const bool varlen = p.query_start_loc != nullptr;
  const int t0 = varlen ? p.query_start_loc[b] : 0;
  const int L = varlen ? p.query_start_loc[b + 1] - t0 : p.seqlen;
  const int slot = p.cache_indices ? p.cache_indices[b] : b;
  if (slot == p.pad_slot || d >= p.dim) return;      // whole lane groups leave together (dim % CPW == 0)
  const int64_t tok_stride = varlen ? p.total_tokens : p.seqlen;
  // element (channel d, time t) of u/delta/z/out; (group g, state n, time t) of B/C
  const int64_t ud_base = varlen ? (int64_t)d * tok_stride + t0 : ((int64_t)b * p.dim + d) * tok_stride;
  const int g = d / (p.dim / p.groups);
  const int64_t bc_base = varlen ? (int64_t)g * p.dstate * tok_stride + t0
                                 : ((int64_t)b * p.groups + g) * p.dstate * tok_stride;
  const T* u = reinterpret_cast<const T*>(p.u) + ud_base;
  const T* dl = reinterpret_cast<const T*>(p.delta) + ud_base;
  const T* z = p.z ? reinterpret_cast<const T*>(p.z) + ud_base : nullptr;
  T* out = reinterpret_cast<T*>(p.out) + ud_base;
  const T* Bm = reinterpret_cast<const T*>(p.B) + bc_base;
  const T* Cm = reinterpret_cast<const T*>(p.C) + bc_base;
  float a[4], h[4];
  float* st = p.state + ((int64_t)slot * p.dim + d) * p.dstate;
  const bool init = p.has_initial_state && p.has_initial_state[b];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = sub * 4 + i;
    a[i] = p.A[(int64_t)d * p.dstate + n];
    h[i] = init ? st[n] : 0.f;
  }
  const float Dv = p.D ? p.D[d] : 0.f;
  const float bias = p.delta_bias ? p.delta_bias[d] : 0.f;
  for (int t = 0; t < L; ++t) {
    float dt = to_f(dl[t]) + bias;
    if (p.softplus) dt = dt > 20.f ? dt : log1pf(__expf(dt));
    const float uv = to_f(u[t]);
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t n = sub * 4 + i;
      h[i] = __expf(dt * a[i]) * h[i] + dt * to_f(Bm[n * tok_stride + t]) * uv;
      y += h[i] * to_f(Cm[n * tok_stride + t]);
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
    if (sub == 0) {
      y += Dv * uv;
      if (z) {
        const float zv = to_f(z[t]);
        y *= zv / (1.f + __expf(-zv));
      }
      out[t] = from_f<T>(y);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) st[sub * 4 + i] = h[i];
}

// dstate in {4, 8, 16, 32, 64, 128}; dim a multiple of 32.  dtype: 0 bf16, 1 fp16, 2 fp32.
int selective_scan_fwd(const ScanParams& p, int dtype, cudaStream_t stream) {
  if (p.batch <= 0 || p.dim <= 0) return 0;
  const int lanes = p.dstate / 4;
  if (p.dstate % 4 || lanes < 1 || lanes > 32 || (lanes & (lanes - 1)) || p.dim % 32 || p.dim % p.groups) return 1;
  const int cpw = 32 / lanes;
  dim3 grid(ceil_div(p.dim, 4 * cpw), p.batch);
#define SCAN(T, LN) selective_scan_kernel<T, LN><<<grid, 128, 0, stream>>>(p)
#define SCAN_T(T)                                                                                         \
  switch (lanes) {                                                                                        \
    case 1: SCAN(T, 1); break; case 2: SCAN(T, 2); break; case 4: SCAN(T, 4); break;                      \
    case 8: SCAN(T, 8); break; case 16: SCAN(T, 16); break; default: SCAN(T, 32); break;                  \
  }
  if (dtype == 0) { SCAN_T(__nv_bfloat16) } else if (dtype == 1) { SCAN_T(__half) } else { SCAN_T(float) }
#undef SCAN_T
#undef SCAN
  return 0;
}

}  // namespace b200
