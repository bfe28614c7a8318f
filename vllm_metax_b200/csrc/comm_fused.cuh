// Shared pieces of the fused compute + collective kernels: parameter blocks, system-scope
// flag primitives with bounded waits.
//
// Cross-GPU traffic goes over NVLink to IPC-mapped buffers as plain peer loads / stores, bulk copies and
// TMA tensor stores from shared memory, and plain (never cluster-multicast) TMA loads of peer rows; no NCCL call
// and no library kernel is ever handed peer memory.  Every wait on a value another GPU writes is bounded by an
// SM-clock budget; on expiry the waiter records {site, expected, observed} in the status word
// and carries on without the data, so a missing peer can never hang the GPU - the host turns the
// status into an exception.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "comm_params.h"

namespace b200 {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Spin until *p >= want (wrap-safe compare) or the cycle budget runs out.  Returns success.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t want, long long budget, uint32_t* seen) {
  const long long t0 = clock64();
  for (;;) {
    const uint32_t v = ld_acquire_sys(p);
    if ((int32_t)(v - want) >= 0) return true;
    if (clock64() - t0 > budget) {
      *seen = v;
      return false;
    }
    __nanosleep(64);
  }
}

}  // namespace b200
