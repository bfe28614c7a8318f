// Peer copy kernels: local (or peer) source -> peer (or local) destination, used by the symmetric-memory
// utilities and to measure what one GPU can push over NVLink with a given number of CTAs.
//   mode 0  plain 16-byte loads / stores, `ctas` CTAs x 256 threads, 4 vectors in flight per thread
//   mode 1  bulk async copies: each CTA streams 16 KB pieces global -> shared -> global through a 12-slot ring
//           (one issuing thread per CTA)
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
using namespace ptx;

__global__ void __launch_bounds__(256) p2p_copy_plain_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t nvec) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < nvec; i += stride) dst[i] = src[i];
}

constexpr int kP2pPiece = 16384, kP2pSlots = 12, kP2pLag = 8;

__global__ void __launch_bounds__(32) p2p_copy_bulk_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                                                          size_t nbytes, StatusWord* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kP2pSlots * kP2pPiece);
  if (threadIdx.x != 0) return;
  for (int s = 0; s < kP2pSlots; ++s) mbar_init(&full[s], 1);
  fence_mbar_init();
  const size_t pieces = nbytes / kP2pPiece;
  const size_t mine = pieces > blockIdx.x ? (pieces - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  for (size_t i = 0; i < mine + kP2pLag; ++i) {
    if (i < mine) {
      const int s = (int)(i % kP2pSlots);
      tma_store_wait_read<kP2pSlots - kP2pLag - 1>();
      const size_t off = (blockIdx.x + i * gridDim.x) * (size_t)kP2pPiece;
      mbar_expect_tx(&full[s], kP2pPiece);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_u32(smem + s * kP2pPiece)), "l"(src + off), "r"(kP2pPiece), "r"(smem_u32(&full[s])) : "memory");
    }
    if (i >= kP2pLag) {
      const size_t j = i - kP2pLag;
      const int s = (int)(j % kP2pSlots);
      if (!mbar_wait(&full[s], (uint32_t)((j / kP2pSlots) & 1))) {
        report_status(status, kWaitTimeout, 170, (int)j, s);
        return;
      }
      const size_t off = (blockIdx.x + j * gridDim.x) * (size_t)kP2pPiece;
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + off),
                   "r"(smem_u32(smem + s * kP2pPiece)), "r"(kP2pPiece) : "memory");
      tma_store_commit();
    }
  }
  tma_store_wait<0>();
}

// nbytes must be a multiple of 16 (mode 0) or 16384 (mode 1).
void p2p_copy(void* dst, const void* src, size_t nbytes, int ctas, int mode, void* status, cudaStream_t stream) {
  if (nbytes == 0) return;
  if (mode == 0) {
    p2p_copy_plain_kernel<<<ctas, 256, 0, stream>>>((uint4*)dst, (const uint4*)src, nbytes / 16);
  } else {
    const int smem = kP2pSlots * kP2pPiece + kP2pSlots * 8 + 256;
    static bool set = false;
    if (!set) {
      cudaFuncSetAttribute(p2p_copy_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      set = true;
    }
    p2p_copy_bulk_kernel<<<ctas, 32, smem, stream>>>((uint8_t*)dst, (const uint8_t*)src, nbytes,
                                                     reinterpret_cast<StatusWord*>(status));
  }
}

}  // namespace b200
