// Device helpers shared by the cluster kernels of the GEMM -> activation -> GEMM chain.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace ditto_b200 {

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// Bulk copy from this CTA's shared memory into a peer's; completion (bytes) on the peer's mbarrier.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, const void* src, uint32_t bytes,
                                                  uint32_t mbar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster_addr), "r"(smem_u32(src)), "r"(bytes), "r"(mbar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word,
                                                  uint32_t code) {
  for (uint32_t spin = 0; spin < (1u << 22); ++spin) {   // unhinted polls: the default limit
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_word != 0u) return false;
    if (spin > 4096u) __nanosleep(64);
  }
  atomicCAS(const_cast<uint32_t*>(abort_word), 0u, code);
  return false;
}


}  // namespace ditto_b200
