// Bulk asynchronous copies (TMA, untiled form) and the mbarrier they complete on.
// Device code is inline PTX for sm_90+/sm_100a; the host versions are plain copies so
// that the block bodies can be emulated on a CPU.
//
// Rules kept here: both addresses 16-byte aligned and the size a multiple of 16
// bytes (checked by the host before this path is chosen); no cluster multicast;
// every wait is bounded and reports failure instead of spinning for ever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace cvb {

#ifdef __CUDA_ARCH__
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// global -> this block's shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if the phase did not complete within `limit` polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int limit) {
  for (int i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
#else
inline uint32_t smem_u32(const void*) { return 0; }
inline void mbar_init(uint64_t*, int) {}
inline void mbar_fence_init() {}
inline void mbar_expect_tx(uint64_t*, uint32_t) {}
inline void mbar_arrive(uint64_t*) {}
inline void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t*) { memcpy(dst, src, bytes); }
inline bool mbar_try_wait(uint64_t*, uint32_t) { return true; }
inline bool mbar_wait_bounded(uint64_t*, uint32_t, int) { return true; }
#endif

}  // namespace cvb
