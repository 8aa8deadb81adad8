// mbarrier / TMA (cp.async.bulk) primitives shared by the kernels, as inline PTX.
// Every wait is bounded: after WAIT_LIMIT polls it records a code in a status word (when one is
// given) and returns, so that a lost completion shows up as an error flag, never as a hang.
// A kernel also gives its waits one word of shared memory (`abort`, zero at start): the first wait of the CTA
// that expires sets it, and every other wait of that CTA returns false within a few polls of seeing it, so that
// after one lost completion all roles run out of their loops promptly (on meaningless data -- the status word
// says so) and the normal exit path still frees what the CTA holds (tensor memory, cluster barriers).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tma {

constexpr int WAIT_LIMIT = 1 << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code, int* abort = nullptr,
                                          int limit = WAIT_LIMIT) {
  for (int it = 0; it < limit; ++it) {
    if (mbar_try(bar, parity)) return true;
    if (abort != nullptr && (it & 15) == 15 && *reinterpret_cast<volatile int*>(abort) != 0) return false;
  }
  if (abort != nullptr) *reinterpret_cast<volatile int*>(abort) = code;
  if (status) atomicCAS(status, 0, code);            // the first code stays: it names the wait that gave up
  return false;
}
// Contiguous global -> shared copy; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

}  // namespace tma
