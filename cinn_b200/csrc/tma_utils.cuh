// Bulk asynchronous copy (TMA, non-tensor form) and mbarrier helpers shared by the streaming kernels.
//
// Only the plain global -> shared::cluster form is used (no multicast qualifier, no tensor maps): a CTA launched
// without a cluster is its own cluster of one, so the destination window is this CTA's shared memory.  Sizes are
// multiples of 16 bytes and both addresses 16-byte aligned.  Every wait is bounded.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cinn_b200 {

// Each translation unit that waits on mbarriers owns a device counter of bounded waits that gave up (device code is
// compiled without relocatable linking, so a counter cannot be shared between files).  The macro defines the
// counter, a host function that reads and clears it, and registers that function; cinn_b200_device_status sums
// the counters of all files.
typedef unsigned int (*AsyncTimeoutReader)(int* cuda_status);
int RegisterAsyncTimeoutReader(AsyncTimeoutReader reader);  // runtime.cc

#define CINN_B200_DEFINE_ASYNC_TIMEOUT_COUNTER(counter)                                                   \
  __device__ unsigned int counter = 0;                                                                    \
  static unsigned int ReadAndClear_##counter(int* cuda_status) {                                          \
    unsigned int v = 0, zero = 0;                                                                         \
    cudaError_t e = cudaMemcpyFromSymbol(&v, counter, sizeof(v));                                         \
    if (e == cudaSuccess && v != 0) e = cudaMemcpyToSymbol(counter, &zero, sizeof(zero));                 \
    if (cuda_status) *cuda_status = (int)e;                                                               \
    return v;                                                                                             \
  }                                                                                                       \
  static int registered_##counter = ::cinn_b200::RegisterAsyncTimeoutReader(&ReadAndClear_##counter)

constexpr int kMaxStages      = 8;
constexpr unsigned kWaitLimit = 1u << 22;  // try_wait calls before a wait is abandoned

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (unsigned i = 0; i < kWaitLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Global -> this CTA's shared memory, `bytes` a multiple of 16, both addresses 16-byte aligned; completion is
// signalled on `bar` as transferred bytes.  (A CTA launched without a cluster is its own cluster of one, so the
// shared::cluster destination window is this CTA's shared memory.)
__device__ __forceinline__ void bulk_load_row(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}


}  // namespace cinn_b200
