// Thin wrappers over the sm_100a PTX used by the kernels: mbarriers, bulk asynchronous
// copies, proxy fences and bounded waits.  Device code only.
#pragma once

#include <cstdint>

namespace aq {

constexpr uint32_t kSpinLimit = 1u << 24;  // polls before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on phase `parity` of an mbarrier.  Returns false when the CTA is
// aborting: either this wait ran out of polls (it then raises `abort_flag` in shared
// memory and records `code` in the global `status` word) or another thread did.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          int* status, int code) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag != 0) return false;
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

// 1-D bulk asynchronous copy global -> shared; both addresses 16-byte aligned, size a
// multiple of 16; completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Asks the L2 cache to fetch `bytes` (a multiple of 16, 16-byte aligned address) of this GPU's
// own global memory; nothing waits for it and nothing is written.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// This CTA's share of a look-ahead prefetch: the `total_bytes` at `base` are cut into one
// contiguous slice per CTA (128-byte granules) and requested in pieces of at most 16 KiB.
// The pieces are dealt to `issuers` callers (`issuer` = 0 .. issuers - 1, one thread each): a
// bulk instruction holds its issuing warp for about 150 cycles whatever its size, so a slice
// of a dozen pieces asked for by one thread would hold that warp for a microsecond.
__device__ __forceinline__ void prefetch_slice_l2(const uint8_t* base, int64_t total_bytes, int64_t cta, int64_t ctas,
                                                  int issuer = 0, int issuers = 1) {
  const int64_t slice = (((total_bytes + ctas - 1) / ctas) + 127) & ~static_cast<int64_t>(127);
  const int64_t begin = cta * slice;
  const int64_t end = begin + slice < total_bytes ? begin + slice : total_bytes;
  for (int64_t at = begin + static_cast<int64_t>(issuer) * 16384; at < end; at += static_cast<int64_t>(issuers) * 16384) {
    const int64_t left = end - at;
    bulk_prefetch_l2(base + at, static_cast<uint32_t>(left < 16384 ? left : 16384) & ~15u);
  }
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Programmatic dependent launch: wait for the preceding grid's memory / let the next
// grid start its independent prologue.  Both are no-ops for ordinary launches.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace aq
