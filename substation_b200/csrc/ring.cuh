// Shared-memory input ring fed by bulk copies (cp.async.bulk, this CTA's own memory only).
//
// The LayerNorm forward and backward operators stream whole token rows: one producer warp keeps a ring of
// stages filled, each stage holding every input row of one token, while the consumer warps work out of shared
// memory.  Bytes in flight per SM are then the ring size (100-170 KB), not what the consumers' registers can
// hold, and a consumer's critical path per token no longer contains a trip to HBM.
//   full[s]   one arrival (the producer's expect_tx) + the stage's bytes
//   empty[s]  one arrival per consumer warp that read the stage
// Every wait is bounded: after ~2 s the waiter records a code in g_ring_error and the CTA leaves its loops; the
// host reads the flag through sb_device_error.

#pragma once

#include "common.cuh"

namespace sb {
namespace ring {

__device__ int g_ring_error = 0;   // first failure code since the last reset (per device)

constexpr unsigned long long kWaitNs = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kWaitNs, or earlier when another CTA already failed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
  unsigned long long t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 0x3ffu) == 0) {
      if (*reinterpret_cast<volatile int*>(&g_ring_error) != 0) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitNs) { atomicCAS(&g_ring_error, 0, code); return false; }
    }
  }
}
// `bytes` (a multiple of 16) from global `src` (16-byte aligned) to shared `dst` (16-byte aligned); completion is
// counted on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

}  // namespace ring
}  // namespace sb
