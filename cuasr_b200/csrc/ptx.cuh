// Thin wrappers over the sm_100a PTX this library uses: mbarrier, TMA (plain per-CTA cp.async.bulk.tensor
// loads only), packed fp32x2 arithmetic and three-input min/max.
//
// Every wait is bounded: a wait that runs out of attempts records a code in a device-side status word
// and the waiter stops waiting (the producer returns; consumer warps go through mbar_wait_or_abandon, which lets
// all of them finish their loops so that no warp is left alone at a barrier) instead of spinning forever.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace cuasr_b200 {

// Codes a kernel may leave in the device-side status word it is handed (0 = no error).
enum DeviceStatus : unsigned int {
  kDeviceOk              = 0,
  kDeviceTimeoutFull     = 1,  // a consumer gave up waiting for a tile to land in shared memory
  kDeviceTimeoutEmpty    = 2,  // the producer gave up waiting for a stage to be released
  kDeviceTimeoutPeerFlag = 3,  // a rank gave up waiting for a peer's arrival flag
};

__device__ __forceinline__ void report_device_error(unsigned int* status, unsigned int code) {
  if (status != nullptr) atomicCAS(status, 0u, code);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                   smem_u32(bar)),
               "r"(bytes)
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

// Each try_wait suspends for a hardware-defined slice of time, so the limit below is seconds, not
// microseconds: long enough for any healthy pipeline, short enough that a broken one returns.
constexpr uint32_t kMaxWaitAttempts = 1u << 24;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* status,
                                          unsigned int code_on_timeout) {
  for (uint32_t i = 0; i < kMaxWaitAttempts; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  report_device_error(status, code_on_timeout);
  return false;
}

// The consumers' form of the wait.  Consumer warps of a CTA meet at named barriers (split tiles), so one of them
// must not leave while the others go on.  When a wait runs out here, the code is recorded and a flag in shared
// memory is raised; from then on every wait of the CTA that does not succeed at once returns after a few attempts,
// and all warps finish their loops on whatever the stages hold.  The result of such a launch is void and the status
// word says so; what matters is that the kernel ends.
__device__ __forceinline__ void mbar_wait_or_abandon(uint64_t* bar, uint32_t parity, unsigned int* status,
                                                     unsigned int code_on_timeout, volatile unsigned int* abandoned) {
  if (mbar_try_wait(bar, parity)) return;
  for (uint32_t i = 0; i < kMaxWaitAttempts; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63) == 63 && *abandoned != 0) return;
  }
  report_device_error(status, code_on_timeout);
  *abandoned = 1;
}

// 2-D tiled TMA load into this CTA's shared memory, completion signalled on `bar`.
// x is the coordinate along the contiguous dimension and must keep x * sizeof(element) a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- packed / three-input arithmetic (sm_100 and later) ----

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
  float r;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

}  // namespace cuasr_b200
