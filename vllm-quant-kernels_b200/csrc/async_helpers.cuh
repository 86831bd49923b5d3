// mbarrier / bulk-copy (TMA) helpers shared by the asynchronous lm_head kernels.
// Every wait is bounded: when it runs out the kernel raises g_stream_error, flags the CTA as
// aborting and drains, so a wrong descriptor can cost a wrong answer but never a hung GPU.
#pragma once

#include "vqk_common.cuh"

namespace vqk {

// one copy per translation unit (no relocatable device code); the host reads each copy
static __device__ int g_stream_error = 0;
static inline int read_stream_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_stream_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

static inline int clear_stream_error() {
  const int zero = 0;
  return cudaMemcpyToSymbol(g_stream_error, &zero, sizeof(int)) == cudaSuccess ? 0 : -1;
}

constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait; false means the CTA is aborting (flag set by whoever ran out first)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(&g_stream_error, 1);
  return false;
}
// Drain of a producer's own copies before its CTA exits: wait, with a limit and whatever the
// abort flag says, until the barrier phase that the copy completes has passed.  On the normal
// path the consumer has already waited for it and this returns at once.
__device__ __forceinline__ bool mbar_drain(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 20); ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// warp-uniform form: every lane polls, the warp proceeds only if every lane got through
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}


}  // namespace vqk
