// Helpers for asynchronous copies into shared memory: mbarriers with bounded waits, TMA tile
// loads (cp.async.bulk.tensor), plain bulk copies (cp.async.bulk) and the host-side encoder of
// tensor maps.  No load here uses cluster multicast.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace rl {

#ifndef RL_MBAR_SLEEP_NS
#define RL_MBAR_SLEEP_NS 1000u
#endif
// Polls of an mbarrier before a waiter gives up (and raises the CTA's abort flag).
constexpr int kSpinLimit = 1 << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
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
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same, but the thread may sleep in the instruction for up to about `ns` nanoseconds (it is woken
// when the phase completes): a waiting warp then hardly takes issue slots from the working ones.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity; false if the CTA is aborting or the limit ran out.  A
// poll sleeps for up to a microsecond, so the limit is a matter of seconds.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
  if (mbar_try_wait(bar, parity)) return true;
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait_sleep(bar, parity, RL_MBAR_SLEEP_NS)) return true;
    if (*abort) return false;
  }
  *abort = 1;
  return false;
}

// The same for waits on the critical path of a pipeline: polls without a sleep hint (a poll still
// blocks in the instruction for a short, hardware-chosen time), so that the waiter goes on at once
// when the phase completes.  Bounded alike: the limit is a matter of seconds.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* abort) {
  for (int i = 0; i < (kSpinLimit >> 4); ++i) {
#pragma unroll 1
    for (int j = 0; j < 64; ++j)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
  }
  *abort = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Plain bulk copy of `bytes` (a multiple of 16; both addresses 16-byte aligned) that completes on an mbarrier.
__device__ __forceinline__ void bulk_load(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

}  // namespace rl

namespace rl {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace rl
