// TMA / mbarrier / tensor-map helpers shared by the kernels that stream operands
// through shared memory (sm_100a).  Every wait is bounded: a wait that runs out
// records an error code and lets the kernel drain and return instead of hanging.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

// ---- host: tensor maps ------------------------------------------------------
// Encodes a 2-D tiled tensor map over a row-major [outer, inner] array.  The driver
// entry point is resolved at run time so the library does not link libcuda.
// swizzle: 0 none, 1 32B, 2 64B, 3 128B.  Returns false on failure.
bool tl_encode_tmap_2d(CUtensorMap* map, int elem_bytes, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle);

#ifdef __CUDACC__
constexpr int kWaitTimeoutIters = 1 << 22;  // each try_wait blocks for a while; this bounds a wait to seconds

enum { TL_DEV_OK = 0, TL_DEV_TIMEOUT_FULL = 1, TL_DEV_TIMEOUT_EMPTY = 2, TL_DEV_TIMEOUT_TMEM = 3 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when it gave up or when another role already raised
// the abort flag; the caller records `code` and leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (int it = 0; it < kWaitTimeoutIters; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63) == 63 && *abort_flag) return false;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
#endif  // __CUDACC__
