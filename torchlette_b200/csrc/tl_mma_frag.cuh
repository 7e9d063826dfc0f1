// int8 -> f16/bf16 pair conversion and the mma.sync.m16n8k16 wrapper shared by the small-batch
// kernels (tl_qgemv.cu, tl_qgemv_stream.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

template <typename AT> struct MmaOps;
template <> struct MmaOps<__half> {
  // bytes (b0,b1) / (b2,b3) of x = word ^ 0x80808080 -> f16 pairs holding q exactly:
  // 0x6400 | u is 1024 + u; subtracting 1152 (0x6480) leaves u - 128 = q.
  __device__ static void cvt(uint32_t word, uint32_t& lo, uint32_t& hi) {
    const uint32_t x = word ^ 0x80808080u;
    uint32_t l = __byte_perm(x, 0x64646464u, 0x4140);
    uint32_t h = __byte_perm(x, 0x64646464u, 0x4342);
    const uint32_t magic = 0x64806480u;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(l), "r"(magic));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h), "r"(magic));
  }
  __device__ static void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                             uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  // the same product as a plain (non-volatile) statement: the compiler may interleave independent
  // accumulator chains
  __device__ static void mma_free(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                  uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <> struct MmaOps<__nv_bfloat16> {
  // bf16 keeps 8 significant bits, so the byte cannot be stuffed whole.  With s the
  // sign bit and l the low 7 bits of the raw byte, q = l - 128*s:
  // (0x4300 | l) is 128 + l and (0x4300 | s<<7) is 128 or 256; their difference is q.
  __device__ static void cvt(uint32_t word, uint32_t& lo, uint32_t& hi) {
    const uint32_t l = __byte_perm(word, 0u, 0x4140);  // [b0,0,b1,0]
    const uint32_t h = __byte_perm(word, 0u, 0x4342);
    const uint32_t lm = (l & 0x007f007fu) | 0x43004300u, lc = (l & 0x00800080u) | 0x43004300u;
    const uint32_t hm = (h & 0x007f007fu) | 0x43004300u, hc = (h & 0x00800080u) | 0x43004300u;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(lm), "r"(lc));
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(hm), "r"(hc));
  }
  __device__ static void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                             uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  __device__ static void mma_free(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                  uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

