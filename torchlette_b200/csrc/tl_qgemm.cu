// Quantized matmul on the 5th-generation tensor cores (tcgen05 + TMEM), with the
// int8 -> f16/bf16 dequantization fused into the operand path.  Replaces the
// reference's explicit-dequant + tiled-matmul pair for m > 1
// (src/backend/webgpu/ops/matmul-ops.ts:163-181, src/schedule/matmul-skeleton.ts:738-966).
//
//   out[m, n] = epilogue(alpha * sum_k a[m, k] * W[n, k])
//
// The problem is run "swapped": the WEIGHT rows are the 128-row M dimension of the
// MMA and the tokens are its N dimension, D[128 weight rows, BN tokens] in TMEM.
//   - a producer thread streams raw int8 weight boxes [128 rows x KSTEP bytes] and
//     activation boxes [BN tokens x 64 k] into a shared-memory ring with TMA;
//   - converter warps own one weight row per thread (= one TMEM lane): they read the
//     row's bytes from the swizzled box, turn them into f16/bf16 pairs in registers
//     (exactly; grouped scales are multiplied in here) and write them with
//     tcgen05.st into a TMEM operand slot -- the dequantized weight never touches
//     shared or global memory;
//   - one thread issues tcgen05.mma with the A operand in TMEM and the activations
//     (B) read from shared memory through a 128-byte-swizzle descriptor;
//   - epilogue warps read the f32 accumulator back with tcgen05.ld (one weight row
//     = one output column per thread, so the per-channel scale and the bias are
//     per-thread constants), apply alpha / scale / the fused op chain and store.
// Accumulators are double buffered in TMEM so the epilogue of tile i overlaps the
// main loop of tile i+1.  One persistent CTA per SM walks the tiles, token tiles
// fastest so that CTAs running side by side share weight boxes through L2.
//
// Every wait is bounded; a wait that runs out raises a status word, all roles
// drain, TMEM is released and the kernel returns.
#include <algorithm>
#include <type_traits>

#include "tl_common.cuh"
#include "tl_tcgen05.cuh"
#include "tl_tma.cuh"

#define TL_TR(role, it, ev) do {} while (0)

namespace {

// int8 word -> two packed pairs holding q exactly (see the GEMV kernels for the bit tricks)
template <typename AT> struct Cvt;
template <> struct Cvt<__half> {
  static constexpr uint32_t kFmt = 0;  // instruction-descriptor operand format
  __device__ static void word(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t x = w ^ 0x80808080u;
    const uint32_t l = __byte_perm(x, 0x64646464u, 0x4140), h = __byte_perm(x, 0x64646464u, 0x4342);
    const uint32_t magic = 0x64806480u;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(l), "r"(magic));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h), "r"(magic));
  }
  __device__ static uint32_t mul(uint32_t a, uint32_t s) {
    uint32_t r;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(s));
    return r;
  }
  __device__ static uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
  }
  __device__ static uint32_t splat(float s) {
    const __half2 h = __float2half2_rn(s);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  __device__ static uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
};
template <> struct Cvt<__nv_bfloat16> {
  static constexpr uint32_t kFmt = 1;
  __device__ static void word(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t l = __byte_perm(w, 0u, 0x4140), h = __byte_perm(w, 0u, 0x4342);
    const uint32_t lm = (l & 0x007f007fu) | 0x43004300u, lc = (l & 0x00800080u) | 0x43004300u;
    const uint32_t hm = (h & 0x007f007fu) | 0x43004300u, hc = (h & 0x00800080u) | 0x43004300u;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(lm), "r"(lc));
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(hm), "r"(hc));
  }
  __device__ static uint32_t mul(uint32_t a, uint32_t s) {
    uint32_t r;
    asm("mul.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(s));
    return r;
  }
  __device__ static uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
  }
  __device__ static uint32_t splat(float s) {
    const __nv_bfloat162 h = __float2bfloat162_rn(s);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  __device__ static uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
};

// The weight as a 16-bit [N, K] matrix in scratch, for the dense kernel (variant "dequant+dense"):
// per-channel weights as q itself (the scale is applied per output column in that kernel's epilogue,
// as the fused kernel does), grouped weights as round(q * scale), the fused converters' arithmetic.
template <typename AT, bool GROUPED>
__global__ void __launch_bounds__(256)
dequant_int8_16_kernel(const uint2* __restrict__ packed, const void* __restrict__ scales, int scales_dtype, float wscale, int group,
                       int groups_per_row, int64_t k, int64_t n_oct, uint4* __restrict__ out) {
  // One octet (8 weights: 8 bytes in, 16 bytes out) per thread and step, so that a warp's loads AND its
  // stores are each one contiguous run; four independent steps in flight.
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t o0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; o0 < n_oct; o0 += 4 * stride) {
    uint2 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (o0 + u * stride < n_oct) raw[u] = __ldcs(packed + o0 + u * stride);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t o = o0 + u * stride;
      if (o >= n_oct) break;
      uint32_t v[4];
      if (GROUPED) {
        const int64_t e = o * 8, row = e / k;
        const float sc = tl_load_scale(scales, scales_dtype, row * groups_per_row + (e - row * k) / group) * wscale;
        const uint32_t w2[2] = {raw[u].x, raw[u].y};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t x = w2[j] ^ 0x80808080u;
          const float f0 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650)) - 8388736.f) * sc;
          const float f1 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651)) - 8388736.f) * sc;
          const float f2 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652)) - 8388736.f) * sc;
          const float f3 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653)) - 8388736.f) * sc;
          v[2 * j] = Cvt<AT>::pack(f0, f1);
          v[2 * j + 1] = Cvt<AT>::pack(f2, f3);
        }
      } else {
        Cvt<AT>::word(raw[u].x, v[0], v[1]);
        Cvt<AT>::word(raw[u].y, v[2], v[3]);
      }
      out[o] = make_uint4(v[0], v[1], v[2], v[3]);
    }
  }
}

// One unary op over sixteen accumulators.  The op and the precision are resolved once, so
// each case is a straight run of sixteen independent chains.
template <int OP, bool APPROX>
__device__ __forceinline__ void unary16_case(float (&o)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j] = APPROX ? tl_unary_approx(OP, o[j]) : tl_unary(OP, o[j]);
}
__device__ __forceinline__ void unary16(int op, bool approx, float (&o)[16]) {
#define TL_U16(OP) case OP: if (approx) unary16_case<OP, true>(o); else unary16_case<OP, false>(o); break;
  switch (op) {
    TL_U16(TL_UNARY_RELU)
    TL_U16(TL_UNARY_SILU)
    TL_U16(TL_UNARY_SIGMOID)
    TL_U16(TL_UNARY_TANH)
    TL_U16(TL_UNARY_GELU_TANH)
    TL_U16(TL_UNARY_GELU_ERF)
    default: break;
  }
#undef TL_U16
}

struct GemmArgs {
  const void* scales;
  void* out;
  int64_t m, n, k;
  int32_t group, groups_per_row, scales_dtype, out_dtype;
  float wscale;
  int* status;
  int32_t n_tiles, m_tiles, ksteps;
  // Work decomposition: tiles [0, full_tiles) are whole-K items; each of the rem_tiles after
  // them is cut into `splits` K ranges of ks_per_split steps so that the last, partial wave
  // still fills the machine.  Split partials meet in `slabs`; `counters` (zero between
  // launches) elects the finishing CTA of each cut tile.
  int32_t full_tiles, rem_tiles, splits, ks_per_split;
  float* slabs;
  int* counters;
};

struct WorkItem { int tile, ks0, nks, slot, part; };

// The i-th work item of this CTA (items are dealt round-robin over the grid).
__device__ __forceinline__ bool get_work(const GemmArgs& p, int i, WorkItem& w) {
  const int idx = int(blockIdx.x) + i * int(gridDim.x);
  if (idx < p.full_tiles) {
    w.tile = idx; w.ks0 = 0; w.nks = p.ksteps; w.slot = -1; w.part = 0;
    return true;
  }
  const int j = idx - p.full_tiles;
  if (j >= p.rem_tiles * p.splits) return false;
  if (p.splits == 1) {
    w.tile = p.full_tiles + j; w.ks0 = 0; w.nks = p.ksteps; w.slot = -1; w.part = 0;
    return true;
  }
  w.slot = j / p.splits;
  w.part = j - w.slot * p.splits;
  w.tile = p.full_tiles + w.slot;
  w.ks0 = w.part * p.ks_per_split;
  w.nks = min(p.ks_per_split, p.ksteps - w.ks0);
  return true;
}

constexpr int kTileRows = 128;  // weight rows per CTA tile = TMEM lanes

__host__ __device__ constexpr uint32_t pow2_at_least(uint32_t v) {
  uint32_t p = 32;
  while (p < v) p <<= 1;
  return p;
}

template <typename AT, int BN, int KSTEP, int STAGES, int NCW, bool GROUPED>
__global__ void __launch_bounds__((NCW + 10) * 32, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap amap, GemmArgs p,
                EpiParams epi) {
  static_assert(KSTEP == 64 || KSTEP == 128, "one weight box row is 64 or 128 bytes");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "MMA N");
  static_assert(NCW == 4 || NCW == 8 || NCW == 16, "converter warps");
  constexpr int kWBytes = kTileRows * KSTEP;        // int8 weight box
  constexpr int kABox = BN * 128;                   // one [BN x 64] activation box
  constexpr int kABoxes = KSTEP / 64;
  constexpr int kStageBytes = kWBytes + kABoxes * kABox;
  constexpr int kSlotCols = KSTEP / 2;              // TMEM columns of one dequantized operand slot
  // The shared-memory ring (STAGES deep) has to cover the TMA round trip; the TMEM operand
  // ring only has to cover conversion -> MMA, so it is sized by what TMEM has left (TS slots).
  constexpr int kFreeCols = 512 - 2 * BN;
  constexpr int TS = (kFreeCols / kSlotCols) < STAGES ? (kFreeCols / kSlotCols) : STAGES;
  static_assert(TS >= 2, "TMEM operand ring");
  constexpr uint32_t kTmemCols = pow2_at_least(2 * BN + TS * kSlotCols);
  static_assert(kTmemCols <= 512, "TMEM budget");
  constexpr int kParts = NCW / 4;                   // converter threads per weight row
  constexpr int kChunks = KSTEP / 16 / kParts;      // 16-byte chunks per converter thread and stage
  constexpr int kEpiWarp0 = NCW, kEpiWarps = 8, kProducerWarp = NCW + 8, kMmaWarp = NCW + 9;
  // Both operands carry the activation type: kind::f16 with an f16 weight operand against
  // bf16 activations raised "illegal instruction" on B200, so the cheaper f16 bit trick cannot
  // be used for bf16 problems.
  using WT = AT;
  constexpr uint32_t kIdesc = (1u << 4) | (Cvt<WT>::kFmt << 7) | (Cvt<AT>::kFmt << 10) | (uint32_t(BN >> 3) << 17) |
                              (uint32_t(kTileRows >> 4) << 24);

  extern __shared__ uint8_t gemm_smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], aready_bar[TS], slotfree_bar[TS], tfull_bar[2], tempty_bar[2], esync_bar[2];
  __shared__ int split_last;
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < TS; ++s) {
      mbar_init(&aready_bar[s], NCW);
      mbar_init(&slotfree_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], kEpiWarps);
      mbar_init(&esync_bar[b], kEpiWarps);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&tmem_base_smem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&wmap);
      tma_prefetch_desc(&amap);
      int it = 0;
      WorkItem w;
      for (int wi = 0; get_work(p, wi, w) && !abort_flag; ++wi) {
        const int n_tile = w.tile / p.m_tiles, m_tile = w.tile - n_tile * p.m_tiles;
        for (int ks = w.ks0; ks < w.ks0 + w.nks; ++ks, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1, &abort_flag)) {
            if (!abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_EMPTY); }
            break;
          }
          TL_TR(0, it, 0);
          uint8_t* st = stages + size_t(s) * kStageBytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          tma_load_2d(st, &wmap, ks * KSTEP, n_tile * kTileRows, &full_bar[s]);
#pragma unroll
          for (int b = 0; b < kABoxes; ++b)
            tma_load_2d(st + kWBytes + b * kABox, &amap, ks * KSTEP + b * 64, m_tile * BN, &full_bar[s]);
          TL_TR(0, it, 1);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int it = 0, tl = 0;
      WorkItem w;
      for (; get_work(p, tl, w) && !abort_flag; ++tl) {
        const int acc = tl & 1;
        if (tl >= 2 && !mbar_wait(&tempty_bar[acc], ((tl >> 1) - 1) & 1, &abort_flag)) {
          if (!abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_TMEM); }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        bool ok = true;
        for (int ks = w.ks0; ks < w.ks0 + w.nks && ok; ++ks, ++it) {
          const int s = it % STAGES, sl = it % TS;
          TL_TR(1, it, 0);
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, &abort_flag);
          TL_TR(1, it, 1);
          ok = ok && mbar_wait(&aready_bar[sl], (it / TS) & 1, &abort_flag);
          TL_TR(1, it, 2);
          if (!ok) {
            if (!abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_FULL); }
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(stages + size_t(s) * kStageBytes + kWBytes);
          const uint32_t a_tmem = tmem_base + uint32_t(2 * BN + sl * kSlotCols);
#pragma unroll
          for (int kk = 0; kk < KSTEP / 16; ++kk) {
            const uint64_t bdesc = make_b_desc(a_base + (kk >> 2) * kABox + (kk & 3) * 32);
            tc_mma_ts(d_tmem, a_tmem + kk * 8, bdesc, kIdesc, (ks > w.ks0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);      // the shared-memory stage is free once these MMAs have run
          tc_commit(&slotfree_bar[sl]);  // and so is the TMEM operand slot
          TL_TR(1, it, 3);
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
      }
    }
  } else if (warp < NCW) {
    // ------------------------------ converters ------------------------------
    const int quad = warp & 3, part = warp >> 2;
    const int r = quad * 32 + lane;  // weight row inside the tile = TMEM lane
    const uint32_t swz = KSTEP == 128 ? uint32_t(r & 7) : uint32_t((r >> 1) & 3);
    const uint32_t row_off = uint32_t(r) * KSTEP;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    // Per k-step: wait for the stage, read this thread's bytes of its row, convert in registers,
    // wait for a free TMEM operand slot, store, and signal the MMA issuer right away.  (Overlapping
    // the next step's conversion with these stores measured slower: it delays the signal, and the
    // short shared-memory ring makes the loop latency bound, not throughput bound.)
    uint32_t v[kChunks][8];
    auto convert = [&](int it, int ks, int n_tile) -> bool {
      const int s = it % STAGES;
      if (warp == 0 && lane == 0) TL_TR(2, it, 0);
      if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, &abort_flag)) return false;
      if (warp == 0 && lane == 0) TL_TR(2, it, 1);
      const uint32_t wb = smem_u32(stages + size_t(s) * kStageBytes) + row_off;
      uint4 raw[kChunks];
#pragma unroll
      for (int i = 0; i < kChunks; ++i) raw[i] = lds128(wb + ((uint32_t(part * kChunks + i) ^ swz) << 4));
      int64_t grow = 0;
      if (GROUPED) grow = min(int64_t(n_tile) * kTileRows + r, p.n - 1);
#pragma unroll
      for (int i = 0; i < kChunks; ++i) {
        const int c = part * kChunks + i;
        if (GROUPED) {
          // exact: q -> f32 by exponent stuffing, one f32 multiply by the group scale, one
          // rounding to the 16-bit operand type (the oracle's dequantize-then-round)
          const int grp = (ks * KSTEP + c * 16) / p.group;
          const float sc = (grp < p.groups_per_row ? tl_load_scale(p.scales, p.scales_dtype, grow * p.groups_per_row + grp) : 0.f) * p.wscale;
          const uint32_t w4[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t x = w4[j] ^ 0x80808080u;
            const float f0 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650)) - 8388736.f) * sc;
            const float f1 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651)) - 8388736.f) * sc;
            const float f2 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652)) - 8388736.f) * sc;
            const float f3 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653)) - 8388736.f) * sc;
            v[i][2 * j] = Cvt<AT>::pack(f0, f1);
            v[i][2 * j + 1] = Cvt<AT>::pack(f2, f3);
          }
        } else {
          Cvt<WT>::word(raw[i].x, v[i][0], v[i][1]);
          Cvt<WT>::word(raw[i].y, v[i][2], v[i][3]);
          Cvt<WT>::word(raw[i].z, v[i][4], v[i][5]);
          Cvt<WT>::word(raw[i].w, v[i][6], v[i][7]);
        }
      }
      return true;
    };
    bool ok = true;
    int it = 0;
    WorkItem w;
    for (int wi = 0; ok && get_work(p, wi, w); ++wi) {
      const int n_tile = w.tile / p.m_tiles;
      for (int ks = w.ks0; ks < w.ks0 + w.nks; ++ks, ++it) {
        const int sl = it % TS;
        if (!convert(it, ks, n_tile)) { ok = false; break; }
        if (warp == 0 && lane == 0) TL_TR(2, it, 2);
        if (it >= TS && !mbar_wait(&slotfree_bar[sl], ((it / TS) - 1) & 1, &abort_flag)) { ok = false; break; }
        if (warp == 0 && lane == 0) TL_TR(2, it, 3);
        tc_fence_after();
        const uint32_t slot = tmem_base + lane_addr + uint32_t(2 * BN + sl * kSlotCols);
#pragma unroll
        for (int i = 0; i < kChunks; ++i) tmem_st8(slot + (part * kChunks + i) * 8, v[i]);
        if (warp == 0 && lane == 0) TL_TR(2, it, 4);
        tmem_st_wait();      // this thread's TMEM stores are complete
        if (warp == 0 && lane == 0) TL_TR(2, it, 5);
        tc_fence_before();
        __syncwarp();        // ... and so are those of the other 31 lanes
        if (lane == 0) mbar_arrive(&aready_bar[sl]);  // one arrival per warp keeps the barrier cheap
      }
    }
    if (!ok && lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_FULL); }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = (warp - kEpiWarp0) & 3, ehalf = (warp - kEpiWarp0) >> 2;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    // this warp's share of the BN token columns, in chunks of 16
    constexpr int kChunksN = BN / 16;
    const int cbeg = ehalf == 0 ? 0 : (kChunksN + 1) / 2, cend = ehalf == 0 ? (kChunksN + 1) / 2 : kChunksN;
    int tl = 0, esync = 0;
    WorkItem w;
    for (; get_work(p, tl, w); ++tl) {
      const int acc = tl & 1;
      const int n_tile = w.tile / p.m_tiles, m_tile = w.tile - n_tile * p.m_tiles;
      const int r = quad * 32 + lane;
      const int64_t ncol = int64_t(n_tile) * kTileRows + r;  // this thread's output column
      const bool n_ok = ncol < p.n;
      float sc = p.wscale;
      if (!GROUPED) sc *= n_ok ? tl_load_scale(p.scales, p.scales_dtype, ncol) : 0.f;
      if (GROUPED) sc = 1.f;  // group scales (and the convention factor) went in at conversion
      const bool fast = epi.fast != 0, approx = p.out_dtype != TL_F32;
      const float sca = sc * epi.alpha;
      const float bias = (fast && epi.fast_bias && n_ok) ? __ldg(epi.fast_bias + ncol) : 0.f;
      const int esz = p.out_dtype == TL_F32 ? 4 : 2;
      const int64_t row_bytes = p.n * esz;
      // sixteen accumulators of this thread's column (token rows m0 .. m0+15): epilogue + store
      auto emit16 = [&](int c0, const uint32_t (&v)[16]) {
        const int64_t m0 = int64_t(m_tile) * BN + c0;
        const int jmax = n_ok ? int(min(int64_t(16), p.m - m0)) : 0;
        uint8_t* optr = reinterpret_cast<uint8_t*>(p.out) + m0 * row_bytes + ncol * esz;
        if (fast) {
          // sixteen independent chains with the op decided once per chunk, not per element
          float o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = fmaf(__uint_as_float(v[j]), sca, bias);
          if (epi.fast_unary) unary16(epi.fast_unary, approx, o);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < jmax) {
              if (p.out_dtype == TL_F32) *reinterpret_cast<float*>(optr) = o[j];
              else if (p.out_dtype == TL_F16) *reinterpret_cast<__half*>(optr) = __float2half_rn(o[j]);
              else *reinterpret_cast<__nv_bfloat16*>(optr) = __float2bfloat16_rn(o[j]);
            }
            optr += row_bytes;
          }
        } else {
          // general op chain (binary operands, casts, several ops): rolled, one element at a time
          float vv[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) vv[j] = __uint_as_float(v[j]);
#pragma unroll 1
          for (int j = 0; j < jmax; ++j) {
            const float o = tl_apply_epilogue(epi, vv[j] * sc, m0 + j, ncol, p.n);
            if (p.out_dtype == TL_F32) *reinterpret_cast<float*>(optr) = o;
            else if (p.out_dtype == TL_F16) *reinterpret_cast<__half*>(optr) = __float2half_rn(o);
            else *reinterpret_cast<__nv_bfloat16*>(optr) = __float2bfloat16_rn(o);
            optr += row_bytes;
          }
        }
      };
      if (!mbar_wait(&tfull_bar[acc], (tl >> 1) & 1, &abort_flag)) {
        if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_TMEM); }
        break;
      }
      tc_fence_after();
      const bool split = w.slot >= 0;
      float* my_slab = split ? p.slabs + (size_t(w.slot) * p.splits + w.part) * size_t(kTileRows * BN) : nullptr;
      uint32_t vn[16];
      if (cbeg < cend) tmem_ld16(tmem_base + lane_addr + uint32_t(acc * BN + cbeg * 16), vn);
#pragma unroll 1
      for (int ch = cbeg; ch < cend; ++ch) {
        const int c0 = ch * 16;
        uint32_t v[16];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = vn[j];
        if (ch + 1 < cend) tmem_ld16(tmem_base + lane_addr + uint32_t(acc * BN + c0 + 16), vn);  // next chunk in flight
        if (!split) {
          emit16(c0, v);
        } else {
          // a K range of a cut tile: park the partial sums, token-major so that lanes coalesce
#pragma unroll
          for (int j = 0; j < 16; ++j) my_slab[(c0 + j) * kTileRows + r] = __uint_as_float(v[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (split) {
        // Elect the CTA that finishes this tile: the one whose partial arrives last.  The
        // epilogue warps meet on mbarriers (bounded waits), never on bar.sync, so a warp that
        // gave up cannot strand the others.
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(&esync_bar[0]);
        bool ok = mbar_wait(&esync_bar[0], esync & 1, &abort_flag);
        if (ok && warp == kEpiWarp0 && lane == 0) {
          const int prev = atomicAdd(p.counters + w.slot, 1);
          split_last = prev == p.splits - 1;
          if (split_last) p.counters[w.slot] = 0;  // every part has arrived: leave the counter clear
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&esync_bar[1]);
        ok = ok && mbar_wait(&esync_bar[1], esync & 1, &abort_flag);
        ++esync;
        if (!ok) {
          if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_TMEM); }
          break;
        }
        if (split_last) {
          __threadfence();
          const float* slab0 = p.slabs + size_t(w.slot) * p.splits * size_t(kTileRows * BN);
#pragma unroll 1
          for (int ch = cbeg; ch < cend; ++ch) {
            const int c0 = ch * 16;
            float sum[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) sum[j] = 0.f;
            for (int part = 0; part < p.splits; ++part) {  // fixed order: the result does not depend on arrival order
              const float* sp = slab0 + size_t(part) * size_t(kTileRows * BN) + size_t(c0) * kTileRows + r;
#pragma unroll
              for (int j = 0; j < 16; ++j) sum[j] += __ldcg(sp + j * kTileRows);
            }
            uint32_t v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(sum[j]);
            emit16(c0, v);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
constexpr int kTc = 0, kSliced = 1, kDequantDense = 2;

struct TcConfig { int bn, kstep, stages, ncw; };
// the instantiated tile configurations (tl_variant p0..p3)
const TcConfig kTcConfigs[] = {{192, 64, 6, 4}, {192, 64, 6, 8}, {128, 64, 8, 4}, {128, 64, 8, 8},
                               {64, 128, 6, 8}, {32, 128, 8, 8}, {16, 128, 8, 8},
                               {128, 128, 4, 8}, {192, 128, 3, 8}, {128, 128, 4, 16}, {192, 128, 3, 16}};

bool tc_config_known(const tl_variant& v) {
  for (const auto& c : kTcConfigs)
    if (c.bn == v.p0 && c.kstep == v.p1 && c.stages == v.p2 && c.ncw == v.p3) return true;
  return false;
}

template <typename AT, int BN, int KSTEP, int STAGES, int NCW>
cudaError_t launch_tc(bool grouped, int grid, cudaStream_t s, const CUtensorMap& wmap, const CUtensorMap& amap,
                      const GemmArgs& p, const EpiParams& e) {
  constexpr size_t smem = size_t(STAGES) * (kTileRows * KSTEP + (KSTEP / 64) * BN * 128) + 1024;
  constexpr int block = (NCW + 10) * 32;
  if (grouped) {
    auto kern = qgemm_tc_kernel<AT, BN, KSTEP, STAGES, NCW, true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    kern<<<grid, block, smem, s>>>(wmap, amap, p, e);
  } else {
    auto kern = qgemm_tc_kernel<AT, BN, KSTEP, STAGES, NCW, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    kern<<<grid, block, smem, s>>>(wmap, amap, p, e);
  }
  return cudaGetLastError();
}

template <typename AT>
cudaError_t launch_tc_cfg(const tl_variant& v, bool grouped, int grid, cudaStream_t s, const CUtensorMap& wmap,
                          const CUtensorMap& amap, const GemmArgs& p, const EpiParams& e) {
#define TL_TC_CASE(BN_, KS_, ST_, NCW_)                                             \
  if (v.p0 == BN_ && v.p1 == KS_ && v.p2 == ST_ && v.p3 == NCW_)                   \
    return launch_tc<AT, BN_, KS_, ST_, NCW_>(grouped, grid, s, wmap, amap, p, e);
  TL_TC_CASE(192, 64, 6, 4)
  TL_TC_CASE(192, 64, 6, 8)
  TL_TC_CASE(128, 64, 8, 4)
  TL_TC_CASE(128, 64, 8, 8)
  TL_TC_CASE(64, 128, 6, 8)
  TL_TC_CASE(32, 128, 8, 8)
  TL_TC_CASE(16, 128, 8, 8)
  TL_TC_CASE(128, 128, 4, 8)
  TL_TC_CASE(192, 128, 3, 8)
  TL_TC_CASE(128, 128, 4, 16)
  TL_TC_CASE(192, 128, 3, 16)
#undef TL_TC_CASE
  return cudaErrorInvalidValue;
}

}  // namespace

bool tl_qgemm_variant_applicable(const tl_variant& v, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q) {
  (void)n;
  if (v.family != TL_FAMILY_QGEMM || m < 1) return false;
  if (v.kernel == kSliced) return true;
  if (v.kernel == kDequantDense)
    return (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 16 == 0 && q.group_size % 16 == 0 &&
           tl_dense_tc_applicable(nullptr, nullptr, m, n, k, a_dtype, a_dtype) && uint64_t(n) * uint64_t(k) * 2 <= (uint64_t(4) << 30);
  if (v.kernel != kTc) return false;
  return (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 16 == 0 && q.group_size % 16 == 0 && tc_config_known(v);
}

int32_t tl_qgemm_default_variant(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q, tl_variant* out) {
  tl_variant v{};
  v.family = TL_FAMILY_QGEMM;
  if ((a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 16 == 0 && q.group_size % 16 == 0) {
    v.kernel = kTc;
    if (m <= 16) { v.p0 = 16; v.p1 = 128; v.p2 = 8; v.p3 = 8; }
    else if (m <= 32) { v.p0 = 32; v.p1 = 128; v.p2 = 8; v.p3 = 8; }
    else if (m <= 64) { v.p0 = 64; v.p1 = 128; v.p2 = 6; v.p3 = 8; }
    else {
      // 192 tokens x 128 k per step measured ~1.3x the throughput of the 128-token tile per padded
      // token, so it wins unless it pads the token count by more than that
      const int64_t pad192 = (m + 191) / 192 * 192, pad128 = (m + 127) / 128 * 128;
      if (pad192 * 3 <= pad128 * 4) { v.p0 = 192; v.p1 = 128; v.p2 = 3; v.p3 = 8; }
      else { v.p0 = 128; v.p1 = 128; v.p2 = 4; v.p3 = 8; }
      // With many tokens per weight byte, writing the weight out once as a 16-bit matrix and running the
      // dense kernel (whose operands both come from shared memory at its full tile sizes) beats converting
      // on the operand path: compare the modelled times.  Fused: 0.87 us per 128-k step of a 128 x 192 tile
      // (measured; 1.4 us with group scales), the last partial wave cut along K; dequantization: 3 bytes of
      // HBM traffic per weight (the pass alone runs at the copy peak, 27 us for 14336 x 4096; the model charges 4 TB/s
      // because the dense kernel that follows reads a freshly written operand and runs a little slower for it).  E.g. 2048 tokens: n = 4096,
      // k = 14336 runs 200 us this way against 229 us fused, n = 14336, k = 4096 228 against 229 (stays fused),
      // the same with groups of 128 218 against 368; 8192 tokens x 4096 x 4096: 231 against 284.
      tl_variant dd{TL_FAMILY_QGEMM, kDequantDense, 0, 0, 0, 0};
      if (v.p0 == 192 && tl_qgemm_variant_applicable(dd, m, n, k, a_dtype, q)) {
        const int sms = ctx ? ctx->sm_count : 148;
        const double tiles = double((n + kTileRows - 1) / kTileRows) * double((m + 191) / 192);
        const double waves = std::max(1.0, std::ceil(tiles / sms * 4.0) / 4.0);
        const double fused_us = waves * double((k + 127) / 128) * (q.group_size != k ? 1.4 : 0.87);  // group scales: an f32 multiply per weight
        const double dense_us = tl_dense_tc_choose(m, n, k, sms).cost_us + double(n) * double(k) * 3.0 / 4.0e6 + 6.0;
        if (dense_us < 0.92 * fused_us) v = dd;
      }
    }
  } else {
    v.kernel = kSliced;  // f32 activations or odd K: sixteen-row slices through the small-batch kernels
  }
  *out = v;
  return TL_OK;
}

int32_t tl_qgemm_candidates(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc& q,
                            std::vector<tl_variant>* out) {
  tl_variant d;
  tl_qgemm_default_variant(ctx, m, n, k, a_dtype, q, &d);
  out->clear();
  out->push_back(d);
  if (d.kernel == kSliced) return TL_OK;
  {
    tl_variant dd{TL_FAMILY_QGEMM, kDequantDense, 0, 0, 0, 0};
    if (d.kernel != kDequantDense && m >= 256 && tl_qgemm_variant_applicable(dd, m, n, k, a_dtype, q)) out->push_back(dd);
  }
  for (const auto& c : kTcConfigs) {
    if (c.bn < 64 && m > 4 * c.bn) continue;  // narrow token tiles re-stream the weight too often
    tl_variant v{TL_FAMILY_QGEMM, kTc, c.bn, c.kstep, c.stages, c.ncw};
    bool dup = false;
    for (const auto& o : *out) dup = dup || (o.kernel == v.kernel && o.p0 == v.p0 && o.p1 == v.p1 && o.p2 == v.p2 && o.p3 == v.p3);
    if (!dup) out->push_back(v);
  }
  return TL_OK;
}

int32_t tl_launch_qgemm(tl_ctx* ctx, const tl_variant& v, const void* a, int32_t a_dtype, const void* packed,
                        const void* scales, void* out, int32_t out_dtype, int64_t m, int64_t n, int64_t k,
                        const tl_quant_desc& q, const EpiParams& epi, tl_plan_receipt* receipt) {
  if (!tl_qgemm_variant_applicable(v, m, n, k, a_dtype, q))
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "qgemm: variant %s cannot run m=%lld n=%lld k=%lld G=%d %s",
                        tl_variant_name(&v), (long long)m, (long long)n, (long long)k, q.group_size,
                        tl_dtype_name(a_dtype));
  if (v.kernel == kDequantDense) {
    if (receipt) {
      receipt->choice = v;
      const TlDenseTcChoice ch = tl_dense_tc_choose(m, n, k, ctx->sm_count);
      receipt->choice.p0 = ch.bn; receipt->choice.p1 = ch.stages; receipt->choice.p2 = ch.mh;
      receipt->grid[0] = ch.grid; receipt->grid[1] = 1; receipt->grid[2] = 1;
      receipt->block = 576; receipt->split_k = 1;
      return TL_OK;
    }
    if ((reinterpret_cast<uintptr_t>(packed) & 15) || (reinterpret_cast<uintptr_t>(a) & 15))
      return tl_set_error(ctx, TL_ERR_INVALID_ARG, "qgemm: weight and activation pointers must be 16-byte aligned");
    void* wbuf = nullptr;
    int32_t rc = tl_ensure_scratch(ctx, size_t(n) * size_t(k) * 2, &wbuf);
    if (rc != TL_OK) return rc;
    const bool grouped = q.group_size != k;
    const float wscale = q.scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
    const int64_t n_oct = n * k / 8;
    const int grid = int(std::min<int64_t>((n_oct + 1023) / 1024, int64_t(ctx->sm_count) * 8));
    const uint2* pk = static_cast<const uint2*>(packed);
    uint4* wo = static_cast<uint4*>(wbuf);
    const int gpr = int(k / q.group_size);
    if (a_dtype == TL_F16) {
      if (grouped) dequant_int8_16_kernel<__half, true><<<grid, 256, 0, ctx->stream>>>(pk, scales, q.scales_dtype, wscale, q.group_size, gpr, k, n_oct, wo);
      else dequant_int8_16_kernel<__half, false><<<grid, 256, 0, ctx->stream>>>(pk, scales, q.scales_dtype, wscale, q.group_size, gpr, k, n_oct, wo);
    } else {
      if (grouped) dequant_int8_16_kernel<__nv_bfloat16, true><<<grid, 256, 0, ctx->stream>>>(pk, scales, q.scales_dtype, wscale, q.group_size, gpr, k, n_oct, wo);
      else dequant_int8_16_kernel<__nv_bfloat16, false><<<grid, 256, 0, ctx->stream>>>(pk, scales, q.scales_dtype, wscale, q.group_size, gpr, k, n_oct, wo);
    }
    TL_CUDA(ctx, cudaGetLastError());
    ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
    return tl_launch_dense_tc(ctx, a, wbuf, out, m, n, k, a_dtype, out_dtype, epi, grouped ? nullptr : scales, q.scales_dtype, wscale);
  }
  if (v.kernel == kSliced) {
    if (receipt) {
      receipt->choice = v;
      receipt->grid[0] = int32_t((m + 15) / 16); receipt->grid[1] = 1; receipt->grid[2] = 1;
      receipt->block = 0; receipt->split_k = 1;
      return TL_OK;
    }
    for (int64_t m0 = 0; m0 < m; m0 += 16) {
      const int32_t ms = int32_t(std::min<int64_t>(16, m - m0));
      tl_variant gv;
      int32_t rc = tl_qgemv_default_variant(ctx, ms, n, k, a_dtype, q, &gv);
      if (rc != TL_OK) return rc;
      EpiParams e = epi;  // full-size binary operands are indexed by absolute token row: shift them per slice
      const float* shifted[TL_EPI_MAX_INPUTS];
      bool is_binary[TL_EPI_MAX_INPUTS] = {false, false, false, false};
      for (int i = 0; i < e.n_ops; ++i)
        if (e.kind[i] == TL_EPI_BINARY) is_binary[e.idx[i]] = true;
      for (int i = 0; i < TL_EPI_MAX_INPUTS; ++i) {
        shifted[i] = (is_binary[i] && epi.inputs[i]) ? epi.inputs[i] + m0 * n : epi.inputs[i];
        e.inputs[i] = shifted[i];
      }
      rc = tl_launch_qgemv(ctx, gv, reinterpret_cast<const uint8_t*>(a) + size_t(m0) * k * tl_dtype_size(a_dtype),
                           a_dtype, packed, scales,
                           reinterpret_cast<uint8_t*>(out) + size_t(m0) * n * tl_dtype_size(out_dtype), out_dtype, ms, n,
                           k, q, e, nullptr);
      if (rc != TL_OK) return rc;
    }
    return TL_OK;
  }

  const int bn = v.p0, kstep = v.p1;
  GemmArgs p{};
  p.scales = scales; p.out = out; p.m = m; p.n = n; p.k = k;
  p.group = q.group_size; p.groups_per_row = int32_t(k / q.group_size);
  p.scales_dtype = q.scales_dtype; p.out_dtype = out_dtype;
  p.wscale = q.scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
  p.status = ctx->dev_status;
  p.n_tiles = int32_t((n + kTileRows - 1) / kTileRows);
  p.m_tiles = int32_t((m + bn - 1) / bn);
  p.ksteps = int32_t((k + kstep - 1) / kstep);
  const int64_t tiles = int64_t(p.n_tiles) * p.m_tiles;
  // Whole waves run one tile per CTA; the tiles of the last, partial wave are cut along K
  // (at most kMaxSplits ways) so that it still occupies most of the machine.
  constexpr int kMaxSplits = 4;
  const int sms = ctx->sm_count;
  p.full_tiles = int32_t(tiles / sms * sms);
  p.rem_tiles = int32_t(tiles - p.full_tiles);
  p.splits = 1;
  if (p.rem_tiles > 0) {
    int s = std::min<int>({sms / p.rem_tiles, kMaxSplits, p.ksteps});
    while (s > 1 && (s - 1) * ((p.ksteps + s - 1) / s) >= p.ksteps) --s;  // every part gets at least one step
    p.splits = std::max(1, s);
  }
  p.ks_per_split = (p.ksteps + p.splits - 1) / p.splits;
  const int64_t items = int64_t(p.full_tiles) + int64_t(p.rem_tiles) * p.splits;
  const int grid = int(std::min<int64_t>(sms, items));
  if (receipt) {
    receipt->choice = v;
    receipt->grid[0] = grid; receipt->grid[1] = 1; receipt->grid[2] = 1;
    receipt->block = (v.p3 + 10) * 32; receipt->split_k = p.splits;
    return TL_OK;
  }
  if (p.splits > 1) {
    void* slabs = nullptr;
    void* counters = nullptr;
    int32_t rc = tl_ensure_scratch(ctx, size_t(p.rem_tiles) * p.splits * kTileRows * bn * sizeof(float), &slabs);
    if (rc == TL_OK) rc = tl_ensure_zeroed_scratch(ctx, size_t(p.rem_tiles) * sizeof(int), &counters);
    if (rc != TL_OK) return rc;
    p.slabs = static_cast<float*>(slabs);
    p.counters = static_cast<int*>(counters);
  }
  if ((reinterpret_cast<uintptr_t>(packed) & 15) || (reinterpret_cast<uintptr_t>(a) & 15))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "qgemm: weight and activation pointers must be 16-byte aligned");
  CUtensorMap wmap, amap;
  if (!tl_encode_tmap_2d(&wmap, 1, packed, uint64_t(k), uint64_t(n), uint64_t(k), uint32_t(kstep), kTileRows,
                         kstep == 128 ? 3 : 2) ||
      !tl_encode_tmap_2d(&amap, 2, a, uint64_t(k), uint64_t(m), uint64_t(k) * 2, 64, uint32_t(bn), 3))
    return tl_set_error(ctx, TL_ERR_CUDA, "qgemm: cuTensorMapEncodeTiled failed (m=%lld n=%lld k=%lld)", (long long)m,
                        (long long)n, (long long)k);
  const bool grouped = q.group_size != k;
  cudaError_t e = a_dtype == TL_F16 ? launch_tc_cfg<__half>(v, grouped, grid, ctx->stream, wmap, amap, p, epi)
                                    : launch_tc_cfg<__nv_bfloat16>(v, grouped, grid, ctx->stream, wmap, amap, p, epi);
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "qgemm: launch failed: %s", cudaGetErrorString(e));
  }
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

