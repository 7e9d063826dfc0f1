// Dense matmul on the 5th-generation tensor cores: out[m, n] = epilogue(alpha * sum_k A[m, k] * B[n, k])
// with both operands 2-byte (f16 or bf16), K-major, fed by TMA into shared memory and read by
// tcgen05.mma through 128-byte-swizzle descriptors; f32 accumulators in TMEM, double buffered, the
// epilogue written straight from TMEM.  The large-M kernel of tl_matmul; replaces the reference's
// tiled matmul body + epilogue (src/schedule/matmul-skeleton.ts:738-966) for the NT layout that
// `linear` produces and for the other three (an operand stored with k as its slow dimension -- B [K, N],
// A [K, M] -- is staged and multiplied MN-major as it lies, no transposed copy).
//
//   tile: 128 x MH rows of A (tokens, = TMEM lanes; MH = 1 or 2 row halves) x BN rows of B (output columns,
//         = TMEM columns; BN a multiple of 16 up to 256), 64 k per pipeline stage (one 128-byte swizzled row
//         per operand row), 4 MMAs of K = 16 per stage and row half;
//   MH = 1: two accumulators of BN columns, so the epilogue of tile i overlaps the main loop of tile i+1.
//   MH = 2: both row halves multiply the SAME B tile in shared memory.  What paces this kernel is the
//         SM's shared-memory bandwidth (128 bytes per clock), not the tensor pipe: every operand byte is
//         written once by TMA and read once per MMA that uses it, so a 64-k step of a 128 x 256 tile moves
//         2 x (16 + 32) KB = 96 KB = 750 clocks for 512 clocks of MMA (measured 0.424 us per step), and a
//         256 x 256 tile (32 + 32) KB of writes + (32 + 2 x 32) KB of reads = 160 KB for twice the flops
//         (0.742 us) -- 17 % fewer bytes per flop.  (Sharing B between two SMs with cta_group::2 is the
//         step that would take the reads down further; this kernel stays within one CTA.)  The two halves
//         fill TMEM (2 x BN columns), so the epilogue (one warp per lane quarter, half and column half)
//         does not overlap the next tile; it is a few percent when K is in the thousands.
//         The host picks MH and BN from a per-tile time model times the number of waves (tl_dense_tc_choose);
//         (Stages of 32 k -- 64-byte-swizzle rows, seven deep in the same shared memory -- computed the same
//         results 6 to 10 % slower at 256-row tiles.)
//   warp 0: TMA producer (one elected lane); warp 1: TMEM allocation + MMA issue (one elected lane);
//   warps 2..17: epilogue, four warps per TMEM lane quarter (MH = 1: each takes a quarter of the columns;
//         MH = 2: a row half and half of the columns) -- the epilogue is a latency-bound instruction
//         stream, and with K in the low thousands it, not the MMA, paced the tile until it had 16 warps;
//   persistent: one CTA per SM walks the tiles round-robin, row tiles fastest so that CTAs running
//   side by side read the same B rows through L2.
// Ragged edges: TMA zero-fills out-of-range rows and k, stores are masked.
// Every wait is bounded; a wait that runs out raises the context's status word, all roles drain,
// TMEM is released and the kernel returns.
#include <algorithm>
#include <climits>

#include "tl_common.cuh"
#include "tl_tcgen05.cuh"
#include "tl_tma.cuh"

namespace {

constexpr int kDenseThreads = 32 * (2 + 16);  // TMA warp, MMA warp, 16 epilogue warps
constexpr int kBM = 128, kBK = 64;  // kBM: rows per MMA (TMEM lanes); a tile has kBM * MH rows

struct DenseTcArgs {
  void* out;
  int64_t m, n, k;
  int32_t out_dtype;
  int32_t m_tiles, n_tiles, ksteps;
  int* status;
  // optional factor per output column, applied to the accumulator before the op chain (the per-channel
  // scales of a dequantized int8 weight whose 16-bit copy holds q itself): value = colscale[col] * colscale_mul
  const void* colscale;
  int32_t colscale_dtype;
  float colscale_mul;
};

template <typename T> struct OperandFmt;
template <> struct OperandFmt<__half> { static constexpr uint32_t kFmt = 0; };
template <> struct OperandFmt<__nv_bfloat16> { static constexpr uint32_t kFmt = 1; };

// The precise unary ops and the general op chain, out of line (one call per element).
__device__ __noinline__ float dense_unary_outlined(int op, bool approx, float x) { return approx ? tl_unary_approx(op, x) : tl_unary(op, x); }
__device__ __noinline__ float dense_epilogue_outlined(const EpiParams& e, float v, int64_t row, int64_t col, int64_t n) {
  return tl_apply_epilogue(e, v, row, col, n);
}

// MN-major operand descriptor, 128-byte swizzle: the operand is stored [k][n] (n contiguous), staged as
// 64-column slabs of [64 k x 128 bytes]; 8-k groups 1024 bytes apart (stride offset), slabs `slab_bytes`
// apart (leading offset).
__device__ __forceinline__ uint64_t dense_mn_desc(uint32_t smem_addr, uint32_t slab_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr >> 4) & 0x3fffu);
  d |= uint64_t((slab_bytes >> 4) & 0x3fffu) << 16;
  d |= uint64_t((1024 >> 4) & 0x3fff) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

// BMN = 1: B is stored [K, N] (the NN layout of matmul(a, b)); its tiles are staged and multiplied MN-major,
// so no transposed copy of B is made.  BN must then be a multiple of 64.  AMN = 1: the same for an A stored
// [K, M] (a transposed view of the first operand).
template <typename AT, int BN, int STAGES, int MH, int BMN, int AMN>
__global__ void __launch_bounds__(kDenseThreads, 1)
dense_tc_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, DenseTcArgs p, EpiParams epi) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "MMA N");
  static_assert(MH == 1 || MH == 2, "row halves");
  constexpr int kTileM = kBM * MH, kAcc = MH == 1 ? 2 : 1;  // accumulator sets in TMEM (each MH x BN columns)
  constexpr int kABytes = kTileM * 128, kBBytes = BN * 128, kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  constexpr int kEpiWarp0 = 2, kEpiWarps = 16;
  static_assert(BMN == 0 || BN % 64 == 0, "MN-major B is staged in 64-column slabs");
  constexpr uint32_t kIdesc = (1u << 4) | (OperandFmt<AT>::kFmt << 7) | (OperandFmt<AT>::kFmt << 10) | (uint32_t(AMN) << 15) | (uint32_t(BMN) << 16) |
                              (uint32_t(BN >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
  constexpr int kSlabBytes = kBK * 128;  // one 64-column slab of an MN-major B stage

  extern __shared__ uint8_t dense_smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dense_smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], kEpiWarps);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&amap);
      tma_prefetch_desc(&bmap);
      int it = 0;
      for (int t = blockIdx.x; t < tiles && !abort_flag; t += gridDim.x) {
        const int n_tile = t / p.m_tiles, m_tile = t - n_tile * p.m_tiles;
        for (int ks = 0; ks < p.ksteps; ++ks, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1, &abort_flag)) {
            if (!abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_EMPTY); }
            break;
          }
          uint8_t* st = stages + size_t(s) * kStageBytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          if (AMN) {
#pragma unroll
            for (int sl = 0; sl < kTileM / 64; ++sl)
              tma_load_2d(st + sl * kSlabBytes, &amap, m_tile * kTileM + sl * 64, ks * kBK, &full_bar[s]);
          } else {
            tma_load_2d(st, &amap, ks * kBK, m_tile * kTileM, &full_bar[s]);
          }
          if (BMN) {
#pragma unroll
            for (int sl = 0; sl < BN / 64; ++sl)
              tma_load_2d(st + kABytes + sl * kSlabBytes, &bmap, n_tile * BN + sl * 64, ks * kBK, &full_bar[s]);
          } else {
            tma_load_2d(st + kABytes, &bmap, ks * kBK, n_tile * BN, &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int it = 0, tl = 0;
      for (int t = blockIdx.x; t < tiles && !abort_flag; t += gridDim.x, ++tl) {
        const int acc = tl % kAcc, use = tl / kAcc;
        if (use >= 1 && !mbar_wait(&tempty_bar[acc], (use - 1) & 1, &abort_flag)) {
          if (!abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_TMEM); }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * MH * BN);
        bool ok = true;
        for (int ks = 0; ks < p.ksteps; ++ks, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, &abort_flag)) {
            if (!abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_FULL); }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(stages + size_t(s) * kStageBytes);
          const uint32_t b_base = a_base + kABytes;
#pragma unroll
          for (int h = 0; h < MH; ++h)
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk)
              tc_mma_ss(d_tmem + uint32_t(h * BN),
                        AMN ? dense_mn_desc(a_base + h * (kBM * 128) + kk * 2048, kSlabBytes) : make_b_desc(a_base + h * (kBM * 128) + kk * 32),
                        BMN ? dense_mn_desc(b_base + kk * 2048, kSlabBytes) : make_b_desc(b_base + kk * 32), kIdesc,
                        (ks > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // Four warps per TMEM lane quarter.  Everything per chunk stays in registers: the loops are fully
    // unrolled, the op chain is decoded once per kernel into `mode`, and the general chain is an
    // out-of-line call per element (it is the rare case; inlined 16 times it would evict the hot loop).
    constexpr int kColParts = (kEpiWarps / 4) / MH;
    const int quad = warp & 3, part = (warp - kEpiWarp0) >> 2;
    const int ehalf = MH == 2 ? part / kColParts : 0, cpart = MH == 2 ? part % kColParts : part;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    constexpr int kChunksN = BN / 16;
    const int cbeg = cpart * kChunksN / kColParts, cend = (cpart + 1) * kChunksN / kColParts;
    const bool approx = p.out_dtype != TL_F32;
    enum { kPlain, kGelu, kRelu, kSilu, kUnary, kGeneric };
    const int fu = epi.fast_unary;
    const int mode = !epi.fast ? kGeneric
                   : fu == 0 ? kPlain
                   : (approx && fu == TL_UNARY_GELU_TANH) ? kGelu
                   : fu == TL_UNARY_RELU ? kRelu
                   : (approx && fu == TL_UNARY_SILU) ? kSilu : kUnary;
    const float* bias = epi.fast ? epi.fast_bias : nullptr;
    const float alpha = epi.alpha;
    const int esz = p.out_dtype == TL_F32 ? 4 : 2;
    const bool vec_ok = (p.n * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    int tl = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tl) {
      const int acc = tl % kAcc;
      const int n_tile = t / p.m_tiles, m_tile = t - n_tile * p.m_tiles;
      const int64_t row = int64_t(m_tile) * kTileM + ehalf * kBM + quad * 32 + lane;  // this thread's output row
      const bool row_ok = row < p.m;
      const uint32_t acc_col = uint32_t(acc * MH * BN + ehalf * BN);
      if (!mbar_wait(&tfull_bar[acc], (tl / kAcc) & 1, &abort_flag)) {
        if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_TMEM); }
        break;
      }
      tc_fence_after();
      uint32_t vn[16];
      if (cbeg < cend) tmem_ld16(tmem_base + lane_addr + acc_col + uint32_t(cbeg * 16), vn);
#pragma unroll 1
      for (int ch = cbeg; ch < cend; ++ch) {
        const int64_t col0 = int64_t(n_tile) * BN + ch * 16;
        float o[16];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] = __uint_as_float(vn[j]);
        if (ch + 1 < cend) tmem_ld16(tmem_base + lane_addr + acc_col + uint32_t((ch + 1) * 16), vn);  // next chunk in flight
        if (!row_ok || col0 >= p.n) continue;
        const int jmax = int(min(int64_t(16), p.n - col0));
        if (p.colscale) {
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] *= j < jmax ? tl_load_scale(p.colscale, p.colscale_dtype, col0 + j) * p.colscale_mul : 0.f;
        }
        if (mode != kGeneric) {
          if (bias) {
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = fmaf(o[j], alpha, j < jmax ? __ldg(bias + col0 + j) : 0.f);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] *= alpha;
          }
          if (mode == kGelu) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              o[j] = (0.5f * o[j]) * (1.f + tl_tanh_approx(0.7978845608f * (o[j] + 0.044715f * (o[j] * (o[j] * o[j])))));
          } else if (mode == kRelu) {
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = fmaxf(o[j], 0.f);
          } else if (mode == kSilu) {
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __fdividef(o[j], 1.f + __expf(-o[j]));
          } else if (mode == kUnary) {
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = dense_unary_outlined(fu, approx, o[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < jmax) o[j] = dense_epilogue_outlined(epi, o[j], row, col0 + j, p.n);
        }
        uint8_t* optr = reinterpret_cast<uint8_t*>(p.out) + (row * p.n + col0) * esz;
        if (jmax == 16 && vec_ok) {
          if (p.out_dtype == TL_F32) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              reinterpret_cast<float4*>(optr)[q4] = make_float4(o[4 * q4], o[4 * q4 + 1], o[4 * q4 + 2], o[4 * q4 + 3]);
          } else {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (p.out_dtype == TL_F16) {
                const __half2 h = __floats2half2_rn(o[2 * j], o[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
              } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
              }
            }
            reinterpret_cast<uint4*>(optr)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(optr)[1] = make_uint4(w[4], w[5], w[6], w[7]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < jmax) tl_store_out(p.out, p.out_dtype, row * p.n + col0 + j, o[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename AT, int BN, int STAGES, int MH, int BMN = 0, int AMN = 0>
cudaError_t launch_dense(int grid, cudaStream_t s, const CUtensorMap& amap, const CUtensorMap& bmap, const DenseTcArgs& p,
                         const EpiParams& e) {
  constexpr size_t smem = size_t(STAGES) * (kBM * MH * 128 + BN * 128) + 1024;
  static_assert(smem <= 227 * 1024, "shared memory per CTA");
  auto kern = dense_tc_kernel<AT, BN, STAGES, MH, BMN, AMN>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  kern<<<grid, kDenseThreads, smem, s>>>(amap, bmap, p, e);
  return cudaGetLastError();
}

}  // namespace

bool tl_dense_tc_applicable(const void* a, const void* b, int64_t m, int64_t n, int64_t k, int32_t dtype_a, int32_t dtype_b) {
  if (dtype_a != dtype_b || (dtype_a != TL_F16 && dtype_a != TL_BF16)) return false;
  if (m < 32 || n < 64 || k < 64 || k % 8 != 0) return false;  // TMA row pitch must be a multiple of 16 bytes
  if (a && (reinterpret_cast<uintptr_t>(a) & 15)) return false;
  if (b && (reinterpret_cast<uintptr_t>(b) & 15)) return false;
  return true;
}

// p0 of the receipt: BN (columns per tile); p1: stages; p2: MH (row halves per tile).  The choice minimises
// waves x tile time, waves = ceil(tiles / SMs), with the tile time taken from measurements on B200 (bf16,
// shapes from 1024^3 to 8192^3): a 64-k step costs `step_us` whatever the shape -- it follows the bytes the
// step moves through shared memory (TMA writes + MMA reads, at about 226 KB per us), not the MMA's clocks,
// which is why 256-row tiles win on large shapes (0.742 us for 256 x 256 against 2 x 0.424 for 128 x 256);
// the three-stage tiles run a little under that rate, which is why four stages (BN <= 192 at
// MH = 2) beat three.  With MH = 1 the epilogue hides behind the next tile unless K is short; with MH = 2
// it adds to every tile.  E.g. m = 2048, n = 14336, k = 4096 on 148 SMs: 128 x 224 tiles run 7 waves of
// 27 us, 256 x 208 tiles 4 waves of 46 us.
namespace {
struct DenseCfg { int mh, bn, stages; float step_us; };
constexpr DenseCfg kDenseCfgs[] = {{1, 256, 4, 0.424f}, {1, 224, 5, 0.410f}, {1, 192, 5, 0.373f}, {1, 160, 6, 0.358f},
                                   {1, 128, 6, 0.348f}, {2, 256, 3, 0.742f}, {2, 240, 3, 0.734f}, {2, 224, 3, 0.700f},
                                   {2, 208, 3, 0.684f}, {2, 192, 4, 0.580f}, {2, 176, 4, 0.586f}, {2, 160, 4, 0.583f}};
}  // namespace

TlDenseTcChoice tl_dense_tc_choose(int64_t m, int64_t n, int64_t k, int sms, int forced_bn, int forced_mh, int bn_multiple) {
  const int64_t ksteps = (k + kBK - 1) / kBK;
  TlDenseTcChoice best{128, 1, 6, 1, 1e300};
  for (const DenseCfg& c : kDenseCfgs) {
    if (c.bn % bn_multiple != 0) continue;  // an MN-major operand is staged in 64-column slabs
    if (forced_bn > 0) {
      if (c.bn != forced_bn || c.mh != (forced_mh == 2 ? 2 : 1)) continue;
    } else {
      if (c.bn > 128 && n < c.bn) continue;
      if (c.mh == 2 && m <= kBM) continue;
    }
    const int64_t t = ((m + kBM * c.mh - 1) / (kBM * c.mh)) * ((n + c.bn - 1) / c.bn);
    const double main_us = double(ksteps) * c.step_us;
    const double tile = c.mh == 1 ? std::max(main_us, 0.012 * c.bn + 0.5) + 0.3 : main_us + 0.0094 * c.bn + 0.5;
    const double cost = double((t + sms - 1) / sms) * tile;
    if (cost < best.cost_us) best = TlDenseTcChoice{c.bn, c.mh, c.stages, int(std::min<int64_t>(sms, t)), cost};
  }
  return best;
}

int32_t tl_launch_dense_tc(tl_ctx* ctx, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int32_t dtype,
                           int32_t out_dtype, const EpiParams& epi, const void* colscale, int32_t colscale_dtype, float colscale_mul,
                           bool b_mn, bool a_mn) {
  const bool forced = ctx->has_forced && ctx->forced.family == TL_FAMILY_MATMUL && ctx->forced.kernel == 2 && ctx->forced.p0 > 0;
  const TlDenseTcChoice ch = tl_dense_tc_choose(m, n, k, ctx->sm_count, forced ? ctx->forced.p0 : 0, forced ? ctx->forced.p2 : 0,
                                                (b_mn || a_mn) ? 64 : 16);
  const int bn = ch.bn, mh = ch.mh, grid = ch.grid;
  if (forced && (bn != ctx->forced.p0 || mh != (ctx->forced.p2 == 2 ? 2 : 1)))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_matmul: no tensor-core tile with BN=%d MH=%d", ctx->forced.p0, ctx->forced.p2);
  const int tile_m = kBM * mh;
  DenseTcArgs p{};
  p.out = out; p.m = m; p.n = n; p.k = k; p.out_dtype = out_dtype;
  p.m_tiles = int32_t((m + tile_m - 1) / tile_m);
  p.n_tiles = int32_t((n + bn - 1) / bn);
  p.ksteps = int32_t((k + kBK - 1) / kBK);
  p.status = ctx->dev_status;
  p.colscale = colscale; p.colscale_dtype = colscale_dtype; p.colscale_mul = colscale_mul;
  CUtensorMap amap, bmap;
  if (!(a_mn ? tl_encode_tmap_2d(&amap, 2, a, uint64_t(m), uint64_t(k), uint64_t(m) * 2, 64, kBK, 3)  // a stored [K, M]
             : tl_encode_tmap_2d(&amap, 2, a, uint64_t(k), uint64_t(m), uint64_t(k) * 2, kBK, uint32_t(tile_m), 3)) ||
      !(b_mn ? tl_encode_tmap_2d(&bmap, 2, b, uint64_t(n), uint64_t(k), uint64_t(n) * 2, 64, kBK, 3)  // b stored [K, N]: 64 columns x 64 k per box
             : tl_encode_tmap_2d(&bmap, 2, b, uint64_t(k), uint64_t(n), uint64_t(k) * 2, kBK, uint32_t(bn), 3)))
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_matmul: cuTensorMapEncodeTiled failed (m=%lld n=%lld k=%lld)", (long long)m,
                        (long long)n, (long long)k);
  cudaError_t e = cudaErrorInvalidValue;
#define TL_DENSE_CASE(MH_, BN_, ST_)                                                                          \
  if (mh == MH_ && bn == BN_)                                                                                \
    e = dtype == TL_F16 ? launch_dense<__half, BN_, ST_, MH_>(grid, ctx->stream, amap, bmap, p, epi)         \
                        : launch_dense<__nv_bfloat16, BN_, ST_, MH_>(grid, ctx->stream, amap, bmap, p, epi);
  if (b_mn || a_mn) {
#define TL_DENSE_MN_CASE(MH_, BN_, ST_)                                                                                  \
  if (mh == MH_ && bn == BN_) {                                                                                         \
    if (a_mn && b_mn)                                                                                                   \
      e = dtype == TL_F16 ? launch_dense<__half, BN_, ST_, MH_, 1, 1>(grid, ctx->stream, amap, bmap, p, epi)            \
                          : launch_dense<__nv_bfloat16, BN_, ST_, MH_, 1, 1>(grid, ctx->stream, amap, bmap, p, epi);    \
    else if (a_mn)                                                                                                      \
      e = dtype == TL_F16 ? launch_dense<__half, BN_, ST_, MH_, 0, 1>(grid, ctx->stream, amap, bmap, p, epi)            \
                          : launch_dense<__nv_bfloat16, BN_, ST_, MH_, 0, 1>(grid, ctx->stream, amap, bmap, p, epi);    \
    else                                                                                                                \
      e = dtype == TL_F16 ? launch_dense<__half, BN_, ST_, MH_, 1, 0>(grid, ctx->stream, amap, bmap, p, epi)            \
                          : launch_dense<__nv_bfloat16, BN_, ST_, MH_, 1, 0>(grid, ctx->stream, amap, bmap, p, epi);    \
  }
    TL_DENSE_MN_CASE(1, 256, 4)
    TL_DENSE_MN_CASE(1, 192, 5)
    TL_DENSE_MN_CASE(1, 128, 6)
    TL_DENSE_MN_CASE(2, 256, 3)
    TL_DENSE_MN_CASE(2, 192, 4)
#undef TL_DENSE_MN_CASE
  } else {
  TL_DENSE_CASE(1, 256, 4)
  TL_DENSE_CASE(1, 224, 5)
  TL_DENSE_CASE(1, 192, 5)
  TL_DENSE_CASE(1, 160, 6)
  TL_DENSE_CASE(1, 128, 6)
  TL_DENSE_CASE(2, 256, 3)
  TL_DENSE_CASE(2, 240, 3)
  TL_DENSE_CASE(2, 224, 3)
  TL_DENSE_CASE(2, 208, 3)
  TL_DENSE_CASE(2, 192, 4)
  TL_DENSE_CASE(2, 176, 4)
  TL_DENSE_CASE(2, 160, 4)
  }
#undef TL_DENSE_CASE
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_matmul: tensor-core launch failed: %s", cudaGetErrorString(e));
  }
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}
