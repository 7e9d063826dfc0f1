// Dense matmul on the 5th-generation tensor cores: out[m, n] = epilogue(alpha * sum_k A[m, k] * B[n, k])
// with both operands 2-byte (f16 or bf16), K-major, fed by TMA into shared memory and read by
// tcgen05.mma through 128-byte-swizzle descriptors; f32 accumulators in TMEM, double buffered, the
// epilogue written straight from TMEM.  The large-M kernel of tl_matmul; replaces the reference's
// tiled matmul body + epilogue (src/schedule/matmul-skeleton.ts:738-966) for the NT layout that
// `linear` produces (other layouts are brought to it by one transposition pass, see tl_matmul).
//
//   tile: 128 rows of A (tokens, = TMEM lanes) x BN rows of B (output columns, = TMEM columns; BN is 128,
//         160, 192, 224 or 256, whichever leaves the fewest idle SMs in the last wave),
//         64 k per pipeline stage (one 128-byte swizzled row per operand row), 4 MMAs of K = 16 per stage;
//   warp 0: TMA producer (one elected lane); warp 1: TMEM allocation + MMA issue (one elected lane);
//   warps 2..9: epilogue, two warps per TMEM lane quarter, each taking half of the tile's columns;
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

constexpr int kBM = 128, kBK = 64;

struct DenseTcArgs {
  void* out;
  int64_t m, n, k;
  int32_t out_dtype;
  int32_t m_tiles, n_tiles, ksteps;
  int* status;
};

template <typename T> struct OperandFmt;
template <> struct OperandFmt<__half> { static constexpr uint32_t kFmt = 0; };
template <> struct OperandFmt<__nv_bfloat16> { static constexpr uint32_t kFmt = 1; };

template <typename AT, int BN, int STAGES>
__global__ void __launch_bounds__(320, 1)
dense_tc_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, DenseTcArgs p, EpiParams epi) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "MMA N");
  constexpr int kABytes = kBM * 128, kBBytes = BN * 128, kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  constexpr int kEpiWarp0 = 2, kEpiWarps = 8;
  constexpr uint32_t kIdesc = (1u << 4) | (OperandFmt<AT>::kFmt << 7) | (OperandFmt<AT>::kFmt << 10) | (uint32_t(BN >> 3) << 17) |
                              (uint32_t(kBM >> 4) << 24);

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
          tma_load_2d(st, &amap, ks * kBK, m_tile * kBM, &full_bar[s]);
          tma_load_2d(st + kABytes, &bmap, ks * kBK, n_tile * BN, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int it = 0, tl = 0;
      for (int t = blockIdx.x; t < tiles && !abort_flag; t += gridDim.x, ++tl) {
        const int acc = tl & 1;
        if (tl >= 2 && !mbar_wait(&tempty_bar[acc], ((tl >> 1) - 1) & 1, &abort_flag)) {
          if (!abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_TMEM); }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
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
          for (int kk = 0; kk < kBK / 16; ++kk)
            tc_mma_ss(d_tmem, make_b_desc(a_base + kk * 32), make_b_desc(b_base + kk * 32), kIdesc, (ks > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3, ehalf = (warp - kEpiWarp0) >> 2;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    constexpr int kChunksN = BN / 16;
    const int cbeg = ehalf == 0 ? 0 : (kChunksN + 1) / 2, cend = ehalf == 0 ? (kChunksN + 1) / 2 : kChunksN;
    const bool fast = epi.fast != 0, approx = p.out_dtype != TL_F32;
    const int esz = p.out_dtype == TL_F32 ? 4 : 2;
    const bool vec_ok = (p.n * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    int tl = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tl) {
      const int acc = tl & 1;
      const int n_tile = t / p.m_tiles, m_tile = t - n_tile * p.m_tiles;
      const int64_t row = int64_t(m_tile) * kBM + quad * 32 + lane;  // this thread's output row
      const bool row_ok = row < p.m;
      if (!mbar_wait(&tfull_bar[acc], (tl >> 1) & 1, &abort_flag)) {
        if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_TMEM); }
        break;
      }
      tc_fence_after();
      uint32_t vn[16];
      if (cbeg < cend) tmem_ld16(tmem_base + lane_addr + uint32_t(acc * BN + cbeg * 16), vn);
#pragma unroll 1
      for (int ch = cbeg; ch < cend; ++ch) {
        const int64_t col0 = int64_t(n_tile) * BN + ch * 16;
        uint32_t v[16];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = vn[j];
        if (ch + 1 < cend) tmem_ld16(tmem_base + lane_addr + uint32_t(acc * BN + (ch + 1) * 16), vn);  // next chunk in flight
        if (!row_ok || col0 >= p.n) continue;
        float o[16];
        const int jmax = int(min(int64_t(16), p.n - col0));
        if (fast) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float b = (epi.fast_bias && j < jmax) ? __ldg(epi.fast_bias + col0 + j) : 0.f;
            o[j] = fmaf(__uint_as_float(v[j]), epi.alpha, b);
            if (epi.fast_unary) o[j] = approx ? tl_unary_approx(epi.fast_unary, o[j]) : tl_unary(epi.fast_unary, o[j]);
          }
        } else {
#pragma unroll 1
          for (int j = 0; j < jmax; ++j) o[j] = tl_apply_epilogue(epi, __uint_as_float(v[j]), row, col0 + j, p.n);
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
#pragma unroll 1
          for (int j = 0; j < jmax; ++j) tl_store_out(p.out, p.out_dtype, row * p.n + col0 + j, o[j]);
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

template <typename AT, int BN, int STAGES>
cudaError_t launch_dense(int grid, cudaStream_t s, const CUtensorMap& amap, const CUtensorMap& bmap, const DenseTcArgs& p,
                         const EpiParams& e) {
  constexpr size_t smem = size_t(STAGES) * (kBM * 128 + BN * 128) + 1024;
  auto kern = dense_tc_kernel<AT, BN, STAGES>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  kern<<<grid, 320, smem, s>>>(amap, bmap, p, e);
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

// p0 of the receipt: BN (columns per tile); p1: stages.  A tile's time grows with BN (the MMA is the
// long pole), so the cost of a choice is waves x BN with waves = ceil(tiles / SMs): e.g. n = 14336,
// m = 2048 on 148 SMs is 7 waves at BN = 256 but also 7 waves at BN = 224 (6.92 full), 12 % less work.
void tl_dense_tc_shape(int64_t m, int64_t n, int sms, int* bn, int* stages, int* grid) {
  const int64_t m_tiles = (m + kBM - 1) / kBM;
  int64_t best_cost = INT64_MAX;
  int best = 128;
  for (int b : {256, 224, 192, 160, 128}) {
    if (b > 128 && n < b) continue;
    const int64_t t = m_tiles * ((n + b - 1) / b);
    const int64_t cost = ((t + sms - 1) / sms) * b;
    if (cost < best_cost) { best_cost = cost; best = b; }
  }
  *bn = best;
  *stages = best == 256 ? 4 : best >= 192 ? 5 : 6;
  const int64_t t = m_tiles * ((n + best - 1) / best);
  *grid = int(std::min<int64_t>(sms, t));
}

int32_t tl_launch_dense_tc(tl_ctx* ctx, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int32_t dtype,
                           int32_t out_dtype, const EpiParams& epi) {
  int bn, stages, grid;
  tl_dense_tc_shape(m, n, ctx->sm_count, &bn, &stages, &grid);
  DenseTcArgs p{};
  p.out = out; p.m = m; p.n = n; p.k = k; p.out_dtype = out_dtype;
  p.m_tiles = int32_t((m + kBM - 1) / kBM);
  p.n_tiles = int32_t((n + bn - 1) / bn);
  p.ksteps = int32_t((k + kBK - 1) / kBK);
  p.status = ctx->dev_status;
  CUtensorMap amap, bmap;
  if (!tl_encode_tmap_2d(&amap, 2, a, uint64_t(k), uint64_t(m), uint64_t(k) * 2, kBK, kBM, 3) ||
      !tl_encode_tmap_2d(&bmap, 2, b, uint64_t(k), uint64_t(n), uint64_t(k) * 2, kBK, uint32_t(bn), 3))
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_matmul: cuTensorMapEncodeTiled failed (m=%lld n=%lld k=%lld)", (long long)m,
                        (long long)n, (long long)k);
  cudaError_t e = cudaErrorInvalidValue;
#define TL_DENSE_CASE(BN_, ST_)                                                                              \
  if (bn == BN_)                                                                                             \
    e = dtype == TL_F16 ? launch_dense<__half, BN_, ST_>(grid, ctx->stream, amap, bmap, p, epi)              \
                        : launch_dense<__nv_bfloat16, BN_, ST_>(grid, ctx->stream, amap, bmap, p, epi);
  TL_DENSE_CASE(256, 4)
  TL_DENSE_CASE(224, 5)
  TL_DENSE_CASE(192, 5)
  TL_DENSE_CASE(160, 6)
  TL_DENSE_CASE(128, 6)
#undef TL_DENSE_CASE
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_matmul: tensor-core launch failed: %s", cudaGetErrorString(e));
  }
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}
