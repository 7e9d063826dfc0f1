// Dense (unquantized) matmul behind the same epilogue seam: out = epi(alpha * op(A) . op(B)).
// Replaces dispatchTiledMatmul and the dense GEMV builders of the reference
// (src/backend/webgpu/matmul/dispatch.ts:1331, src/backend/webgpu/matmul/gemv.ts:430-532,
// tiled body src/schedule/matmul-skeleton.ts:738-908, read-wider-cast-on-load
// src/backend/webgpu/matmul/variants.ts:170-175, batch broadcast strides dispatch.ts:1411-1510).
//
// Three kernels of family TL_FAMILY_MATMUL:
//   0 "tiled"  the always-applicable one (the reference's `tiled` variant): 64 x 64 output tiles,
//              16 x 16 threads with 4 x 4 register tiles, operands staged through shared memory
//              16 k at a time, any of NN / NT / TN / TT, f32 / f16 / bf16 operands in any
//              combination (widened exactly to f32, optionally rounded through a narrower type
//              first: the cast prologue), batched with broadcast strides, ragged edges masked,
//              f32 accumulation in ascending k.
//   1 "gemv"   m <= 16, B stored [N, K] (transB), both operands the same 2-byte type, one batch:
//              the small-batch tensor-core tile of the quantized path without the converter --
//              16 rows per CTA, warps interleaved over 32-wide k blocks, mma.sync.m16n8k16 with the
//              weight rows as the A operand and the batch as the B operand.  HBM-bound.
//   2 "tc"     m >= 32, n >= 64, k >= 64, k % 8 == 0, both operands f16 or both bf16, no cast prologue: the
//              tcgen05 kernel of tl_matmul_tc.cu.  It computes the NT layout; an A stored [K, M] or a
//              B stored [K, N] is first transposed into library scratch (one extra HBM pass over
//              that operand).  Batches run as one launch each.
#include <algorithm>

#include "tl_common.cuh"
#include "tl_mma_frag.cuh"

namespace {

constexpr int kTiled = 0, kGemv = 1, kTc = 2;

struct MatmulArgs {
  const void* a;
  const void* b;
  void* out;
  int32_t m, n, k, batch;
  int64_t stride_a, stride_b, stride_c;  // elements between batches (0 = broadcast)
  int32_t trans_a, trans_b;              // A stored [K, M] / B stored [N, K]
  int32_t dtype_a, dtype_b, out_dtype;
  int32_t cast_a, cast_b;                // -1, or the type the operand is rounded through on load
};

__device__ __forceinline__ float load_elem(const void* base, int dtype, int64_t idx, int cast) {
  float v;
  if (dtype == TL_F32) v = reinterpret_cast<const float*>(base)[idx];
  else if (dtype == TL_F16) v = __half2float(reinterpret_cast<const __half*>(base)[idx]);
  else v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  if (cast == TL_F16) v = __half2float(__float2half_rn(v));
  else if (cast == TL_BF16) v = __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

// ---------------------------------------------------------------------------
// 0: tiled
// ---------------------------------------------------------------------------
constexpr int kTM = 64, kTN = 64, kTK = 16;

__global__ void __launch_bounds__(256) matmul_tiled_kernel(MatmulArgs p, EpiParams epi) {
  __shared__ float sa[kTK][kTM + 4];
  __shared__ float sb[kTK][kTN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t row0 = int64_t(blockIdx.y) * kTM, col0 = int64_t(blockIdx.x) * kTN;
  const int bz = blockIdx.z;
  const uint8_t* a = reinterpret_cast<const uint8_t*>(p.a) + size_t(bz) * p.stride_a * (p.dtype_a == TL_F32 ? 4 : 2);
  const uint8_t* b = reinterpret_cast<const uint8_t*>(p.b) + size_t(bz) * p.stride_b * (p.dtype_b == TL_F32 ? 4 : 2);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < p.k; k0 += kTK) {
    // stage A [kTK x kTM] and B [kTK x kTN]; the thread -> element map follows the operand's
    // contiguous dimension so that the loads coalesce for either storage order
    for (int e = threadIdx.x; e < kTK * kTM; e += 256) {
      int kk, mm;
      if (p.trans_a) { mm = e % kTM; kk = e / kTM; } else { kk = e % kTK; mm = e / kTK; }
      const int64_t gr = row0 + mm, gk = k0 + kk;
      float v = 0.f;
      if (gr < p.m && gk < p.k) v = load_elem(a, p.dtype_a, p.trans_a ? gk * p.m + gr : gr * p.k + gk, p.cast_a);
      sa[kk][mm] = v;
    }
    for (int e = threadIdx.x; e < kTK * kTN; e += 256) {
      int kk, nn;
      if (p.trans_b) { kk = e % kTK; nn = e / kTK; } else { nn = e % kTN; kk = e / kTN; }
      const int64_t gc = col0 + nn, gk = k0 + kk;
      float v = 0.f;
      if (gc < p.n && gk < p.k) v = load_elem(b, p.dtype_b, p.trans_b ? gc * p.k + gk : gk * p.n + gc, p.cast_b);
      sb[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  uint8_t* out = reinterpret_cast<uint8_t*>(p.out) + size_t(bz) * p.stride_c * (p.out_dtype == TL_F32 ? 4 : 2);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t row = row0 + ty * 4 + i;
    if (row >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t col = col0 + tx * 4 + j;
      if (col >= p.n) continue;
      const float r = tl_apply_epilogue(epi, acc[i][j], row, col, p.n);
      tl_store_out(out, p.out_dtype, row * p.n + col, r);
    }
  }
}

// ---------------------------------------------------------------------------
// 1: dense small-batch GEMV (NT).  Thread (g, t) of a warp loads 16 bytes = 8 consecutive k of
// weight rows g and g+8 and of batch row g; words (0,1) of the chunk feed one MMA's k slots
// (2t,2t+1) and (2t+8,2t+9), words (2,3) the next MMA's -- the same permutation on both operands.
// ---------------------------------------------------------------------------
template <typename AT, int NT>
__global__ void __launch_bounds__(512) dense_gemv_kernel(MatmulArgs p, EpiParams epi) {
  extern __shared__ float red[];  // [warps][NT][4][32]
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t tile_row = int64_t(blockIdx.x) * 16;
  const int64_t r_lo = min(tile_row + g, int64_t(p.n) - 1), r_hi = min(tile_row + g + 8, int64_t(p.n) - 1);
  const AT* w = reinterpret_cast<const AT*>(p.b);
  const AT* x = reinterpret_cast<const AT*>(p.a);
  const AT* w_lo = w + r_lo * p.k + 8 * t;
  const AT* w_hi = w + r_hi * p.k + 8 * t;
  const AT* x_col[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) x_col[nt] = x + int64_t(min(g + 8 * nt, p.m - 1)) * p.k + 8 * t;
  float c[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) c[nt][e] = 0.f;
  const int kblocks = p.k >> 5;  // 32 k per block
  // (Requesting four blocks' weights before using the first measured SLOWER, 33.7 vs 29.3 us on
  // 4096 x 14336: the extra registers cost a resident CTA.  So did a per-thread cp.async ring of 8
  // slots: 28.9 us at m = 1, 46-49 us at m = 8 and 16, where the activation loads then wait behind
  // the ring's wait_group.)
  for (int kb = warp; kb < kblocks; kb += warps) {
    const uint4 wl = __ldg(reinterpret_cast<const uint4*>(w_lo + kb * 32));
    const uint4 wh = __ldg(reinterpret_cast<const uint4*>(w_hi + kb * 32));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x_col[nt] + kb * 32));
      MmaOps<AT>::mma(c[nt], wl.x, wh.x, wl.y, wh.y, xv.x, xv.y);
      MmaOps<AT>::mma(c[nt], wl.z, wh.z, wl.w, wh.w, xv.z, xv.w);
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[((warp * NT + nt) * 4 + e) * 32 + lane] = c[nt][e];
  __syncthreads();
  for (int o = threadIdx.x; o < NT * 128; o += blockDim.x) {
    const int nt = o >> 7, e = (o >> 5) & 3, ln = o & 31;
    float v = 0.f;
    for (int ww = 0; ww < warps; ++ww) v += red[((ww * NT + nt) * 4 + e) * 32 + ln];
    const int64_t row = tile_row + (ln >> 2) + ((e & 2) ? 8 : 0);  // weight row = output column
    const int col = 8 * nt + 2 * (ln & 3) + (e & 1);               // batch row
    if (row < p.n && col < p.m) {
      const float r = tl_apply_epilogue(epi, v, col, row, p.n);
      tl_store_out(p.out, p.out_dtype, int64_t(col) * p.n + row, r);
    }
  }
}

// Which operands the tensor-core kernel multiplies MN-major as they are stored (no transposed copy): a B
// stored [K, N], an A stored [K, M], when the row pitch allows a TMA map (a multiple of 16 bytes) and the
// 64-column tiles that form needs are not wasted on a narrow output.
void dense_mn_operands(bool trans_a, bool trans_b, int64_t m, int64_t n, bool* a_mn, bool* b_mn) {
  *b_mn = !trans_b && n % 8 == 0 && n >= 128;
  *a_mn = trans_a && m % 8 == 0 && n >= 128;
}

bool gemv_applicable(const MatmulArgs& p, const EpiParams& epi) {
  // dense GEMV: m <= 16, one batch, B stored [N, K], same 2-byte operand type, no cast prologue,
  // epilogue of bias / unary ops only (gemv.ts:135-159), vector loads need k % 32 == 0 and alignment
  if (p.m < 1 || p.m > 16 || p.batch != 1 || !p.trans_b || p.trans_a) return false;
  if (p.dtype_a != p.dtype_b || (p.dtype_a != TL_F16 && p.dtype_a != TL_BF16) || p.cast_a >= 0 || p.cast_b >= 0) return false;
  if (p.k % 32 != 0 || p.k < 32) return false;
  if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15)) return false;
  (void)epi;  // every epilogue op runs in the GEMV's store loop (a superset of gemv.ts:135-159)
  return true;
}

}  // namespace

extern "C" int32_t tl_matmul(tl_ctx* ctx, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int64_t batch,
                             int64_t stride_a, int64_t stride_b, int64_t stride_c, int32_t trans_a, int32_t trans_b, float alpha,
                             int32_t dtype_a, int32_t dtype_b, int32_t out_dtype, int32_t cast_a, int32_t cast_b,
                             const tl_epilogue* epilogue, tl_plan_receipt* receipt_only) {
  TL_CHECK_CTX(ctx);
  TlProfileScope prof(receipt_only ? nullptr : ctx, "matmul", m, n, k);
  if (!receipt_only && (!a || !b || !out)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_matmul: null pointer");
  if (m < 0 || n < 0 || k < 0 || batch < 1)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_matmul: bad shape m=%lld n=%lld k=%lld batch=%lld", (long long)m, (long long)n,
                        (long long)k, (long long)batch);
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX || batch > 65535)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_matmul: dimension too large");
  if (!tl_dtype_valid(dtype_a) || !tl_dtype_valid(dtype_b) || !tl_dtype_valid(out_dtype))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_matmul: unknown dtype");
  if ((cast_a >= 0 && cast_a != TL_F16 && cast_a != TL_BF16) || (cast_b >= 0 && cast_b != TL_F16 && cast_b != TL_BF16))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_matmul: the cast prologue rounds through f16 or bf16");
  if (stride_a < 0 || stride_b < 0 || stride_c < 0 || (batch > 1 && stride_c < m * n))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_matmul: bad batch strides (outputs of different batches must not overlap)");
  EpiParams epi;
  bool has_ops = false;
  int32_t rc = tl_make_epi(ctx, epilogue, alpha, &epi, &has_ops);
  if (rc != TL_OK) return rc;
  if (batch > 1)
    for (int i = 0; i < epi.n_ops; ++i)
      if (epi.kind[i] == TL_EPI_BINARY)
        return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_matmul: a binary epilogue input needs batch == 1");
  MatmulArgs p{};
  p.a = a; p.b = b; p.out = out;
  p.m = int32_t(m); p.n = int32_t(n); p.k = int32_t(k); p.batch = int32_t(batch);
  p.stride_a = stride_a; p.stride_b = stride_b; p.stride_c = stride_c;
  p.trans_a = trans_a ? 1 : 0; p.trans_b = trans_b ? 1 : 0;
  p.dtype_a = dtype_a; p.dtype_b = dtype_b; p.out_dtype = out_dtype;
  p.cast_a = cast_a; p.cast_b = cast_b;
  // selection (variants.ts:160-183): the GEMV when it applies and is not switched off, else tiled
  const char* env = getenv("TORCHLETTE_GEMV");
  const bool gemv_off = env && env[0] == '0';
  const bool forced_tiled = ctx->has_forced && ctx->forced.family == TL_FAMILY_MATMUL && ctx->forced.kernel == kTiled;
  const bool use_gemv = !gemv_off && !forced_tiled && (receipt_only ? (m >= 1 && m <= 16 && batch == 1 && trans_b && !trans_a &&
                                                                       dtype_a == dtype_b && dtype_a != TL_F32 && cast_a < 0 &&
                                                                       cast_b < 0 && k % 32 == 0 && k >= 32)
                                                                    : gemv_applicable(p, epi));
  int warps = 8;
  if (use_gemv) {
    const int kblocks = int(k / 32);
    warps = kblocks >= 16 ? 16 : kblocks >= 8 ? 8 : kblocks >= 4 ? 4 : kblocks >= 2 ? 2 : 1;
    if (m > 8 && warps > 4) warps = 4;  // two batch tiles: 31.7 us against 36.2 with 16 warps on 4096 x 14336
    // A/B hook: {TL_FAMILY_MATMUL, 1, warps} forces the CTA width
    if (ctx->has_forced && ctx->forced.family == TL_FAMILY_MATMUL && ctx->forced.kernel == kGemv && ctx->forced.p0 >= 1 &&
        ctx->forced.p0 <= 16 && (ctx->forced.p0 & (ctx->forced.p0 - 1)) == 0)
      warps = ctx->forced.p0;
  }
  const bool forced_tc = ctx->has_forced && ctx->forced.family == TL_FAMILY_MATMUL && ctx->forced.kernel == kTc;
  const size_t esz_ab = 2;
  const bool batch_aligned = batch == 1 || ((stride_a * esz_ab) % 16 == 0 && (stride_b * esz_ab) % 16 == 0);
  const bool use_tc = !use_gemv && !forced_tiled && cast_a < 0 && cast_b < 0 && batch_aligned &&
                      tl_dense_tc_applicable(a, b, m, n, k, dtype_a, dtype_b);
  if (forced_tc && !use_tc)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_matmul: the tensor-core kernel cannot run m=%lld n=%lld k=%lld with these dtypes / casts",
                        (long long)m, (long long)n, (long long)k);
  if (receipt_only) {
    tl_variant v{};
    v.family = TL_FAMILY_MATMUL; v.kernel = use_gemv ? kGemv : use_tc ? kTc : kTiled; v.p0 = use_gemv ? warps : 8;
    receipt_only->choice = v;
    receipt_only->grid[0] = use_gemv ? int32_t((n + 15) / 16) : int32_t((n + kTN - 1) / kTN);
    receipt_only->grid[1] = use_gemv ? 1 : int32_t((m + kTM - 1) / kTM);
    receipt_only->grid[2] = use_gemv ? 1 : int32_t(batch);
    receipt_only->block = use_gemv ? warps * 32 : 256;
    if (use_tc) {
      const bool f = forced_tc && ctx->forced.p0 > 0;
      bool ra_mn, rb_mn;
      dense_mn_operands(trans_a != 0, trans_b != 0, m, n, &ra_mn, &rb_mn);
      const TlDenseTcChoice ch = tl_dense_tc_choose(m, n, k, ctx->sm_count, f ? ctx->forced.p0 : 0, f ? ctx->forced.p2 : 0,
                                                    (ra_mn || rb_mn) ? 64 : 16);
      receipt_only->choice.p0 = ch.bn; receipt_only->choice.p1 = ch.stages; receipt_only->choice.p2 = ch.mh;
      receipt_only->grid[0] = ch.grid; receipt_only->grid[1] = 1; receipt_only->grid[2] = 1;
      receipt_only->block = 576;
    }
    receipt_only->split_k = 1;
    receipt_only->from_tuning_cache = 0;
    receipt_only->epilogue_engaged = has_ops ? 1 : 0;
    return TL_OK;
  }
  if (m == 0 || n == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  if (use_gemv) {
    const int grid = int((n + 15) / 16), block = warps * 32;
    const int nt = m > 8 ? 2 : 1;
    const size_t smem = size_t(warps) * nt * 128 * sizeof(float);
    if (dtype_a == TL_F16) {
      if (nt == 2) dense_gemv_kernel<__half, 2><<<grid, block, smem, ctx->stream>>>(p, epi);
      else dense_gemv_kernel<__half, 1><<<grid, block, smem, ctx->stream>>>(p, epi);
    } else {
      if (nt == 2) dense_gemv_kernel<__nv_bfloat16, 2><<<grid, block, smem, ctx->stream>>>(p, epi);
      else dense_gemv_kernel<__nv_bfloat16, 1><<<grid, block, smem, ctx->stream>>>(p, epi);
    }
    ctx->counters[TL_COUNTER_GEMV]++;
    if (has_ops) ctx->counters[TL_COUNTER_QGEMV_EPILOGUE]++;
  } else if (use_tc) {
    // bring the operands to the NT layout (A [M, K], B [N, K]) in scratch where they are stored transposed
    // a B stored [K, N] is multiplied as it lies (MN-major tiles) when its row pitch allows a TMA map
    bool a_mn, b_mn;
    dense_mn_operands(p.trans_a != 0, p.trans_b != 0, m, n, &a_mn, &b_mn);
    const size_t a_elems = (p.trans_a && !a_mn) ? size_t(m) * k : 0, b_elems = (p.trans_b || b_mn) ? 0 : size_t(n) * k;
    uint8_t* scratch = nullptr;
    if (a_elems + b_elems) {
      void* sp = nullptr;
      rc = tl_ensure_scratch(ctx, (a_elems + b_elems) * 2 + 256, &sp);
      if (rc != TL_OK) return rc;
      scratch = static_cast<uint8_t*>(sp);
    }
    for (int64_t bi = 0; bi < batch; ++bi) {
      const uint8_t* ab = static_cast<const uint8_t*>(a) + size_t(bi) * stride_a * 2;
      const uint8_t* bb = static_cast<const uint8_t*>(b) + size_t(bi) * stride_b * 2;
      uint8_t* ob = static_cast<uint8_t*>(out) + size_t(bi) * stride_c * tl_dtype_size(out_dtype);
      if (p.trans_a && !a_mn && (bi == 0 || stride_a != 0)) {
        rc = tl_transpose2d(ctx, ab, scratch, 1, k, m, 2);  // stored [K, M] -> [M, K]
        if (rc != TL_OK) return rc;
      }
      uint8_t* bt = scratch + ((a_elems * 2 + 255) & ~size_t(255));
      if (!p.trans_b && !b_mn && (bi == 0 || stride_b != 0)) {
        rc = tl_transpose2d(ctx, bb, bt, 1, k, n, 2);       // stored [K, N] -> [N, K]
        if (rc != TL_OK) return rc;
      }
      rc = tl_launch_dense_tc(ctx, (p.trans_a && !a_mn) ? scratch : ab, (p.trans_b || b_mn) ? bb : bt, ob, m, n, k, dtype_a, out_dtype,
                              epi, nullptr, 0, 1.0f, b_mn, a_mn);
      if (rc != TL_OK) return rc;
    }
    ctx->counters[TL_COUNTER_MATMUL]++;
    return TL_OK;
  } else {
    dim3 grid(unsigned((n + kTN - 1) / kTN), unsigned((m + kTM - 1) / kTM), unsigned(batch));
    matmul_tiled_kernel<<<grid, 256, 0, ctx->stream>>>(p, epi);
    ctx->counters[TL_COUNTER_MATMUL]++;
  }
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}
