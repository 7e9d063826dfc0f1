// Small-batch (m = 1..16) weight-only int8 matmul: out[m,n] = epi(alpha * a[m,k] . W[n,k]).
// HBM-bound: the int8 weight is streamed once with 128-bit loads, dequantized in
// registers and never materialized.  Replaces the WGSL GEMV builder
// (src/backend/webgpu/matmul/gemv.ts:311-466, quant load :400-429).
//
// Kernel ids (tl_variant.kernel) of family TL_FAMILY_QGEMV:
//   0 "scalar" one lane per packed word, per-element dequant in the reference's
//              own order; any K % 4 == 0 and any group size.  The fallback.
//   1 "simt"   one warp per R rows, 16-byte weight loads, byte->f32 by exponent
//              stuffing (prmt), f32 FMA, per-chunk group scale.  K % 16 == 0,
//              G % 16 == 0.  Exact f32 activations.
//   2 "mma"    one CTA per 16 rows, warps interleaved over 64-wide k blocks, raw
//              bytes -> f16/bf16 pairs in registers -> mma.sync m16n8k16 with f32
//              accumulators; the batch is the MMA n dimension.  f16/bf16
//              activations, K % 64 == 0, G % 64 == 0.
//   4 "ring"   kernel 2's tiling with the weight bytes prefetched global -> shared by
//              per-thread cp.async rings (no registers held in flight).  The default.
//              p0 = warps per tile, p1 = ring depth (2/4/6/8), p2 = 2: 32-row tiles.
//              Also: a batched launch (several matrices, same activations), a launch fused
//              with the tensor-parallel all-reduce, and the persistent chain (kernel id 7
//              only names the chain's CTA shape for tl_force_variant).
//   6 "bulk"   persistent grid fed by contiguous cp.async.bulk copies of whole 8-row
//              blocks; batch as the MMA A operand; no cross-CTA partial sums.
//              p0 = consumer warps, p1 = stage size target in KB.
//   5 "tma"    persistent grid fed by 32 KB tensor-map TMA boxes through a shared-memory
//              ring; 16 consumer warps x 16 rows; balanced contiguous shares of boxes.
//              f16/bf16 activations, K % 128 == 0, G % 64 == 0.  p0 = stages.
//   3 "sk"     persistent grid, the weight dealt out to warps in equal contiguous
//              shares of 8-row x 128-byte units; partial tiles meet in an f32
//              scratch.  f16/bf16 activations, K % 128 == 0, G % 128 == 0.
//   8 "stream" persistent warp-specialised kernel (tl_qgemv_stream.cu): bulk-copy producers, MMA
//              consumers, an epilogue warp; two launches resident per SM with a drain-timed
//              ring fill.  p0 = consumer warps (8), p1 = ring stages, p2 = producer warps,
//              p3 = k blocks per stage (16 or 32).
// Variant parameters: p0 = warps per CTA (sk: CTAs per SM), p1 = rows per warp
// (simt) / k blocks in flight (mma, sk, ring), p2 = see ring, p3 = reserved.
#include <algorithm>

#include "tl_common.cuh"
#include "tl_mma_frag.cuh"
#include "tl_tma.cuh"

namespace {

constexpr int kScalar = 0, kSimt = 1, kMma = 2, kSk = 3, kRing = 4, kTma = 5, kBulk = 6, kChain = 7, kStream = 8;

// geometry of the "bulk" kernel for a given k: tiles per stage, stage bytes, stages, warps per tile
struct BulkGeom { int rt, nstages, p; uint32_t stage_bytes; size_t smem; bool ok; };
inline BulkGeom bulk_geom(int64_t k, int cwarps, int target_kb) {
  BulkGeom gm{};
  const int64_t tile_bytes = 8 * k;
  gm.rt = int(std::max<int64_t>(1, (int64_t(target_kb) * 1024) / tile_bytes));
  gm.stage_bytes = uint32_t(gm.rt * tile_bytes);
  int kb128 = int(k / 128), pw = 1;
  while (pw * 2 <= kb128 && pw * 2 <= cwarps) pw *= 2;
  gm.p = pw;
  const size_t red = size_t(2) * gm.rt * gm.p * 128 * sizeof(float);
  const size_t budget = 220 * 1024;
  gm.ok = tile_bytes <= 100 * 1024 && red + 2 * size_t(gm.stage_bytes) + 128 <= budget;
  gm.nstages = gm.ok ? int(std::min<size_t>(8, (budget - red - 128) / gm.stage_bytes)) : 0;
  gm.smem = size_t(gm.nstages) * gm.stage_bytes + red + 128;
  return gm;
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  // weights are read exactly once: keep them out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct GemvArgs {
  const void* a;
  const uint32_t* packed;
  const void* scales;
  void* out;
  int32_t m, n, k;
  int32_t group, groups_per_row;
  int32_t scales_dtype, out_dtype;
  float wscale;    // 1/127 for the snorm convention, 1 for direct
  int32_t row0;    // first batch row of this launch (epilogue binary inputs index absolute rows)
  int32_t m_total;
};


// ---------------------------------------------------------------------------
// 0: scalar fallback.  One warp per output row; lane l walks words l, l+32, ...
// Element arithmetic as in the reference kernel: acc += a[k] * ((q/127) * s).
// ---------------------------------------------------------------------------
template <typename AT>
__global__ void __launch_bounds__(256) qgemv_scalar_kernel(GemvArgs p, EpiParams epi) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * warps + (threadIdx.x >> 5);
  if (row >= p.n) return;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const int words = p.k >> 2;
  const uint32_t* wrow = p.packed + row * words;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (int w = lane; w < words; w += 32) {
    const uint32_t word = __ldg(wrow + w);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int kk = 4 * w + b;
      const float s = tl_load_scale(p.scales, p.scales_dtype, row * p.groups_per_row + kk / p.group);
      const int q = int(int8_t((word >> (8 * b)) & 0xffu));
      const float wv = (float(q) * p.wscale) * s;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (i < p.m) acc[i] = fmaf(DT<AT>::to_f32(a[int64_t(i) * p.k + kk]), wv, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (i < p.m) {
      const float v = warp_sum(acc[i]);
      if (lane == 0) {
        const float r = tl_apply_epilogue(epi, v, p.row0 + i, row, p.n);
        tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + i) * p.n + row, r);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// 1: SIMT.  Byte b of x = word ^ 0x80808080 is q+128; prmt drops it into the
// low mantissa byte of 0x4B000000 (2^23), so the float is 2^23 + 128 + q exactly
// and one subtraction yields q.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void bytes_to_f32(uint32_t word, float (&f)[4]) {
  const uint32_t x = word ^ 0x80808080u;
  f[0] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650)) - 8388736.f;
  f[1] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651)) - 8388736.f;
  f[2] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652)) - 8388736.f;
  f[3] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653)) - 8388736.f;
}

template <typename AT> struct ActChunk;  // 16 activations of one batch row as f32
template <> struct ActChunk<float> {
  __device__ static void load(const float* p, float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
      x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
  }
};
template <> struct ActChunk<__half> {
  __device__ static void load(const __half* p, float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        x[8 * i + 2 * j] = f.x; x[8 * i + 2 * j + 1] = f.y;
      }
    }
  }
};
template <> struct ActChunk<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16* p, float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
        x[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
  }
};

// MT batch rows, R output rows per warp.  Lane l handles 16-byte chunks l, l+32, ...
template <typename AT, int MT, int R, bool GROUPED>
__global__ void __launch_bounds__(256) qgemv_simt_kernel(GemvArgs p, EpiParams epi) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_base = (int64_t(blockIdx.x) * warps + (threadIdx.x >> 5)) * R;
  if (row_base >= p.n) return;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const int chunks = p.k >> 4;
  const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(p.packed);
  int64_t rows[R];
#pragma unroll
  for (int r = 0; r < R; ++r) rows[r] = min(row_base + r, int64_t(p.n) - 1);  // tail rows clamp, stores mask
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[r][i] = 0.f;

  for (int c = lane; c < chunks; c += 32) {
    uint4 wv[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wv[r] = ldg_stream(wbytes + rows[r] * p.k + int64_t(c) * 16);
    float x[MT][16];
#pragma unroll
    for (int i = 0; i < MT; ++i) ActChunk<AT>::load(a + int64_t(i) * p.k + int64_t(c) * 16, x[i]);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t w4[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
      float part[MT];
#pragma unroll
      for (int i = 0; i < MT; ++i) part[i] = GROUPED ? 0.f : acc[r][i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float f[4];
        bytes_to_f32(w4[j], f);
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int i = 0; i < MT; ++i) part[i] = fmaf(f[b], x[i][4 * j + b], part[i]);
      }
      if (GROUPED) {
        const float s = tl_load_scale(p.scales, p.scales_dtype, rows[r] * p.groups_per_row + (c * 16) / p.group);
#pragma unroll
        for (int i = 0; i < MT; ++i) acc[r][i] = fmaf(s, part[i], acc[r][i]);
      } else {
#pragma unroll
        for (int i = 0; i < MT; ++i) acc[r][i] = part[i];
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int64_t row = row_base + r;
    float s = p.wscale;
    if (!GROUPED) s *= tl_load_scale(p.scales, p.scales_dtype, rows[r]);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const float v = warp_sum(acc[r][i]) * s;
      if (lane == 0 && row < p.n) {
        const float o = tl_apply_epilogue(epi, v, p.row0 + i, row, p.n);
        tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + i) * p.n + row, o);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// 2: tensor-core small-batch kernel.
//
// CTA = W warps, one 16-row weight tile.  Warp w owns k blocks kb = w, w+W, ...
// (64 bytes of every row each), so at any moment the CTA reads W*64 contiguous
// bytes per row.  Thread (g = lane/4, t = lane%4) loads 16 bytes of row g and of
// row g+8 at k = 64*kb + 16*t.  Word j of that chunk feeds MMA j of the block:
// its bytes 0,1 sit in k slots 2t,2t+1 and bytes 2,3 in slots 2t+8,2t+9.  The
// k order inside a block is therefore permuted, identically for the weight (A)
// and activation (B) fragments, which leaves the dot product unchanged.
// B for MMA j: halves [4j, 4j+4) of the thread's 16 contiguous activations of
// batch row g (columns of the MMA n dimension = batch rows).
// ---------------------------------------------------------------------------
constexpr int kMmaMaxWarps = 16;

// NT = number of 8-wide batch tiles (1: m <= 8, 2: m <= 16); UNROLL k blocks in flight per warp.
template <typename AT, int NT, bool GROUPED, int UNROLL>
__global__ void __launch_bounds__(kMmaMaxWarps * 32) qgemv_mma_kernel(GemvArgs p, EpiParams epi) {
  __shared__ float red[kMmaMaxWarps][NT][4][32];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t tile_row = int64_t(blockIdx.x) * 16;
  const int64_t r_lo = min(tile_row + g, int64_t(p.n) - 1);
  const int64_t r_hi = min(tile_row + g + 8, int64_t(p.n) - 1);
  const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(p.packed);
  const uint8_t* w_lo = wbytes + r_lo * p.k + 16 * t;
  const uint8_t* w_hi = wbytes + r_hi * p.k + 16 * t;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  // batch rows this thread supplies as MMA columns: g (tile 0) and g+8 (tile 1)
  const AT* a_col[NT];
  bool a_ok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    a_ok[nt] = (g + 8 * nt) < p.m;
    a_col[nt] = a + int64_t(a_ok[nt] ? g + 8 * nt : 0) * p.k + 16 * t;
  }
  const int kblocks = p.k >> 6;

  float total[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) total[nt][i] = 0.f;

  for (int kb0 = warp; kb0 < kblocks; kb0 += warps * UNROLL) {
    uint4 wl[UNROLL], wh[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * warps;
      if (kb < kblocks) {
        wl[u] = ldg_stream(w_lo + int64_t(kb) * 64);
        wh[u] = ldg_stream(w_hi + int64_t(kb) * 64);
      } else {
        wl[u] = make_uint4(0x0, 0x0, 0x0, 0x0);
        wh[u] = make_uint4(0x0, 0x0, 0x0, 0x0);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * warps;
      if (kb >= kblocks) break;
      uint4 bx[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (a_ok[nt]) {
          const uint4* src = reinterpret_cast<const uint4*>(a_col[nt] + int64_t(kb) * 64);
          bx[nt][0] = __ldg(src);
          bx[nt][1] = __ldg(src + 1);
        } else {
          bx[nt][0] = make_uint4(0, 0, 0, 0);
          bx[nt][1] = make_uint4(0, 0, 0, 0);
        }
      }
      float c[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) c[nt][i] = GROUPED ? 0.f : total[nt][i];
      const uint32_t wlo[4] = {wl[u].x, wl[u].y, wl[u].z, wl[u].w};
      const uint32_t whi[4] = {wh[u].x, wh[u].y, wh[u].z, wh[u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a0, a1, a2, a3;
        MmaOps<AT>::cvt(wlo[j], a0, a2);  // row g   : slots (2t,2t+1) and (2t+8,2t+9)
        MmaOps<AT>::cvt(whi[j], a1, a3);  // row g+8
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4 v = bx[nt][j >> 1];
          const uint32_t b0 = (j & 1) ? v.z : v.x, b1 = (j & 1) ? v.w : v.y;
          MmaOps<AT>::mma(c[nt], a0, a1, a2, a3, b0, b1);
        }
      }
      if (GROUPED) {
        const int gi = (kb * 64) / p.group;
        const float s_lo = tl_load_scale(p.scales, p.scales_dtype, r_lo * p.groups_per_row + gi);
        const float s_hi = tl_load_scale(p.scales, p.scales_dtype, r_hi * p.groups_per_row + gi);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          total[nt][0] = fmaf(s_lo, c[nt][0], total[nt][0]);
          total[nt][1] = fmaf(s_lo, c[nt][1], total[nt][1]);
          total[nt][2] = fmaf(s_hi, c[nt][2], total[nt][2]);
          total[nt][3] = fmaf(s_hi, c[nt][3], total[nt][3]);
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) total[nt][i] = c[nt][i];
      }
    }
  }

  // cross-warp sum of the k partitions, then scale + epilogue + store
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp][nt][i][lane] = total[nt][i];
  __syncthreads();
  // one thread per (tile nt, fragment slot i, lane): NT*128 outputs
  for (int o = threadIdx.x; o < NT * 128; o += blockDim.x) {
    const int nt = o >> 7, i = (o >> 5) & 3, ln = o & 31;
    float v = 0.f;
    for (int w = 0; w < warps; ++w) v += red[w][nt][i][ln];
    const int gg = ln >> 2, tt = ln & 3;
    const int64_t row = tile_row + gg + ((i & 2) ? 8 : 0);  // c0,c1: row g ; c2,c3: row g+8
    const int col = 8 * nt + 2 * tt + (i & 1);                // batch row
    if (row < p.n && col < p.m) {
      float s = p.wscale;
      if (!GROUPED) s *= tl_load_scale(p.scales, p.scales_dtype, row);
      const float r = tl_apply_epilogue(epi, v * s, p.row0 + col, row, p.n);
      tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + col) * p.n + row, r);
    }
  }
}

// ---------------------------------------------------------------------------
// 3: balanced streaming kernel ("sk").
//
// The weight is cut into units of 8 rows x 128 bytes.  Units are numbered with k
// fastest inside an 8-row tile, and the flat range is dealt out to the warps of a
// persistent grid in equal contiguous shares, so every SM streams the same number
// of bytes whatever N is (no wave quantisation).  Warps never synchronise with
// one another: a warp that owns only part of a tile's k range adds its partial
// sums to a zero-initialised f32 scratch [M,N] and bumps the tile's unit counter;
// the warp that completes the count applies scale + epilogue, stores, and zeroes
// the scratch and the counter again.  Nobody waits on anybody.
//
// Here the roles of the MMA operands are swapped with respect to kernel 2: the
// batch is the 16-row A operand (so m = 9..16 costs no extra MMA) and 8 weight
// rows are the B operand.  Thread (g,t) loads 32 contiguous bytes of weight row g
// (word j feeds MMA j: bytes 0,1 -> k slots 2t,2t+1; bytes 2,3 -> 2t+8,2t+9) and
// the matching 32 activations of batch rows g and g+8.
// ---------------------------------------------------------------------------
struct SkArgs {
  float* scratch;       // [m, n] f32, all zero between launches
  unsigned* counters;   // [tiles], all zero between launches
  int32_t upt;          // units per tile = k / 128
  int32_t warps_used;
  int64_t total_units;
};

template <typename AT, bool M16, bool GROUPED, int D>
__global__ void __launch_bounds__(256) qgemv_sk_kernel(GemvArgs p, EpiParams epi, SkArgs sk) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int wg = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wg >= sk.warps_used) return;
  const int64_t q = sk.total_units / sk.warps_used, r = sk.total_units % sk.warps_used;
  const int64_t u0 = wg * q + min(int64_t(wg), r);
  const int cnt = int(q + (wg < r ? 1 : 0));
  if (cnt == 0) return;

  const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(p.packed);
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const bool lo_ok = g < p.m, hi_ok = M16 && (g + 8) < p.m;
  const AT* a_lo = a + int64_t(lo_ok ? g : 0) * p.k + 32 * t;
  const AT* a_hi = a + int64_t(hi_ok ? g + 8 : 0) * p.k + 32 * t;

  // load cursor and compute cursor over (tile, unit-in-tile)
  int tile_l = int(u0 / sk.upt), ku_l = int(u0 % sk.upt);
  int tile_c = tile_l, ku_c = ku_l;
  auto wptr = [&](int tile, int ku) {
    const int64_t row = min(int64_t(tile) * 8 + g, int64_t(p.n) - 1);
    return wbytes + row * p.k + int64_t(ku) * 128 + 32 * t;
  };
  uint4 buf[D][2];
#pragma unroll
  for (int d = 0; d < D; ++d) {
    if (d < cnt) {
      const uint8_t* ptr = wptr(tile_l, ku_l);
      buf[d][0] = ldg_stream(ptr);
      buf[d][1] = ldg_stream(ptr + 16);
      if (++ku_l == sk.upt) { ku_l = 0; ++tile_l; }
    }
  }

  float total[4] = {0.f, 0.f, 0.f, 0.f};
  int mine = 0;  // units of the current tile accumulated by this warp
  for (int i = 0; i < cnt; i += D) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
      if (i + d < cnt) {
        const uint32_t w8[8] = {buf[d][0].x, buf[d][0].y, buf[d][0].z, buf[d][0].w,
                                buf[d][1].x, buf[d][1].y, buf[d][1].z, buf[d][1].w};
        if (i + d + D < cnt) {  // refill this slot D units ahead
          const uint8_t* ptr = wptr(tile_l, ku_l);
          buf[d][0] = ldg_stream(ptr);
          buf[d][1] = ldg_stream(ptr + 16);
          if (++ku_l == sk.upt) { ku_l = 0; ++tile_l; }
        }
        // activations of this unit: 32 halves per batch row
        uint32_t xl[16], xh[16];
        {
          const uint4* s0 = reinterpret_cast<const uint4*>(a_lo + int64_t(ku_c) * 128);
          const uint4* s1 = reinterpret_cast<const uint4*>(a_hi + int64_t(ku_c) * 128);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 lo4 = lo_ok ? __ldg(s0 + v) : make_uint4(0, 0, 0, 0);
            xl[4 * v] = lo4.x; xl[4 * v + 1] = lo4.y; xl[4 * v + 2] = lo4.z; xl[4 * v + 3] = lo4.w;
            if (M16) {
              uint4 hi4 = hi_ok ? __ldg(s1 + v) : make_uint4(0, 0, 0, 0);
              xh[4 * v] = hi4.x; xh[4 * v + 1] = hi4.y; xh[4 * v + 2] = hi4.z; xh[4 * v + 3] = hi4.w;
            } else {
              xh[4 * v] = 0; xh[4 * v + 1] = 0; xh[4 * v + 2] = 0; xh[4 * v + 3] = 0;
            }
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float c[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) c[e] = GROUPED ? 0.f : total[e];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int j = half * 4 + jj;
            uint32_t b0, b1;
            MmaOps<AT>::cvt(w8[j], b0, b1);
            MmaOps<AT>::mma(c, xl[2 * j], xh[2 * j], xl[2 * j + 1], xh[2 * j + 1], b0, b1);
          }
          if (GROUPED) {
            const int gi = (ku_c * 128 + half * 64) / p.group;
            const int64_t r0 = min(int64_t(tile_c) * 8 + 2 * t, int64_t(p.n) - 1);
            const int64_t r1 = min(int64_t(tile_c) * 8 + 2 * t + 1, int64_t(p.n) - 1);
            const float s0 = tl_load_scale(p.scales, p.scales_dtype, r0 * p.groups_per_row + gi);
            const float s1 = tl_load_scale(p.scales, p.scales_dtype, r1 * p.groups_per_row + gi);
            total[0] = fmaf(s0, c[0], total[0]);
            total[1] = fmaf(s1, c[1], total[1]);
            total[2] = fmaf(s0, c[2], total[2]);
            total[3] = fmaf(s1, c[3], total[3]);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) total[e] = c[e];
          }
        }
        ++mine;
        const bool tile_done = (ku_c + 1 == sk.upt);
        if (tile_done || i + d + 1 == cnt) {
          // flush the accumulators of tile_c: c0,c1 = batch g, rows 2t,2t+1 ; c2,c3 = batch g+8
          const int64_t rbase = int64_t(tile_c) * 8 + 2 * t;
          bool finalize = (mine == sk.upt);
          if (!finalize) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int b = g + ((e & 2) ? 8 : 0);
              const int64_t row = rbase + (e & 1);
              if (b < p.m && row < p.n) atomicAdd(sk.scratch + int64_t(b) * p.n + row, total[e]);
            }
            __threadfence();
            __syncwarp();  // every lane's partial sums are published before the count moves
            unsigned old = 0;
            if (lane == 0) old = atomicAdd(sk.counters + tile_c, unsigned(mine));
            old = __shfl_sync(0xffffffffu, old, 0);
            finalize = (old + unsigned(mine) == unsigned(sk.upt));
            if (finalize) {
              __threadfence();
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int b = g + ((e & 2) ? 8 : 0);
                const int64_t row = rbase + (e & 1);
                if (b < p.m && row < p.n) {
                  float* sp = sk.scratch + int64_t(b) * p.n + row;
                  total[e] = __ldcg(sp);
                  __stcg(sp, 0.f);
                }
              }
              if (lane == 0) sk.counters[tile_c] = 0;
            }
          }
          if (finalize) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int b = g + ((e & 2) ? 8 : 0);
              const int64_t row = rbase + (e & 1);
              if (b < p.m && row < p.n) {
                float s = p.wscale;
                if (!GROUPED) s *= tl_load_scale(p.scales, p.scales_dtype, row);
                const float o = tl_apply_epilogue(epi, total[e] * s, p.row0 + b, row, p.n);
                tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + b) * p.n + row, o);
              }
            }
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) total[e] = 0.f;
          mine = 0;
        }
        if (++ku_c == sk.upt) { ku_c = 0; ++tile_c; }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// 4: tensor-core kernel with an asynchronous prefetch ring ("ring").
//
// Same tiling and fragment mapping as kernel 2 (one CTA per 16 rows, warps
// interleaved over 64-wide k blocks, weights as the MMA A operand), but the weight
// bytes travel global -> shared with 16-byte cp.async copies that hold no
// registers while in flight.  Every thread owns S private slots of 2 x 16 bytes
// (row g and row g+8 of one k block): it copies, waits for and reads only its own
// slots, so no barrier is needed and consecutive lanes touch consecutive 16-byte
// words (no bank conflicts).  With S k blocks in flight per thread and small CTAs
// (so that many are resident per SM) an SM keeps ~100 KB of loads outstanding,
// which is what it takes to cover HBM latency at full bandwidth.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

// Arguments of the fused row-parallel GEMV + all-reduce (see qgemv_ring_allreduce_kernel).
struct PushArgs {
  uint8_t* base[tl_ctx::kMaxPeers];  // every rank's exchange buffer as mapped on this GPU (own = local)
  int32_t rank, world;
  uint64_t max_bytes;                // size of one slot
  void* dst;                         // [m, n] sum over ranks, in the output type
  int* status;
  int spin_limit;                    // polls of one wait before it gives up (the context's wait_limit_polls)
};
__device__ __forceinline__ uint32_t push_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void push_red_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float push_load(const void* base, int dtype, int64_t idx) {
  // written by other GPUs: volatile loads, never a cached copy
  if (dtype == TL_F32) return __ldcv(reinterpret_cast<const float*>(base) + idx);
  const unsigned short bits = __ldcv(reinterpret_cast<const unsigned short*>(base) + idx);
  if (dtype == TL_F16) return __half2float(__ushort_as_half(bits));
  return __uint_as_float(uint32_t(bits) << 16);
}

// ---------------------------------------------------------------------------
// Push / reduce-on-read: the row-parallel sum of tensor parallelism without a collective launch.
//
// tl_qgemv_nt_push (ring tile, PUSH == 2): every CTA stages its 16-row tile of the LOCAL partial
// product in shared memory, in f32, and stores it into slot (half, rank) of EVERY rank's exchange
// buffer as 8-byte words {two partial sums of 24 bits each, 16-bit tag} (push_pack).  (Not the 16-bit
// output type: a 16-bit partial loses up to half an ulp of a value that may be far larger than the
// total, and eight of them add up to 1e-2 on the parity metric.  Whole f32 values would double the
// NVLink bytes: measured +0.14 ms per step at 8 ranks.)  An 8-byte store arrives
// whole, so the epoch that travels with the data is the arrival signal: the producer needs no fence,
// no atomic and no flag (a system-scope release per CTA, 256 per launch, cost 8 us; fences from
// every thread 12 us), and it waits for nobody.
//
// The NEXT small-batch launch of every rank (the column-parallel q+k+v / gate+up / lm_head product,
// which reads the summed vector as its activations) does the sum in its prologue, after
// griddepcontrol.wait and with its weight prefetch already in flight: its first `nsum` CTAs each
// take a slice of the vector, poll (bounded) the words of all ranks until they carry this push's
// epoch, add them in rank order (every rank computes the same bits) into the activation buffer and
// arrive on done[half]; all CTAs wait for `nsum` arrivals there (a grid-wide gate that can not
// deadlock: the summing CTAs are the first of the grid) and then read the activations.  No
// all-reduce kernel, no NCCL, and the NVLink trip runs under the consumer's weight prefetch.
//
// Words of a rank's exchange buffer (tl_p2p_push_words_offset): done[2] at words 2-3, epoch_p (4),
// epoch_c (5).  Halves alternate per push (epoch_p & 1) so that a rank that is ahead overwrites the
// half its peers no longer read.  The epochs live on the device (a replayed graph keeps counting):
// the producer reads epoch_p and publishes epoch_c = epoch_p + 1, the consumer reads epoch_c and
// publishes epoch_p = epoch_c.  A producer clears done[] of the OTHER half when it starts (its own
// previous consumer has finished with it).  Slots are [2 halves][kMaxPeers][max_bytes] with
// max_bytes >= m * n * 4 (two partial sums and a tag per 8-byte word).
// ---------------------------------------------------------------------------
// One 8-byte word of the push protocol carries TWO partial sums and the arrival tag: each f32 is
// rounded (to nearest even) to 24 bits -- sign, exponent, 15 mantissa bits: 32 times finer than an
// f16 partial, so the sum of eight of them still rounds to the right 16-bit result -- and the last
// 16 bits hold (epoch % 65535) + 1, never 0, so zero-filled memory never looks like an arrival.
//   lo = v0[31:8] | v1[31:24]      hi = v1[23:8] << 16 | tag
__device__ __forceinline__ uint32_t push_round24(float v) {
  const uint32_t b = __float_as_uint(v);
  if ((b & 0x7f800000u) == 0x7f800000u) return b & 0xffffff00u;  // Inf / NaN: truncate, never carry into the sign
  return (b + 0x7fu + ((b >> 8) & 1u)) & 0xffffff00u;
}
__device__ __forceinline__ uint32_t push_tag(uint32_t epoch) { return epoch % 65535u + 1u; }
__device__ __forceinline__ uint2 push_pack(float v0, float v1, uint32_t tag) {
  const uint32_t b0 = push_round24(v0), b1 = push_round24(v1);
  return make_uint2(b0 | (b1 >> 24), ((b1 << 8) & 0xffff0000u) | tag);
}
__device__ __forceinline__ void push_unpack(uint32_t lo, uint32_t hi, float& v0, float& v1) {
  v0 = __uint_as_float(lo & 0xffffff00u);
  v1 = __uint_as_float(((lo & 0xffu) << 24) | ((hi >> 8) & 0x00ffff00u));
}

struct ReduceIn {
  uint8_t* base;        // this rank's exchange buffer
  uint64_t max_bytes;
  void* dst;            // [m, n] summed vector = the consumer's activations
  int32_t world, expected, nsum, count_vec;  // arrivals to wait for; summing CTAs; 16-byte vectors in m*n
  int32_t dtype;        // TL_F16 or TL_BF16
  int* status;
  int32_t spin_limit;
  int32_t poll_ranks;   // ranks whose words are requested together (1..4; the context's push_poll_ranks)
};
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void reduce_in_prologue(const ReduceIn& r) {
  const int tid = threadIdx.x, nthreads = blockDim.x;
  uint32_t* words = reinterpret_cast<uint32_t*>(r.base + tl_p2p_push_words_offset(r.max_bytes));
  // published by the producer kernel, which has completed.  Read through L2: under programmatic
  // dependent launch this CTA's SM may still hold the line from an overlapping earlier kernel.
  const uint32_t epoch = __ldcv(words + 5);
  const int half = int((epoch - 1u) & 1u);
  if (int(blockIdx.x) < r.nsum) {
    {
      const uint8_t* slots = r.base + tl_p2p_push_slots_offset(r.max_bytes) + size_t(half) * tl_ctx::kMaxPeers * r.max_bytes;
      const int per = (r.count_vec + r.nsum - 1) / r.nsum;
      const int v0 = int(blockIdx.x) * per, v1 = min(v0 + per, r.count_vec);
      for (int i = v0 + tid; i < v1; i += nthreads) {
        // output vector i = 8 values = four {two partial sums, tag} words (32 bytes) of every rank's slot
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const uint32_t tag = push_tag(epoch);
        // four ranks' words are requested together (eight 16-byte loads in flight), then checked: polling
        // the ranks one after the other costs an L2 round trip per rank, 5 us per exchange at 8 ranks
        for (int r0 = 0; r0 < r.world; r0 += r.poll_ranks) {
          const int nb = min(r.poll_ranks, r.world - r0);
          uint4 u[4][2];
          int spins = 0;
          for (;;) {
            bool all = true;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j < nb) {
                const uint4* src = reinterpret_cast<const uint4*>(slots + size_t(r0 + j) * r.max_bytes) + 2 * i;
                u[j][0] = __ldcv(src);
                u[j][1] = __ldcv(src + 1);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (j < nb)
                all = all && (u[j][0].y & 0xffffu) == tag && (u[j][0].w & 0xffffu) == tag && (u[j][1].y & 0xffffu) == tag &&
                      (u[j][1].w & 0xffffu) == tag;
            if (all) break;
            if (++spins > r.spin_limit) { atomicExch(r.status, TL_ERR_TIMEOUT); break; }
            __nanosleep(200);  // thousands of threads poll lines that a peer is writing: leave the L2 slice room
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // rank order: every rank computes the same bits
            if (j < nb) {
              float v[8];
              push_unpack(u[j][0].x, u[j][0].y, v[0], v[1]);
              push_unpack(u[j][0].z, u[j][0].w, v[2], v[3]);
              push_unpack(u[j][1].x, u[j][1].y, v[4], v[5]);
              push_unpack(u[j][1].z, u[j][1].w, v[6], v[7]);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[e] += v[e];
            }
          }
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (r.dtype == TL_F16) {
            const __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
            o[j] = *reinterpret_cast<const uint32_t*>(&h);
          } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            o[j] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        __stcg(reinterpret_cast<uint4*>(r.dst) + i, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      atomicAdd(words + 2 + half, 1u);  // also after a time-out: nobody must wait for this CTA
    }
  }
  if (tid == 0) {
    int spins = 0;
    while (int32_t(ld_acquire_gpu_u32(words + 2 + half) - uint32_t(r.nsum)) < 0) {
      if (++spins > r.spin_limit) { atomicExch(r.status, TL_ERR_TIMEOUT); break; }
      __nanosleep(64);  // hundreds of CTAs watch this word; the summing CTAs' arrivals must get through
    }
    if (blockIdx.x == 0) words[4] = epoch;  // the next push takes the other half
  }
  __syncthreads();
}

// MAXT / MINB: launch bounds.  The 4-warp configuration asks for 12 resident CTAs per SM
// (<= 42 registers) so that, under programmatic dependent launch, the CTAs of the NEXT kernel
// fit beside the 6-7 CTAs per SM of the running one and prefetch their weights early.
// PUSH: 0 plain store, 1 fused all-reduce (push, wait, sum), 2 push only (see above).  rin: the
// launch first reduces a pending push into its activation buffer (null for every other launch;
// the wrappers pass a literal, so the branch folds away).
template <typename AT, int NT, bool GROUPED, int S, int PUSH = 0>
__device__ __forceinline__ void ring_tile(const GemvArgs& p, const EpiParams& epi, int64_t tile_index, uint8_t* ring_raw,
                                          const PushArgs* q = nullptr, const ReduceIn* rin = nullptr) {
  uint4* ring = reinterpret_cast<uint4*>(ring_raw);  // [S][2][blockDim.x]
  const int nthreads = blockDim.x, tid = threadIdx.x;
  float* red = reinterpret_cast<float*>(ring_raw + size_t(S) * 2 * nthreads * 16);  // [warps][NT][4][32]
  const int warps = nthreads >> 5, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t tile_row = tile_index * 16;
  const int64_t r_lo = min(tile_row + g, int64_t(p.n) - 1);
  const int64_t r_hi = min(tile_row + g + 8, int64_t(p.n) - 1);
  const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(p.packed);
  const uint8_t* w_lo = wbytes + r_lo * p.k + 16 * t + warp * 64;
  const uint8_t* w_hi = wbytes + r_hi * p.k + 16 * t + warp * 64;
  const int kstride = warps * 64;  // bytes between this warp's consecutive k blocks
  const AT* a = reinterpret_cast<const AT*>(p.a);
  // MMA column c of a tile is batch row c.  Columns past m are never stored and no
  // column feeds another, so lanes past m simply re-read the last batch row instead
  // of branching to a zero fill.
  const AT* a_col[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) a_col[nt] = a + int64_t(min(g + 8 * nt, p.m - 1)) * p.k + 16 * t + warp * 64;
  const int kblocks = p.k >> 6;
  const int nkb = (kblocks - warp + warps - 1) / warps;  // k blocks of this warp
  const uint32_t ring_base = uint32_t(__cvta_generic_to_shared(ring)) + uint32_t(tid) * 16u;
  const uint32_t slot_bytes = uint32_t(nthreads) * 16u;  // one [blockDim] row of 16-byte words

  // let the next kernel in the stream start its own weight prefetch as early as possible
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
  for (int s = 0; s < S; ++s) {
    if (s < nkb) {
      cp_async16(ring_base + (2 * s) * slot_bytes, w_lo + int64_t(s) * kstride);
      cp_async16(ring_base + (2 * s + 1) * slot_bytes, w_hi + int64_t(s) * kstride);
    }
    cp_async_commit();
  }
  // The tile's per-channel scales and bias entries are read in the epilogue, at the very end of a
  // one-wave launch: a cold line there is an exposed DRAM round trip on every launch.  Ask for the
  // lines now (scales and bias are inputs, never a predecessor's output); no register stays live.
  if (tid == 0) {
    if (!GROUPED) prefetch_l1(reinterpret_cast<const uint8_t*>(p.scales) + size_t(tile_row) * (p.scales_dtype == TL_F32 ? 4 : 2));
    if (epi.fast_bias) prefetch_l1(epi.fast_bias + tile_row);
  }
  // weights never depend on the previous kernel; activations (its output) and our own stores do
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (rin) reduce_in_prologue(*rin);  // the activations are written by CTAs of THIS grid: read them through L2
  uint32_t push2_half = 0, push2_epoch = 0;
  if (PUSH == 2) {
    uint32_t* words = reinterpret_cast<uint32_t*>(q->base[q->rank] + tl_p2p_push_words_offset(q->max_bytes));
    const uint32_t ep = __ldcv(words + 4);  // epoch_p: stable while this kernel runs (its consumer bumps it); read through L2
    push2_half = ep & 1u;
    if (blockIdx.x == 0 && tid == 0) {
      words[2 + (push2_half ^ 1u)] = 0u;   // done[other half]
      words[5] = ep + 1u;                  // epoch_c, read by the consumer after this kernel has completed
    }
    push2_epoch = ep + 1u;
  }

  float total[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) total[nt][i] = 0.f;

  for (int i0 = 0; i0 < nkb; i0 += S) {
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int i = i0 + s;
      if (i < nkb) {
        uint4 bx[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4* src = reinterpret_cast<const uint4*>(a_col[nt] + int64_t(i) * kstride);
          // (written by CTAs of THIS grid before the gate: ordinary loads, never the non-coherent path;
          // no line of the buffer can be in this SM's L1 yet, the gate comes before the first read)
          bx[nt][0] = rin ? *src : __ldg(src);
          bx[nt][1] = rin ? *(src + 1) : __ldg(src + 1);
        }
        cp_async_wait<S - 1>();
        const uint4 wl = ring[(2 * s) * nthreads + tid];
        const uint4 wh = ring[(2 * s + 1) * nthreads + tid];
        float c[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) c[nt][e] = GROUPED ? 0.f : total[nt][e];
        const uint32_t wlo[4] = {wl.x, wl.y, wl.z, wl.w};
        const uint32_t whi[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a0, a1, a2, a3;
          MmaOps<AT>::cvt(wlo[j], a0, a2);
          MmaOps<AT>::cvt(whi[j], a1, a3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 v = bx[nt][j >> 1];
            const uint32_t b0 = (j & 1) ? v.z : v.x, b1 = (j & 1) ? v.w : v.y;
            MmaOps<AT>::mma(c[nt], a0, a1, a2, a3, b0, b1);
          }
        }
        // the slot's words now live in registers that have been consumed: refill it
        if (i + S < nkb) {
          cp_async16(ring_base + (2 * s) * slot_bytes, w_lo + int64_t(i + S) * kstride);
          cp_async16(ring_base + (2 * s + 1) * slot_bytes, w_hi + int64_t(i + S) * kstride);
        }
        cp_async_commit();
        if (GROUPED) {
          const int gi = ((warp + i * warps) * 64) / p.group;
          const float s_lo = tl_load_scale(p.scales, p.scales_dtype, r_lo * p.groups_per_row + gi);
          const float s_hi = tl_load_scale(p.scales, p.scales_dtype, r_hi * p.groups_per_row + gi);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            total[nt][0] = fmaf(s_lo, c[nt][0], total[nt][0]);
            total[nt][1] = fmaf(s_lo, c[nt][1], total[nt][1]);
            total[nt][2] = fmaf(s_hi, c[nt][2], total[nt][2]);
            total[nt][3] = fmaf(s_hi, c[nt][3], total[nt][3]);
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) total[nt][e] = c[nt][e];
        }
      } else {
        cp_async_commit();  // keeps the group count uniform for wait_group
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[((warp * NT + nt) * 4 + i) * 32 + lane] = total[nt][i];
  __syncthreads();
  // Fused all-reduce (PUSH): this tile's partial sums go, rounded to the output type, straight
  // into slot (half, rank) of EVERY rank's exchange buffer instead of into p.out.
  uint32_t push_epoch = 0;
  uint32_t* push_words = nullptr;
  __shared__ __align__(16) float push_stage[PUSH == 2 ? 16 : 8][16];  // PUSH == 2: [batch column][row of the tile], f32 partial sums
  if (PUSH == 1) {
    push_words = reinterpret_cast<uint32_t*>(q->base[q->rank] + tl_p2p_fused_offset(q->max_bytes));
    push_epoch = push_words[tile_index];  // owner-only counter; every thread reads it before thread 0 bumps it
  }
  const int push_half = int(push_epoch & 1u);
  for (int o = tid; o < NT * 128; o += nthreads) {
    const int nt = o >> 7, i = (o >> 5) & 3, ln = o & 31;
    float v = 0.f;
    for (int w = 0; w < warps; ++w) v += red[((w * NT + nt) * 4 + i) * 32 + ln];
    const int gg = ln >> 2, tt = ln & 3;
    const int64_t row = tile_row + gg + ((i & 2) ? 8 : 0);
    const int col = 8 * nt + 2 * tt + (i & 1);
    if (row < p.n && col < p.m) {
      float s = p.wscale;
      if (!GROUPED) s *= tl_load_scale(p.scales, p.scales_dtype, row);
      const float r = tl_apply_epilogue(epi, v * s, p.row0 + col, row, p.n);
      if (PUSH == 1) {
        for (int rr = 0; rr < q->world; ++rr)
          tl_store_out(q->base[rr] + tl_p2p_fused_slots_offset(q->max_bytes) + (size_t(push_half) * tl_ctx::kMaxPeers + q->rank) * q->max_bytes, p.out_dtype,
                       int64_t(col) * p.n + row, r);
      } else if (PUSH == 2) {
        push_stage[col][row - tile_row] = r;
      } else {
        tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + col) * p.n + row, r);
      }
    }
  }
  if (PUSH == 2) {
    // the tile [m columns][16 rows] leaves as 8-byte words {two partial sums, tag}, one copy per peer
    __syncthreads();
    const int per_peer = p.m * 8;
    const uint32_t tag = push_tag(push2_epoch);
    for (int idx = tid; idx < per_peer * q->world; idx += nthreads) {
      const int peer = idx / per_peer, v = idx - peer * per_peer, col = v >> 3, rp = v & 7;
      const uint2 word = push_pack(push_stage[col][2 * rp], push_stage[col][2 * rp + 1], tag);
      uint8_t* slot = q->base[peer] + tl_p2p_push_slots_offset(q->max_bytes) +
                      (size_t(push2_half) * tl_ctx::kMaxPeers + q->rank) * q->max_bytes;
      uint2* dst = reinterpret_cast<uint2*>(slot) + ((int64_t(col) * p.n + tile_row) >> 1) + rp;
      // volatile (relaxed at system scope): a weak store to peer memory may be held back indefinitely
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(word.x), "r"(word.y) : "memory");
    }
  }
  if (PUSH == 1) {
    // One arrival per rank on the tile's counter (release at system scope, cumulative over the
    // barrier, so the pushes above are visible first); then wait -- bounded -- until all ranks'
    // versions of THIS tile have arrived here, and sum them in rank order: every rank computes
    // the same bits, the ones the stand-alone all-reduce gives.  A CTA waits only for the same
    // tile of the other GPUs, never for a CTA of its own GPU.  Halves alternate per use of a
    // tile, so a rank that is one call ahead writes the other half.
    __shared__ int push_ok;
    __syncthreads();
    uint32_t* arrive_local = push_words + kP2PFusedMaxTiles + push_half * kP2PFusedMaxTiles + tile_index;
    if (tid == 0) {
      push_words[tile_index] = push_epoch + 1;
      push_ok = 1;
    }
    if (tid < q->world) {
      uint32_t* peer_words = reinterpret_cast<uint32_t*>(q->base[tid] + tl_p2p_fused_offset(q->max_bytes));
      push_red_release_sys(peer_words + kP2PFusedMaxTiles + push_half * kP2PFusedMaxTiles + tile_index, 1u);
    }
    __syncthreads();
    if (tid == 0) {
      const uint32_t want = uint32_t(q->world) * (push_epoch / 2 + 1);  // every use of (half, tile) adds `world` arrivals
      int spins = 0;
      while (int32_t(push_ld_acquire_sys(arrive_local) - want) < 0) {
        if (++spins > q->spin_limit) { push_ok = 0; atomicExch(q->status, TL_ERR_TIMEOUT); break; }
      }
    }
    __syncthreads();
    if (push_ok) {
      for (int o = tid; o < NT * 128; o += nthreads) {
        const int nt = o >> 7, i = (o >> 5) & 3, ln = o & 31;
        const int64_t row = tile_row + (ln >> 2) + ((i & 2) ? 8 : 0);
        const int col = 8 * nt + 2 * (ln & 3) + (i & 1);
        if (row < p.n && col < p.m) {
          const int64_t idx = int64_t(col) * p.n + row;
          float sum = 0.f;
          for (int rr = 0; rr < q->world; ++rr)
            sum += push_load(q->base[q->rank] + tl_p2p_fused_slots_offset(q->max_bytes) + (size_t(push_half) * tl_ctx::kMaxPeers + rr) * q->max_bytes, p.out_dtype, idx);
          tl_store_out(q->dst, p.out_dtype, idx, sum);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------

template <typename AT, int NT, bool GROUPED, int S, int MAXT = kMmaMaxWarps * 32, int MINB = 1>
__global__ void __launch_bounds__(MAXT, MINB) qgemv_ring_kernel(GemvArgs p, EpiParams epi) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  ring_tile<AT, NT, GROUPED, S>(p, epi, blockIdx.x, ring_smem);
}

// ---------------------------------------------------------------------------
// Wide ring tile: 32 weight rows per CTA (two MMA row tiles per warp and k block).
// From m = 8 up the activation fragments weigh as much as the weights (m x 64 x 2 bytes against
// 16 x 64 per warp and k block) and, re-read by every 16-row tile, they make L2 -> SM traffic
// and load-store issue the limit instead of HBM: 5.0 TB/s at m = 8 and 4.1 TB/s at m = 16 on a
// 622 MB matrix against 6.5 TB/s at m = 1.  Here one activation fragment feeds two row tiles:
// half the activation traffic and twice the independent MMA work per load.  Same fragment
// mapping, k interleave and summation order as ring_tile, so the outputs have the same bits.
// ---------------------------------------------------------------------------
template <typename AT, int NT, bool GROUPED, int S>
__device__ __forceinline__ void ring_tile2(const GemvArgs& p, const EpiParams& epi, int64_t tile_index, uint8_t* ring_raw) {
  uint4* ring = reinterpret_cast<uint4*>(ring_raw);  // [S][4][blockDim.x]
  const int nthreads = blockDim.x, tid = threadIdx.x;
  float* red = reinterpret_cast<float*>(ring_raw + size_t(S) * 4 * nthreads * 16);  // [warps][2][NT][4][32]
  const int warps = nthreads >> 5, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t tile_row = tile_index * 32;
  const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(p.packed);
  int64_t rows[4];
  const uint8_t* wp[4];  // rows g, g+8 (first row tile), g+16, g+24 (second)
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    rows[r] = min(tile_row + g + 8 * r, int64_t(p.n) - 1);
    wp[r] = wbytes + rows[r] * p.k + 16 * t + warp * 64;
  }
  const int kstride = warps * 64;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const AT* a_col[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) a_col[nt] = a + int64_t(min(g + 8 * nt, p.m - 1)) * p.k + 16 * t + warp * 64;
  const int kblocks = p.k >> 6;
  const int nkb = (kblocks - warp + warps - 1) / warps;
  const uint32_t ring_base = uint32_t(__cvta_generic_to_shared(ring)) + uint32_t(tid) * 16u;
  const uint32_t slot_bytes = uint32_t(nthreads) * 16u;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
  for (int s = 0; s < S; ++s) {
    if (s < nkb) {
#pragma unroll
      for (int r = 0; r < 4; ++r) cp_async16(ring_base + (4 * s + r) * slot_bytes, wp[r] + int64_t(s) * kstride);
    }
    cp_async_commit();
  }
  if (tid == 0) {  // the epilogue's scales and bias entries: see ring_tile
    if (!GROUPED) prefetch_l1(reinterpret_cast<const uint8_t*>(p.scales) + size_t(tile_row) * (p.scales_dtype == TL_F32 ? 4 : 2));
    if (epi.fast_bias) prefetch_l1(epi.fast_bias + tile_row);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float total[2][NT][4];
#pragma unroll
  for (int rt = 0; rt < 2; ++rt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) total[rt][nt][i] = 0.f;

  for (int i0 = 0; i0 < nkb; i0 += S) {
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int i = i0 + s;
      if (i < nkb) {
        uint4 bx[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4* src = reinterpret_cast<const uint4*>(a_col[nt] + int64_t(i) * kstride);
          bx[nt][0] = __ldg(src);
          bx[nt][1] = __ldg(src + 1);
        }
        cp_async_wait<S - 1>();
#pragma unroll
        for (int rt = 0; rt < 2; ++rt) {
          const uint4 wl = ring[(4 * s + 2 * rt) * nthreads + tid];
          const uint4 wh = ring[(4 * s + 2 * rt + 1) * nthreads + tid];
          float c[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) c[nt][e] = GROUPED ? 0.f : total[rt][nt][e];
          const uint32_t wlo[4] = {wl.x, wl.y, wl.z, wl.w};
          const uint32_t whi[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t a0, a1, a2, a3;
            MmaOps<AT>::cvt(wlo[j], a0, a2);
            MmaOps<AT>::cvt(whi[j], a1, a3);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint4 v = bx[nt][j >> 1];
              const uint32_t b0 = (j & 1) ? v.z : v.x, b1 = (j & 1) ? v.w : v.y;
              MmaOps<AT>::mma(c[nt], a0, a1, a2, a3, b0, b1);
            }
          }
          if (GROUPED) {
            const int gi = ((warp + i * warps) * 64) / p.group;
            const float s_lo = tl_load_scale(p.scales, p.scales_dtype, rows[2 * rt] * p.groups_per_row + gi);
            const float s_hi = tl_load_scale(p.scales, p.scales_dtype, rows[2 * rt + 1] * p.groups_per_row + gi);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              total[rt][nt][0] = fmaf(s_lo, c[nt][0], total[rt][nt][0]);
              total[rt][nt][1] = fmaf(s_lo, c[nt][1], total[rt][nt][1]);
              total[rt][nt][2] = fmaf(s_hi, c[nt][2], total[rt][nt][2]);
              total[rt][nt][3] = fmaf(s_hi, c[nt][3], total[rt][nt][3]);
            }
          } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e) total[rt][nt][e] = c[nt][e];
          }
        }
        if (i + S < nkb) {
#pragma unroll
          for (int r = 0; r < 4; ++r) cp_async16(ring_base + (4 * s + r) * slot_bytes, wp[r] + int64_t(i + S) * kstride);
        }
        cp_async_commit();
      } else {
        cp_async_commit();
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int rt = 0; rt < 2; ++rt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[(((warp * 2 + rt) * NT + nt) * 4 + i) * 32 + lane] = total[rt][nt][i];
  __syncthreads();
  for (int o = tid; o < 2 * NT * 128; o += nthreads) {
    const int rt = o / (NT * 128), o1 = o - rt * (NT * 128);
    const int nt = o1 >> 7, i = (o1 >> 5) & 3, ln = o1 & 31;
    float v = 0.f;
    for (int w = 0; w < warps; ++w) v += red[(((w * 2 + rt) * NT + nt) * 4 + i) * 32 + ln];
    const int gg = ln >> 2, tt = ln & 3;
    const int64_t row = tile_row + 16 * rt + gg + ((i & 2) ? 8 : 0);
    const int col = 8 * nt + 2 * tt + (i & 1);
    if (row < p.n && col < p.m) {
      float sc = p.wscale;
      if (!GROUPED) sc *= tl_load_scale(p.scales, p.scales_dtype, row);
      const float r = tl_apply_epilogue(epi, v * sc, p.row0 + col, row, p.n);
      tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + col) * p.n + row, r);
    }
  }
}

template <typename AT, int NT, bool GROUPED, int S>
__global__ void __launch_bounds__(kMmaMaxWarps * 32) qgemv_ring2_kernel(GemvArgs p, EpiParams epi) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  ring_tile2<AT, NT, GROUPED, S>(p, epi, blockIdx.x, ring_smem);
}

// Row-parallel projection fused with its all-reduce (tensor parallelism, o / down): every CTA
// computes its 16-row tile of the local partial product, pushes it into all ranks' exchange
// buffers over NVLink (plain peer stores), signals, waits for the other ranks' versions of the
// same tile and writes the summed tile -- one kernel where a GEMV and an all-reduce kernel ran.
// Two resident CTAs of 512 threads per SM (64 registers) keep the 256-tile projections in one wave.
template <typename AT, int NT, bool GROUPED, int S>
__global__ void __launch_bounds__(kMmaMaxWarps * 32, 2) qgemv_ring_allreduce_kernel(GemvArgs p, EpiParams epi, PushArgs q) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  ring_tile<AT, NT, GROUPED, S, 1>(p, epi, blockIdx.x, ring_smem, &q);
}

// Row-parallel projection that only pushes its partial tiles to every rank (PUSH == 2).
template <typename AT, int NT, bool GROUPED, int S>
__global__ void __launch_bounds__(kMmaMaxWarps * 32, 2) qgemv_ring_push_kernel(GemvArgs p, EpiParams epi, PushArgs q) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  ring_tile<AT, NT, GROUPED, S, 2>(p, epi, blockIdx.x, ring_smem, &q);
}
// A launch that first reduces a pending push into its activations (reduce-on-read), one matrix.
template <typename AT, int NT, bool GROUPED, int S>
__global__ void __launch_bounds__(kMmaMaxWarps * 32) qgemv_ring_rin_kernel(GemvArgs p, EpiParams epi, const __grid_constant__ ReduceIn rin) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  ring_tile<AT, NT, GROUPED, S, 0>(p, epi, blockIdx.x, ring_smem, nullptr, &rin);
}

// Horizontal fusion: up to four projections that read the SAME activations (q/k/v, gate/up) in
// one launch.  CTA b works on tile b - tile_start[i] of item i; each item keeps its own weight,
// scales, output, alpha and epilogue.
constexpr int kMaxBatchItems = 4;
struct RingBatchArgs {
  GemvArgs p[kMaxBatchItems];
  EpiParams e[kMaxBatchItems];
  int32_t tile_start[kMaxBatchItems + 1];
};
template <typename AT, int NT, bool GROUPED, int S>
__global__ void __launch_bounds__(kMmaMaxWarps * 32) qgemv_ring_batched_kernel(const __grid_constant__ RingBatchArgs b) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  const int blk = int(blockIdx.x);
  const int i = (blk >= b.tile_start[1]) + (blk >= b.tile_start[2]) + (blk >= b.tile_start[3]);
  ring_tile<AT, NT, GROUPED, S>(b.p[i], b.e[i], blk - b.tile_start[i], ring_smem);
}
// the batched launch with the reduce-on-read prologue
template <typename AT, int NT, bool GROUPED, int S>
__global__ void __launch_bounds__(kMmaMaxWarps * 32) qgemv_ring_rin_batched_kernel(const __grid_constant__ RingBatchArgs b,
                                                                                   const __grid_constant__ ReduceIn rin) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  const int blk = int(blockIdx.x);
  const int i = (blk >= b.tile_start[1]) + (blk >= b.tile_start[2]) + (blk >= b.tile_start[3]);
  ring_tile<AT, NT, GROUPED, S, 0>(b.p[i], b.e[i], blk - b.tile_start[i], ring_smem, nullptr, &rin);
}
// the same with 32-row tiles (tile_start counts 32-row tiles)
template <typename AT, int NT, bool GROUPED, int S>
__global__ void __launch_bounds__(kMmaMaxWarps * 32) qgemv_ring2_batched_kernel(const __grid_constant__ RingBatchArgs b) {
  extern __shared__ __align__(16) uint8_t ring_smem[];
  const int blk = int(blockIdx.x);
  const int i = (blk >= b.tile_start[1]) + (blk >= b.tile_start[2]) + (blk >= b.tile_start[3]);
  ring_tile2<AT, NT, GROUPED, S>(b.p[i], b.e[i], blk - b.tile_start[i], ring_smem);
}

// ---------------------------------------------------------------------------
// 5: TMA-fed persistent kernel ("tma").
//
// A producer thread streams the weight with 2-D tensor-map TMA loads: one box is
// 256 rows x 128 bytes (32 KB, 128-byte swizzle), the size at which a single
// load per SM at a time already saturates HBM.  STAGES boxes are in flight per SM
// (192 KB at 6 stages) and cost no registers and almost no issue slots.  Boxes
// are numbered with k fastest inside a 256-row band; the persistent grid deals
// the flat range out in equal contiguous shares (no wave quantisation).
//
// Sixteen consumer warps own 16 rows of the band each (one MMA tile, weights as the
// A operand as in kernel 2) for the whole k range, so warps never reduce
// across each other.  A warp whose CTA covered only part of a band's k range adds
// its partial sums to the zero-initialised scratch and bumps its (band, warp)
// counter; the warp that completes the count finalises.  Nobody waits on anybody.
//
// Shared-memory reads are conflict-free: with the 128-byte swizzle the 16-byte
// chunk c of row r sits at chunk c ^ (r & 7).  Per-channel scales: thread (g,t)
// reads chunks 2t and 2t+1 of rows g and g+8 (32 contiguous weight bytes, k order
// permuted identically for the activations).  Grouped scales need every MMA to
// stay inside one 64-wide group, so there the thread reads chunk 4h+t for half h.
// ---------------------------------------------------------------------------
constexpr int kTmaBoxRows = 256, kTmaBoxBytes = 128, kTmaStageBytes = kTmaBoxRows * kTmaBoxBytes;
constexpr int kTmaConsumerWarps = 16;

struct TmaArgs {
  float* scratch;      // [m, n] f32, all zero between launches
  unsigned* counters;  // [bands * consumer warps], all zero between launches
  int* status;         // device error word (0 = ok)
  int32_t spb;         // stages (boxes) per band = k / 128
  int32_t total_stages;
};

template <typename AT, int NT, bool GROUPED, int STAGES>
__global__ void __launch_bounds__((kTmaConsumerWarps + 1) * 32, 1)
qgemv_tma_kernel(const __grid_constant__ CUtensorMap wmap, GemvArgs p, EpiParams epi, TmaArgs ta) {
  extern __shared__ uint8_t tma_smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ int abort_flag;
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tma_smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t T = ta.total_stages;
  const int i0 = int(T * blockIdx.x / gridDim.x), i1 = int(T * (blockIdx.x + 1) / gridDim.x);
  const int n = i1 - i0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kTmaConsumerWarps);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (n <= 0) return;

  if (warp == kTmaConsumerWarps) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&wmap);
      for (int i = 0; i < n; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES && !mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, &abort_flag)) {
          if (!abort_flag) { abort_flag = 1; atomicExch(ta.status, TL_DEV_TIMEOUT_EMPTY); }
          break;
        }
        const int gi = i0 + i;
        mbar_expect_tx(&full_bar[s], kTmaStageBytes);
        tma_load_2d(stages + size_t(s) * kTmaStageBytes, &wmap, (gi % ta.spb) * kTmaBoxBytes,
                    (gi / ta.spb) * kTmaBoxRows, &full_bar[s]);
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  const int g = lane >> 2, t = lane & 3;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const AT* a_col[NT];
  bool a_ok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    a_ok[nt] = (g + 8 * nt) < p.m;
    a_col[nt] = a + int64_t(a_ok[nt] ? g + 8 * nt : 0) * p.k;
  }
  const uint32_t row_off = uint32_t(warp * 16 + g) * kTmaBoxBytes;  // + 8*128 for the high row
  // byte offsets of this thread's 16-byte chunks inside a swizzled 128-byte row
  const uint32_t c32_0 = uint32_t((2 * t) ^ g) << 4, c32_1 = c32_0 ^ 16u;        // chunks 2t, 2t+1
  const uint32_t c16_0 = uint32_t(t ^ g) << 4, c16_1 = uint32_t((4 + t) ^ g) << 4;  // chunks t, 4+t

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
  int mine = 0;

  for (int i = 0; i < n; ++i) {
    const int s = i % STAGES;
    const int gi = i0 + i, band = gi / ta.spb, ks = gi - band * ta.spb;
    // activations of this 128-wide k block (independent of the weight stream: load first)
    uint32_t xb[NT][16];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (GROUPED) {
        const uint4* s0 = reinterpret_cast<const uint4*>(a_col[nt] + ks * 128 + 16 * t);
        const uint4* s1 = reinterpret_cast<const uint4*>(a_col[nt] + ks * 128 + 64 + 16 * t);
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const uint4 q0 = a_ok[nt] ? __ldg(s0 + v) : make_uint4(0, 0, 0, 0);
          const uint4 q1 = a_ok[nt] ? __ldg(s1 + v) : make_uint4(0, 0, 0, 0);
          xb[nt][4 * v] = q0.x; xb[nt][4 * v + 1] = q0.y; xb[nt][4 * v + 2] = q0.z; xb[nt][4 * v + 3] = q0.w;
          xb[nt][8 + 4 * v] = q1.x; xb[nt][8 + 4 * v + 1] = q1.y; xb[nt][8 + 4 * v + 2] = q1.z; xb[nt][8 + 4 * v + 3] = q1.w;
        }
      } else {
        const uint4* s0 = reinterpret_cast<const uint4*>(a_col[nt] + ks * 128 + 32 * t);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 q0 = a_ok[nt] ? __ldg(s0 + v) : make_uint4(0, 0, 0, 0);
          xb[nt][4 * v] = q0.x; xb[nt][4 * v + 1] = q0.y; xb[nt][4 * v + 2] = q0.z; xb[nt][4 * v + 3] = q0.w;
        }
      }
    }
    if (!mbar_wait(&full_bar[s], (i / STAGES) & 1, &abort_flag)) {
      if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(ta.status, TL_DEV_TIMEOUT_FULL); }
      return;
    }
    const uint32_t sb = smem_u32(stages + size_t(s) * kTmaStageBytes) + row_off;
    uint4 wl[2], wh[2];
    {
      const uint32_t lo = sb, hi = sb + 8 * kTmaBoxBytes;
      wl[0] = lds128(lo + (GROUPED ? c16_0 : c32_0));
      wl[1] = lds128(lo + (GROUPED ? c16_1 : c32_1));
      wh[0] = lds128(hi + (GROUPED ? c16_0 : c32_0));
      wh[1] = lds128(hi + (GROUPED ? c16_1 : c32_1));
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);  // the words are in registers: the box may be refilled

    {
      const uint32_t wlo[8] = {wl[0].x, wl[0].y, wl[0].z, wl[0].w, wl[1].x, wl[1].y, wl[1].z, wl[1].w};
      const uint32_t whi[8] = {wh[0].x, wh[0].y, wh[0].z, wh[0].w, wh[1].x, wh[1].y, wh[1].z, wh[1].w};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float c[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) c[nt][e] = GROUPED ? 0.f : acc[nt][e];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = 4 * h + jj;
          uint32_t a0, a1, a2, a3;
          MmaOps<AT>::cvt(wlo[j], a0, a2);
          MmaOps<AT>::cvt(whi[j], a1, a3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) MmaOps<AT>::mma(c[nt], a0, a1, a2, a3, xb[nt][2 * j], xb[nt][2 * j + 1]);
        }
        if (GROUPED) {
          const int grp = (ks * 128 + h * 64) / p.group;
          const int64_t r_lo = min(int64_t(band) * kTmaBoxRows + warp * 16 + g, int64_t(p.n) - 1);
          const int64_t r_hi = min(r_lo + 8, int64_t(p.n) - 1);
          const float s_lo = tl_load_scale(p.scales, p.scales_dtype, r_lo * p.groups_per_row + grp);
          const float s_hi = tl_load_scale(p.scales, p.scales_dtype, r_hi * p.groups_per_row + grp);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            acc[nt][0] = fmaf(s_lo, c[nt][0], acc[nt][0]);
            acc[nt][1] = fmaf(s_lo, c[nt][1], acc[nt][1]);
            acc[nt][2] = fmaf(s_hi, c[nt][2], acc[nt][2]);
            acc[nt][3] = fmaf(s_hi, c[nt][3], acc[nt][3]);
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = c[nt][e];
        }
      }
    }
    ++mine;

    if (ks + 1 == ta.spb || i + 1 == n) {
      // flush this warp's 32 rows of the band
      bool finalize = (mine == ta.spb);
      if (!finalize) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int64_t row = int64_t(band) * kTmaBoxRows + warp * 16 + g + ((e & 2) ? 8 : 0);
              const int col = 8 * nt + 2 * t + (e & 1);
              if (row < p.n && col < p.m) atomicAdd(ta.scratch + int64_t(col) * p.n + row, acc[nt][e]);
            }
        __threadfence();
        __syncwarp();  // every lane's partial sums are published before the count moves
        unsigned old = 0;
        if (lane == 0) old = atomicAdd(ta.counters + band * kTmaConsumerWarps + warp, unsigned(mine));
        old = __shfl_sync(0xffffffffu, old, 0);
        finalize = (old + unsigned(mine) == unsigned(ta.spb));
        if (finalize) {
          __threadfence();
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int64_t row = int64_t(band) * kTmaBoxRows + warp * 16 + g + ((e & 2) ? 8 : 0);
                const int col = 8 * nt + 2 * t + (e & 1);
                if (row < p.n && col < p.m) {
                  float* sp = ta.scratch + int64_t(col) * p.n + row;
                  acc[nt][e] = __ldcg(sp);
                  __stcg(sp, 0.f);
                }
              }
          if (lane == 0) ta.counters[band * kTmaConsumerWarps + warp] = 0;
        }
      }
      if (finalize) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int64_t row = int64_t(band) * kTmaBoxRows + warp * 16 + g + ((e & 2) ? 8 : 0);
              const int col = 8 * nt + 2 * t + (e & 1);
              if (row < p.n && col < p.m) {
                float sc = p.wscale;
                if (!GROUPED) sc *= tl_load_scale(p.scales, p.scales_dtype, row);
                const float o = tl_apply_epilogue(epi, acc[nt][e] * sc, p.row0 + col, row, p.n);
                tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + col) * p.n + row, o);
              }
            }
      }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
      mine = 0;
    }
  }
}

// ---------------------------------------------------------------------------
// 6: contiguous bulk-copy persistent kernel ("bulk").
//
// Eight consecutive weight rows are one contiguous block of 8*K bytes.  A stage is
// RT such blocks (about 32 KB or more), fetched with plain cp.async.bulk copies of
// whole contiguous memory -- the access pattern HBM likes best -- into a ring of
// shared-memory stages.  Stages are dealt to a persistent grid (one CTA per SM) in
// equal contiguous shares.  Every stage holds complete rows, so no partial sums
// ever cross CTAs: no scratch, no atomics.
//
// The batch is the 16-row MMA A operand and 8 weight rows are the B operand.
// P consumer warps split the k range of a tile (128-wide k blocks, interleaved),
// Q = W/P tiles are worked on at once; the P partial fragments of a tile meet in a
// double-buffered shared array after one named barrier per stage, where
// scale + epilogue + store happen.
// ---------------------------------------------------------------------------
struct BulkArgs {
  int* status;
  int32_t rt;            // 8-row tiles per stage
  int32_t total_stages;
  int32_t kb128;         // k / 128
  int32_t p;             // warps per tile
  uint32_t stage_bytes;  // rt * 8 * k
};

template <typename AT, bool M16, bool GROUPED>
__global__ void __launch_bounds__(17 * 32, 1) qgemv_bulk_kernel(GemvArgs p, EpiParams epi, BulkArgs ba, int nstages,
                                                               int cwarps) {
  extern __shared__ uint8_t bulk_smem_raw[];
  __shared__ uint64_t full_bar[8], empty_bar[8];
  __shared__ int abort_flag;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bulk_smem_raw) + 127) & ~uintptr_t(127));
  // layout: [nstages][stage_bytes] weights, then red[2][rt][p][128] floats
  float* red = reinterpret_cast<float*>(base + size_t(nstages) * ba.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t T = ba.total_stages;
  const int i0 = int(T * blockIdx.x / gridDim.x), i1 = int(T * (blockIdx.x + 1) / gridDim.x);
  const int n = i1 - i0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], cwarps);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (n <= 0) return;
  const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(p.packed);
  const int64_t total_bytes = int64_t(p.n) * p.k;

  if (warp == cwarps) {
    // ---------------- producer ----------------
    if (lane == 0) {
      for (int i = 0; i < n; ++i) {
        const int s = i % nstages;
        if (i >= nstages && !mbar_wait(&empty_bar[s], ((i / nstages) - 1) & 1, &abort_flag)) {
          if (!abort_flag) { abort_flag = 1; atomicExch(ba.status, TL_DEV_TIMEOUT_EMPTY); }
          break;
        }
        const int64_t off = int64_t(i0 + i) * ba.stage_bytes;
        const uint32_t bytes = uint32_t(min(int64_t(ba.stage_bytes), total_bytes - off));  // the last stage may be short
        mbar_expect_tx(&full_bar[s], bytes);
        uint8_t* dst = base + size_t(s) * ba.stage_bytes;
        for (uint32_t o = 0; o < bytes; o += 32768u) {
          const uint32_t piece = min(32768u, bytes - o);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(dst + o)), "l"(wbytes + off + o), "r"(piece), "r"(smem_u32(&full_bar[s]))
                       : "memory");
        }
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  const int g = lane >> 2, t = lane & 3;
  const int kp = warp % ba.p, tq = warp / ba.p, q = cwarps / ba.p;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const bool lo_ok = g < p.m, hi_ok = M16 && (g + 8) < p.m;
  const AT* a_lo = a + int64_t(lo_ok ? g : 0) * p.k;
  const AT* a_hi = a + int64_t(hi_ok ? g + 8 : 0) * p.k;
  const int cthreads = cwarps * 32;

  for (int i = 0; i < n; ++i) {
    const int s = i % nstages;
    if (!mbar_wait(&full_bar[s], (i / nstages) & 1, &abort_flag)) {
      if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(ba.status, TL_DEV_TIMEOUT_FULL); }
      return;
    }
    const uint32_t sb = smem_u32(base + size_t(s) * ba.stage_bytes);
    float* redbuf = red + size_t(i & 1) * ba.rt * ba.p * 128;
    const int64_t row0 = int64_t(i0 + i) * ba.rt * 8;  // first weight row of this stage
    for (int tile = tq; tile < ba.rt; tile += q) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t trow = sb + uint32_t(tile * 8 + g) * uint32_t(p.k);
      for (int kb = kp; kb < ba.kb128; kb += ba.p) {
        uint32_t xl[16], xh[16], w8[8];
        if (GROUPED) {
          // 16-byte chunks: half h covers k = 128*kb + 64*h + 16*t .. +16
          const uint4 w0 = lds128(trow + kb * 128 + 16 * t), w1 = lds128(trow + kb * 128 + 64 + 16 * t);
          w8[0] = w0.x; w8[1] = w0.y; w8[2] = w0.z; w8[3] = w0.w; w8[4] = w1.x; w8[5] = w1.y; w8[6] = w1.z; w8[7] = w1.w;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4* s0 = reinterpret_cast<const uint4*>(a_lo + kb * 128 + 64 * h + 16 * t);
            const uint4* s1 = reinterpret_cast<const uint4*>(a_hi + kb * 128 + 64 * h + 16 * t);
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              const uint4 l4 = lo_ok ? __ldg(s0 + v) : make_uint4(0, 0, 0, 0);
              const uint4 h4 = hi_ok ? __ldg(s1 + v) : make_uint4(0, 0, 0, 0);
              const int b = 8 * h + 4 * v;
              xl[b] = l4.x; xl[b + 1] = l4.y; xl[b + 2] = l4.z; xl[b + 3] = l4.w;
              xh[b] = h4.x; xh[b + 1] = h4.y; xh[b + 2] = h4.z; xh[b + 3] = h4.w;
            }
          }
        } else {
          // 32 contiguous bytes: k = 128*kb + 32*t .. +32
          const uint4 w0 = lds128(trow + kb * 128 + 32 * t), w1 = lds128(trow + kb * 128 + 32 * t + 16);
          w8[0] = w0.x; w8[1] = w0.y; w8[2] = w0.z; w8[3] = w0.w; w8[4] = w1.x; w8[5] = w1.y; w8[6] = w1.z; w8[7] = w1.w;
          const uint4* s0 = reinterpret_cast<const uint4*>(a_lo + kb * 128 + 32 * t);
          const uint4* s1 = reinterpret_cast<const uint4*>(a_hi + kb * 128 + 32 * t);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 l4 = lo_ok ? __ldg(s0 + v) : make_uint4(0, 0, 0, 0);
            const uint4 h4 = hi_ok ? __ldg(s1 + v) : make_uint4(0, 0, 0, 0);
            xl[4 * v] = l4.x; xl[4 * v + 1] = l4.y; xl[4 * v + 2] = l4.z; xl[4 * v + 3] = l4.w;
            xh[4 * v] = h4.x; xh[4 * v + 1] = h4.y; xh[4 * v + 2] = h4.z; xh[4 * v + 3] = h4.w;
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float c[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) c[e] = GROUPED ? 0.f : acc[e];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int j = 4 * h + jj;
            uint32_t b0, b1;
            MmaOps<AT>::cvt(w8[j], b0, b1);
            MmaOps<AT>::mma(c, xl[2 * j], xh[2 * j], xl[2 * j + 1], xh[2 * j + 1], b0, b1);
          }
          if (GROUPED) {
            const int grp = (kb * 128 + h * 64) / p.group;
            const int64_t r0 = min(row0 + tile * 8 + 2 * t, int64_t(p.n) - 1), r1 = min(r0 + 1, int64_t(p.n) - 1);
            const float s0 = tl_load_scale(p.scales, p.scales_dtype, r0 * p.groups_per_row + grp);
            const float s1 = tl_load_scale(p.scales, p.scales_dtype, r1 * p.groups_per_row + grp);
            acc[0] = fmaf(s0, c[0], acc[0]);
            acc[1] = fmaf(s1, c[1], acc[1]);
            acc[2] = fmaf(s0, c[2], acc[2]);
            acc[3] = fmaf(s1, c[3], acc[3]);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = c[e];
          }
        }
      }
      float* dst = redbuf + (size_t(tile) * ba.p + kp) * 128;
#pragma unroll
      for (int e = 0; e < 4; ++e) dst[e * 32 + lane] = acc[e];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);  // this warp no longer reads the stage
    asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
    // reduce the P partial fragments of every tile of the stage, then scale + epilogue + store
    for (int o = threadIdx.x; o < ba.rt * 128; o += cthreads) {
      const int tile = o >> 7, e = (o >> 5) & 3, ln = o & 31;
      const float* src = redbuf + size_t(tile) * ba.p * 128 + e * 32 + ln;
      float v = 0.f;
      for (int w = 0; w < ba.p; ++w) v += src[w * 128];
      const int gg = ln >> 2, tt = ln & 3;
      const int col = gg + ((e & 2) ? 8 : 0);                      // batch row
      const int64_t row = row0 + tile * 8 + 2 * tt + (e & 1);      // weight row = output column
      if (row < p.n && col < p.m) {
        float sc = p.wscale;
        if (!GROUPED) sc *= tl_load_scale(p.scales, p.scales_dtype, row);
        const float r = tl_apply_epilogue(epi, v * sc, p.row0 + col, row, p.n);
        tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + col) * p.n + row, r);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// Launched with programmatic stream serialisation: the kernel may start while its predecessor
// in the stream is still draining, prefetches its weights (which depend on nothing), and only
// then waits (griddepcontrol.wait) for the predecessor before it touches activations or writes.
template <typename K>
void launch_with_smem(K kernel, int grid, int block, size_t smem, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, p, e);
}
template <typename AT, int NT, bool GROUPED>
void launch_ring_s(int depth, int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  const size_t smem = size_t(depth >= 8 ? 8 : depth >= 6 ? 6 : depth >= 4 ? 4 : 2) * 2 * block * 16 + size_t(block / 32) * NT * 128 * 4;
  if (depth >= 8) launch_with_smem(qgemv_ring_kernel<AT, NT, GROUPED, 8>, grid, block, smem, s, p, e);
  else if (depth >= 6) launch_with_smem(qgemv_ring_kernel<AT, NT, GROUPED, 6>, grid, block, smem, s, p, e);
  else if (depth >= 4) launch_with_smem(qgemv_ring_kernel<AT, NT, GROUPED, 4>, grid, block, smem, s, p, e);
  else launch_with_smem(qgemv_ring_kernel<AT, NT, GROUPED, 2>, grid, block, smem, s, p, e);
}
template <typename AT>
void launch_ring(bool two, bool grouped, int depth, int grid, int block, cudaStream_t s, const GemvArgs& p,
                 const EpiParams& e) {
  if (two) {
    if (grouped) launch_ring_s<AT, 2, true>(depth, grid, block, s, p, e);
    else launch_ring_s<AT, 2, false>(depth, grid, block, s, p, e);
  } else {
    if (grouped) launch_ring_s<AT, 1, true>(depth, grid, block, s, p, e);
    else launch_ring_s<AT, 1, false>(depth, grid, block, s, p, e);
  }
}

// ---------------------------------------------------------------------------
// Shape of a ring launch: W warps per 16-row tile, S k blocks in flight per thread.
// A launch whose CTAs are all resident at once has no tail wave, and a tail wave of a few
// CTAs runs at one thread's latency-bound pace: on the decode stack the gate+up launch
// (1536 tiles) took 27 us with 10 resident CTAs per SM (44 registers, 56 CTAs left over) and
// 19 us with 12 (40 registers).  So: the widest CTA (shortest k loop per warp) whose launch
// fits in one wave, and for it the deepest ring that still fits -- asked of the occupancy
// calculator, which knows the registers of each instantiation.  Matrices too large for one
// wave take 4-warp CTAs with the ring sized by shared memory.
// ---------------------------------------------------------------------------
template <typename AT, int NT, bool GROUPED>
const void* ring_kernel_ptr_d(bool batched, int depth) {
  switch (depth) {
    case 8: return batched ? reinterpret_cast<const void*>(&qgemv_ring_batched_kernel<AT, NT, GROUPED, 8>)
                           : reinterpret_cast<const void*>(&qgemv_ring_kernel<AT, NT, GROUPED, 8>);
    case 6: return batched ? reinterpret_cast<const void*>(&qgemv_ring_batched_kernel<AT, NT, GROUPED, 6>)
                           : reinterpret_cast<const void*>(&qgemv_ring_kernel<AT, NT, GROUPED, 6>);
    case 4: return batched ? reinterpret_cast<const void*>(&qgemv_ring_batched_kernel<AT, NT, GROUPED, 4>)
                           : reinterpret_cast<const void*>(&qgemv_ring_kernel<AT, NT, GROUPED, 4>);
    default: return batched ? reinterpret_cast<const void*>(&qgemv_ring_batched_kernel<AT, NT, GROUPED, 2>)
                            : reinterpret_cast<const void*>(&qgemv_ring_kernel<AT, NT, GROUPED, 2>);
  }
}
template <typename AT>
const void* ring_kernel_ptr_at(bool batched, bool two, bool grouped, int depth) {
  if (two) return grouped ? ring_kernel_ptr_d<AT, 2, true>(batched, depth) : ring_kernel_ptr_d<AT, 2, false>(batched, depth);
  return grouped ? ring_kernel_ptr_d<AT, 1, true>(batched, depth) : ring_kernel_ptr_d<AT, 1, false>(batched, depth);
}
inline size_t ring_smem_bytes(int warps, int depth, bool two) {
  return size_t(depth) * 2 * warps * 32 * 16 + size_t(warps) * (two ? 2 : 1) * 128 * 4;
}
int ring_occupancy(tl_ctx* ctx, bool batched, int a_dtype, bool two, bool grouped, int warps, int depth) {
  const int key = (batched ? 1 : 0) | (a_dtype == TL_F16 ? 2 : 0) | (two ? 4 : 0) | (grouped ? 8 : 0) | (warps << 4) | (depth << 10);
  auto it = ctx->ring_occupancy.find(key);
  if (it != ctx->ring_occupancy.end()) return it->second;
  const void* kern = a_dtype == TL_F16 ? ring_kernel_ptr_at<__half>(batched, two, grouped, depth)
                                       : ring_kernel_ptr_at<__nv_bfloat16>(batched, two, grouped, depth);
  const size_t smem = ring_smem_bytes(warps, depth, two);
  int occ = 0;
  if (smem <= 227 * 1024) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, warps * 32, smem) != cudaSuccess) {
      cudaGetLastError();
      occ = 0;
    }
  }
  ctx->ring_occupancy[key] = occ;
  return occ;
}
void ring_pick_shape(tl_ctx* ctx, bool batched, int a_dtype, int m, bool grouped, int64_t tiles, int64_t k, int* warps,
                     int* depth, int* wide = nullptr) {
  if (wide) *wide = 0;
  const bool two = m > 8;
  const int kblocks = int(k >> 6);
  if (wide && two && tiles <= 2 * int64_t(ctx->sm_count)) {
    // Two token tiles on a matrix of few tiles (4096 rows): 32-row tiles, where one activation
    // fragment feeds two row tiles, measured 17.3 against 22.0 us (4096 x 14336, m = 16).
    *wide = 1; *warps = 16; *depth = 4;
    return;
  }
  for (int w : {16, 8, 4}) {
    const int nkb = (kblocks + w - 1) / w;  // k blocks of one warp
    for (int s : {8, 6, 4, 2}) {
      if (s > 2 && s - 2 >= nkb) continue;  // a shallower ring already holds all of them
      const int occ = ring_occupancy(ctx, batched, a_dtype, two, grouped, w, s);
      if (int64_t(occ) * ctx->sm_count >= tiles) { *warps = w; *depth = s; return; }
    }
  }
  // several waves: 4-warp CTAs; the deepest ring whose shared memory still lets
  // ceil(tiles / SMs) CTAs (at most 8) live on one SM
  const int64_t per_sm = std::min<int64_t>(8, (tiles + ctx->sm_count - 1) / ctx->sm_count);
  int d = 2;
  for (int cand : {4, 6, 8})
    if (per_sm * (int64_t(cand) * 4096 + 2048 + 1024) <= 224 * 1024) d = cand;
  // two token tiles (m > 8) double the accumulators: the registers then cap the resident
  // CTAs, and rings deeper than 4 measured 1.5x slower
  if (two) d = std::min(d, 4);
  *warps = 4; *depth = d;
  // many waves and two token tiles: 32-row tiles are ~5 % faster (lm_head at m = 16: 134 against 142 us)
  if (wide && two) *wide = 1;
}

// wide (32-row) ring tiles: depths 2 and 4
template <typename K>
void launch_pdl(K kernel, int grid, int block, size_t smem, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, p, e);
}
inline size_t ring2_smem_bytes(int warps, int depth, bool two) {
  return size_t(depth) * 4 * warps * 32 * 16 + size_t(warps) * 2 * (two ? 2 : 1) * 128 * 4;
}
template <typename AT, int NT, bool GROUPED>
void launch_ring2_s(int depth, int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  const size_t smem = ring2_smem_bytes(block / 32, depth >= 4 ? 4 : 2, NT == 2);
  if (depth >= 4) launch_pdl(qgemv_ring2_kernel<AT, NT, GROUPED, 4>, grid, block, smem, s, p, e);
  else launch_pdl(qgemv_ring2_kernel<AT, NT, GROUPED, 2>, grid, block, smem, s, p, e);
}
template <typename AT>
void launch_ring2(bool two, bool grouped, int depth, int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  if (two) { if (grouped) launch_ring2_s<AT, 2, true>(depth, grid, block, s, p, e); else launch_ring2_s<AT, 2, false>(depth, grid, block, s, p, e); }
  else { if (grouped) launch_ring2_s<AT, 1, true>(depth, grid, block, s, p, e); else launch_ring2_s<AT, 1, false>(depth, grid, block, s, p, e); }
}

template <typename AT, bool M16, bool GROUPED>
void launch_sk_d(int depth, int grid, cudaStream_t s, const GemvArgs& p, const EpiParams& e, const SkArgs& sk) {
  if (depth >= 4) qgemv_sk_kernel<AT, M16, GROUPED, 4><<<grid, 256, 0, s>>>(p, e, sk);
  else qgemv_sk_kernel<AT, M16, GROUPED, 2><<<grid, 256, 0, s>>>(p, e, sk);
}
template <typename AT>
void launch_sk(bool m16, bool grouped, int depth, int grid, cudaStream_t s, const GemvArgs& p, const EpiParams& e,
               const SkArgs& sk) {
  if (m16) {
    if (grouped) launch_sk_d<AT, true, true>(depth, grid, s, p, e, sk);
    else launch_sk_d<AT, true, false>(depth, grid, s, p, e, sk);
  } else {
    if (grouped) launch_sk_d<AT, false, true>(depth, grid, s, p, e, sk);
    else launch_sk_d<AT, false, false>(depth, grid, s, p, e, sk);
  }
}

template <typename AT, int MT, int R>
void launch_simt(bool grouped, int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  if (grouped) qgemv_simt_kernel<AT, MT, R, true><<<grid, block, 0, s>>>(p, e);
  else qgemv_simt_kernel<AT, MT, R, false><<<grid, block, 0, s>>>(p, e);
}
template <typename AT, int R>
void launch_simt_m(int mt, bool grouped, int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  switch (mt) {
    case 1: launch_simt<AT, 1, R>(grouped, grid, block, s, p, e); break;
    case 2: launch_simt<AT, 2, R>(grouped, grid, block, s, p, e); break;
    case 3: launch_simt<AT, 3, R>(grouped, grid, block, s, p, e); break;
    default: launch_simt<AT, 4, R>(grouped, grid, block, s, p, e); break;
  }
}
template <typename AT>
void launch_simt_r(int r, int mt, bool grouped, int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  if (r >= 4) launch_simt_m<AT, 4>(mt, grouped, grid, block, s, p, e);
  else if (r >= 2) launch_simt_m<AT, 2>(mt, grouped, grid, block, s, p, e);
  else launch_simt_m<AT, 1>(mt, grouped, grid, block, s, p, e);
}

template <typename AT, int NT>
void launch_mma(bool grouped, int unroll, int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e) {
  if (grouped) {
    if (unroll >= 4) qgemv_mma_kernel<AT, NT, true, 4><<<grid, block, 0, s>>>(p, e);
    else qgemv_mma_kernel<AT, NT, true, 2><<<grid, block, 0, s>>>(p, e);
  } else {
    if (unroll >= 4) qgemv_mma_kernel<AT, NT, false, 4><<<grid, block, 0, s>>>(p, e);
    else qgemv_mma_kernel<AT, NT, false, 2><<<grid, block, 0, s>>>(p, e);
  }
}

}  // namespace

bool tl_push_matches(tl_ctx* ctx, const void* a, int32_t a_dtype, int32_t m, int64_t k);
int32_t tl_launch_qgemv_rin(tl_ctx* ctx, const void* a, int32_t a_dtype, const GemvArgs* items, const EpiParams* epis, int n_items,
                            int32_t m, int64_t k, bool grouped);

bool tl_qgemv_variant_applicable(const tl_variant& v, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q) {
  (void)n;
  if (v.family != TL_FAMILY_QGEMV || m < 1 || m > 16) return false;
  if (v.p0 < 1 || v.p0 > kMmaMaxWarps) return false;
  switch (v.kernel) {
    case kStream: return tl_qgemv_stream_applicable(v, m, k, a_dtype, q);
    case kScalar: return v.p0 <= 8;
    case kSimt: return v.p0 <= 8 && k % 16 == 0 && q.group_size % 16 == 0 && (v.p1 == 1 || v.p1 == 2 || v.p1 == 4);
    case kMma:
      return (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 64 == 0 && q.group_size % 64 == 0 &&
             (v.p1 == 2 || v.p1 == 4);
    case kBulk:
      return (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 128 == 0 && q.group_size % 64 == 0 &&
             (v.p0 == 8 || v.p0 == 16) && (v.p1 == 32 || v.p1 == 64) && bulk_geom(k, v.p0, v.p1).ok;
    case kTma:
      return (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 128 == 0 && q.group_size % 64 == 0 &&
             (v.p0 == 4 || v.p0 == 5 || v.p0 == 6);
    case kRing:
      return (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 64 == 0 && q.group_size % 64 == 0 &&
             (v.p1 == 2 || v.p1 == 4 || v.p1 == 6 || v.p1 == 8) &&
             (v.p2 == 0 || v.p2 == 1 || (v.p2 == 2 && v.p1 <= 4));  // p2 = 2: 32-row tiles
    case kSk:
      // a thread's 32 contiguous weight bytes feed all of a unit's MMAs, so one MMA spans the whole
      // 128-wide unit: a scale group must cover it
      return (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 128 == 0 && q.group_size % 128 == 0 && v.p0 <= 8 &&
             (v.p1 == 2 || v.p1 == 4);
    default: return false;
  }
}

int32_t tl_qgemv_default_variant(tl_ctx* ctx, int32_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q, tl_variant* out) {
  tl_variant v{};
  v.family = TL_FAMILY_QGEMV;
  if ((a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 64 == 0 && q.group_size % 64 == 0) {
    const int64_t tiles = (n + 15) / 16;
    v.kernel = kRing;
    int w = 4, d = 2, wide = 0;
    ring_pick_shape(ctx, false, a_dtype, m, q.group_size != k, tiles, k, &w, &d, &wide);
    v.p0 = w; v.p1 = d; v.p2 = wide ? 2 : 0;
  } else if (k % 16 == 0 && q.group_size % 16 == 0) {
    v.kernel = kSimt; v.p0 = 8; v.p1 = 2;
  } else {
    v.kernel = kScalar; v.p0 = 8;
  }
  *out = v;
  return TL_OK;
}

int32_t tl_qgemv_candidates(tl_ctx* ctx, int32_t m, int64_t n, int64_t k, int32_t a_dtype,
                            const tl_quant_desc& q, std::vector<tl_variant>* out) {
  tl_variant d;
  tl_qgemv_default_variant(ctx, m, n, k, a_dtype, q, &d);
  out->clear();
  out->push_back(d);  // the default is always a candidate (variants.ts:194-205)
  auto add = [&](int kernel, int p0, int p1) {
    tl_variant v{};
    v.family = TL_FAMILY_QGEMV; v.kernel = kernel; v.p0 = p0; v.p1 = p1; v.p2 = kernel == kMma ? 1 : 0;
    if (!tl_qgemv_variant_applicable(v, m, n, k, a_dtype, q)) return;
    for (const auto& o : *out)
      if (o.kernel == v.kernel && o.p0 == v.p0 && o.p1 == v.p1 && o.p2 == v.p2) return;
    out->push_back(v);
  };
  for (int st : {3, 5}) {
    tl_variant v{};
    v.family = TL_FAMILY_QGEMV; v.kernel = kStream; v.p0 = 8; v.p1 = st; v.p2 = 2; v.p3 = st == 3 ? 32 : 16;
    if (m > 8 && st == 3) continue;  // two token tiles double the fragment buffers: 16-block stages only
    if (tl_qgemv_variant_applicable(v, m, n, k, a_dtype, q)) out->push_back(v);
  }
  for (int w : {8, 16})
    for (int kb : {32, 64}) add(kBulk, w, kb);
  for (int st : {4, 6}) add(kTma, st, 0);
  for (int w : {2, 4, 8, 16})
    for (int u : {2, 4, 6, 8}) add(kRing, w, u);
  for (int w : {4, 8, 16})
    for (int u : {2, 4}) {  // 32-row tiles
      tl_variant v{};
      v.family = TL_FAMILY_QGEMV; v.kernel = kRing; v.p0 = w; v.p1 = u; v.p2 = 2;
      bool dup = false;
      for (const auto& o : *out) dup = dup || (o.kernel == v.kernel && o.p0 == v.p0 && o.p1 == v.p1 && o.p2 == v.p2);
      if (!dup && tl_qgemv_variant_applicable(v, m, n, k, a_dtype, q)) out->push_back(v);
    }
  for (int b : {2, 4, 8})
    for (int u : {2, 4}) add(kSk, b, u);
  for (int w : {4, 8, 16})
    for (int u : {2, 4}) add(kMma, w, u);
  if (m <= 4 || a_dtype == TL_F32)
    for (int w : {4, 8})
      for (int r : {1, 2, 4}) add(kSimt, w, r);
  return TL_OK;
}

int32_t tl_launch_qgemv(tl_ctx* ctx, const tl_variant& v, const void* a, int32_t a_dtype, const void* packed,
                        const void* scales, void* out, int32_t out_dtype, int32_t m, int64_t n, int64_t k,
                        const tl_quant_desc& q, const EpiParams& epi, tl_plan_receipt* receipt) {
  if (!tl_qgemv_variant_applicable(v, m, n, k, a_dtype, q))
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "qgemv: variant %s cannot run m=%d n=%lld k=%lld G=%d %s",
                        tl_variant_name(&v), m, (long long)n, (long long)k, q.group_size, tl_dtype_name(a_dtype));
  if (!receipt && ctx->push_pending) {
    // a tl_qgemv_nt_push is waiting for its sum: this launch must be the one that reads it
    if (!tl_push_matches(ctx, a, a_dtype, m, k) || k % 64 != 0 || q.group_size % 64 != 0 ||
        (reinterpret_cast<uintptr_t>(packed) & 15))
      return tl_set_error(ctx, TL_ERR_INVALID_ARG,
                          "qgemv: a pushed partial sum is pending; the next small-batch launch must read it as its activations "
                          "([m, k] = [%d, %lld]), or call tl_reduce_pending first", ctx->push_m, (long long)ctx->push_n);
    GemvArgs pr{};
    pr.a = a; pr.packed = reinterpret_cast<const uint32_t*>(packed); pr.scales = scales; pr.out = out;
    pr.m = m; pr.n = int32_t(n); pr.k = int32_t(k);
    pr.group = q.group_size; pr.groups_per_row = int32_t(k / q.group_size);
    pr.scales_dtype = q.scales_dtype; pr.out_dtype = out_dtype;
    pr.wscale = q.scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
    pr.row0 = 0; pr.m_total = m;
    return tl_launch_qgemv_rin(ctx, a, a_dtype, &pr, &epi, 1, m, k, q.group_size != k);
  }
  if (v.kernel == kStream) {
    const void* pk[1] = {packed};
    const void* sc[1] = {scales};
    void* ot[1] = {out};
    const int64_t nn[1] = {n};
    return tl_launch_qgemv_stream(ctx, v, a, a_dtype, 1, pk, sc, ot, nn, &epi, out_dtype, m, k, q, receipt);
  }
  GemvArgs p{};
  p.a = a; p.packed = reinterpret_cast<const uint32_t*>(packed); p.scales = scales; p.out = out;
  p.m = m; p.n = int32_t(n); p.k = int32_t(k);
  p.group = q.group_size; p.groups_per_row = int32_t(k / q.group_size);
  p.scales_dtype = q.scales_dtype; p.out_dtype = out_dtype;
  p.wscale = q.scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
  p.row0 = 0; p.m_total = m;
  const bool grouped = q.group_size != k;
  int block = v.p0 * 32;
  int grid = 0, launches = 1;
  SkArgs sk{};
  TmaArgs ta{};
  BulkArgs ba{};
  BulkGeom bg{};
  if (v.kernel == kBulk) {
    bg = bulk_geom(k, v.p0, v.p1);
    block = (v.p0 + 1) * 32;
    ba.rt = bg.rt; ba.kb128 = int32_t(k / 128); ba.p = bg.p; ba.stage_bytes = bg.stage_bytes;
    ba.total_stages = int32_t((n + int64_t(8) * bg.rt - 1) / (int64_t(8) * bg.rt));
    grid = int(std::min<int64_t>(ctx->sm_count, ba.total_stages));
  } else if (v.kernel == kTma) {
    block = (kTmaConsumerWarps + 1) * 32;
    ta.spb = int32_t(k / kTmaBoxBytes);
    const int64_t bands = (n + kTmaBoxRows - 1) / kTmaBoxRows;
    ta.total_stages = int32_t(bands * ta.spb);
    grid = int(std::min<int64_t>(ctx->sm_count, ta.total_stages));
  } else if (v.kernel == kSk) {
    block = 256;
    const int64_t tiles = (n + 7) / 8;
    sk.upt = int32_t(k / 128);
    sk.total_units = tiles * sk.upt;
    const int64_t resident = int64_t(ctx->sm_count) * v.p0 * 8;          // warps the persistent grid can hold
    const int64_t useful = std::max<int64_t>(1, sk.total_units / 4);     // at least 4 units (4 KB) per warp
    sk.warps_used = int32_t(std::min(resident, useful));
    grid = (sk.warps_used + 7) / 8;
  } else if (v.kernel == kScalar) grid = int((n + v.p0 - 1) / v.p0);
  else if (v.kernel == kSimt) { grid = int((n + int64_t(v.p0) * v.p1 - 1) / (int64_t(v.p0) * v.p1)); launches = (m + 3) / 4; }
  else if (v.kernel == kRing && v.p2 == 2) grid = int((n + 31) / 32);
  else grid = int((n + 15) / 16);
  if (receipt) {
    receipt->choice = v;
    receipt->grid[0] = grid; receipt->grid[1] = 1; receipt->grid[2] = launches;
    receipt->block = block; receipt->split_k = 1;
    return TL_OK;
  }
  if (v.kernel != kScalar) {
    // 16-byte vector loads need 16-byte aligned bases (rows are K bytes apart, K % 16 == 0)
    if ((reinterpret_cast<uintptr_t>(packed) & 15) || (reinterpret_cast<uintptr_t>(a) & 15))
      return tl_set_error(ctx, TL_ERR_INVALID_ARG, "qgemv: %s needs 16-byte aligned weight and activation pointers",
                          tl_variant_name(&v));
  }
  cudaStream_t s = ctx->stream;
  if (v.kernel == kBulk) {
    ba.status = ctx->dev_status;
    const bool m16 = m > 8;
#define TL_BULK_LAUNCH(AT_, M16_, G_)                                                                  \
  do {                                                                                                \
    auto kern = qgemv_bulk_kernel<AT_, M16_, G_>;                                                     \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bg.smem));            \
    kern<<<grid, block, bg.smem, s>>>(p, epi, ba, bg.nstages, v.p0);                                  \
  } while (0)
#define TL_BULK_AT(AT_)                                                                                \
  do {                                                                                                \
    if (m16) { if (grouped) TL_BULK_LAUNCH(AT_, true, true); else TL_BULK_LAUNCH(AT_, true, false); } \
    else { if (grouped) TL_BULK_LAUNCH(AT_, false, true); else TL_BULK_LAUNCH(AT_, false, false); }   \
  } while (0)
    if (a_dtype == TL_F16) TL_BULK_AT(__half);
    else TL_BULK_AT(__nv_bfloat16);
#undef TL_BULK_AT
#undef TL_BULK_LAUNCH
  } else if (v.kernel == kTma) {
    const int64_t bands = (n + kTmaBoxRows - 1) / kTmaBoxRows;
    const size_t sbytes = size_t(m) * n * sizeof(float);
    void* base = nullptr;
    int32_t rc = tl_ensure_zeroed_scratch(ctx, sbytes + size_t(bands) * kTmaConsumerWarps * sizeof(unsigned), &base);
    if (rc != TL_OK) return rc;
    ta.scratch = reinterpret_cast<float*>(base);
    ta.counters = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(base) + sbytes);
    ta.status = ctx->dev_status;
    CUtensorMap wmap;
    if (!tl_encode_tmap_2d(&wmap, 1, packed, uint64_t(k), uint64_t(n), uint64_t(k), kTmaBoxBytes, kTmaBoxRows, 3))
      return tl_set_error(ctx, TL_ERR_CUDA, "qgemv: cuTensorMapEncodeTiled failed for the %lldx%lld weight",
                          (long long)n, (long long)k);
    const bool two = m > 8;
    const int st = v.p0;
    const size_t smem = size_t(st) * kTmaStageBytes + 1024;
#define TL_TMA_LAUNCH(AT_, NT_, G_, ST_)                                                                   \
  do {                                                                                                    \
    auto kern = qgemv_tma_kernel<AT_, NT_, G_, ST_>;                                                      \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));                   \
    kern<<<grid, block, smem, s>>>(wmap, p, epi, ta);                                                     \
  } while (0)
#define TL_TMA_ST(AT_, NT_, G_)                                          \
  do {                                                                  \
    if (st == 4) TL_TMA_LAUNCH(AT_, NT_, G_, 4);                        \
    else if (st == 5) TL_TMA_LAUNCH(AT_, NT_, G_, 5);                   \
    else TL_TMA_LAUNCH(AT_, NT_, G_, 6);                                \
  } while (0)
#define TL_TMA_AT(AT_)                                                   \
  do {                                                                  \
    if (two) { if (grouped) TL_TMA_ST(AT_, 2, true); else TL_TMA_ST(AT_, 2, false); }  \
    else { if (grouped) TL_TMA_ST(AT_, 1, true); else TL_TMA_ST(AT_, 1, false); }      \
  } while (0)
    if (a_dtype == TL_F16) TL_TMA_AT(__half);
    else TL_TMA_AT(__nv_bfloat16);
#undef TL_TMA_AT
#undef TL_TMA_ST
#undef TL_TMA_LAUNCH
  } else if (v.kernel == kSk) {
    const int64_t tiles = (n + 7) / 8;
    const size_t sbytes = size_t(m) * n * sizeof(float);
    void* base = nullptr;
    int32_t rc = tl_ensure_zeroed_scratch(ctx, sbytes + size_t(tiles) * sizeof(unsigned), &base);
    if (rc != TL_OK) return rc;
    sk.scratch = reinterpret_cast<float*>(base);
    sk.counters = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(base) + sbytes);
    if (a_dtype == TL_F16) launch_sk<__half>(m > 8, grouped, v.p1, grid, s, p, epi, sk);
    else launch_sk<__nv_bfloat16>(m > 8, grouped, v.p1, grid, s, p, epi, sk);
  } else if (v.kernel == kScalar) {
    if (a_dtype == TL_F32) qgemv_scalar_kernel<float><<<grid, block, 0, s>>>(p, epi);
    else if (a_dtype == TL_F16) qgemv_scalar_kernel<__half><<<grid, block, 0, s>>>(p, epi);
    else qgemv_scalar_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(p, epi);
  } else if (v.kernel == kSimt) {
    // batch rows go through in slices of four; each slice re-streams the weight
    for (int m0 = 0; m0 < m; m0 += 4) {
      GemvArgs ps = p;
      const int mt = std::min(4, m - m0);
      ps.m = mt; ps.row0 = m0;
      ps.a = reinterpret_cast<const uint8_t*>(a) + size_t(m0) * k * tl_dtype_size(a_dtype);
      if (a_dtype == TL_F32) launch_simt_r<float>(v.p1, mt, grouped, grid, block, s, ps, epi);
      else if (a_dtype == TL_F16) launch_simt_r<__half>(v.p1, mt, grouped, grid, block, s, ps, epi);
      else launch_simt_r<__nv_bfloat16>(v.p1, mt, grouped, grid, block, s, ps, epi);
    }
  } else if (v.kernel == kRing && v.p2 == 2) {
    if (a_dtype == TL_F16) launch_ring2<__half>(m > 8, grouped, v.p1, grid, block, s, p, epi);
    else launch_ring2<__nv_bfloat16>(m > 8, grouped, v.p1, grid, block, s, p, epi);
  } else if (v.kernel == kRing) {
    if (a_dtype == TL_F16) launch_ring<__half>(m > 8, grouped, v.p1, grid, block, s, p, epi);
    else launch_ring<__nv_bfloat16>(m > 8, grouped, v.p1, grid, block, s, p, epi);
  } else {
    const bool two = m > 8;
    if (a_dtype == TL_F16) {
      if (two) launch_mma<__half, 2>(grouped, v.p1, grid, block, s, p, epi);
      else launch_mma<__half, 1>(grouped, v.p1, grid, block, s, p, epi);
    } else {
      if (two) launch_mma<__nv_bfloat16, 2>(grouped, v.p1, grid, block, s, p, epi);
      else launch_mma<__nv_bfloat16, 1>(grouped, v.p1, grid, block, s, p, epi);
    }
  }
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES] += launches;
  return TL_OK;
}

// ---------------------------------------------------------------------------
// tl_qgemv_nt_static_scratch: the small-batch quantized matmul for callers that
// must not allocate.
//
// tl_qgemv_nt may grow the context's partial-sum scratch with cudaMalloc the first
// time a shape needs it.  That is unacceptable for a host that calls from a place
// where device allocation is off limits: a serving process that has handed all
// device memory to its own pool (a cudaMalloc from a library can only fail there),
// or a latency-critical loop where the device-wide synchronisation hidden in
// cudaMalloc/cudaFree would stall every other stream.  This entry point runs the
// TMA-fed persistent kernel (variant "tma") with its partial-sum meeting point in a
// fixed array that is part of the loaded module, so the call itself performs no
// cudaMalloc, cudaFree or other allocating routine.
//
// The price is a fixed ceiling and a shared buffer:
//   - m*n*4 + ceil(n/256)*64 bytes must fit in TL_STATIC_SCRATCH_BYTES (4 MiB); larger
//     problems are rejected with TL_ERR_UNSUPPORTED before anything is launched;
//   - every GPU that loads the library carries the 4 MiB until the process exits;
//   - all calls on a device use the same array.  The part a call uses is cleared on
//     the stream before the kernel runs (it keeps whatever the previous call left,
//     including after an aborted kernel), so calls that are ordered on one stream are
//     safe, but two calls that overlap on the GPU (different streams or contexts on
//     the same device) race on it and must be serialised by the caller.
// The array's device address is looked up with cudaGetSymbolAddress the first time
// the entry point is called on a device (the name of a __device__ array is only a
// host-side handle, never a pointer a kernel may be given).  That first call on a
// device therefore does a little set-up work and should come before any stream capture.
// ---------------------------------------------------------------------------
#define TL_STATIC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char tl_static_scratch[TL_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kStaticMaxDevices = 64;
void* g_static_scratch_ptr[kStaticMaxDevices] = {nullptr};

template <typename AT>
void launch_tma_static(bool two, bool grouped, int grid, int block, size_t smem, cudaStream_t s, const CUtensorMap& wmap,
                       const GemvArgs& p, const EpiParams& epi, const TmaArgs& ta) {
#define TL_STATIC_LAUNCH(NT_, G_)                                                                    \
  do {                                                                                              \
    auto kern = qgemv_tma_kernel<AT, NT_, G_, 6>;                                                   \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));             \
    kern<<<grid, block, smem, s>>>(wmap, p, epi, ta);                                               \
  } while (0)
  if (two) { if (grouped) TL_STATIC_LAUNCH(2, true); else TL_STATIC_LAUNCH(2, false); }
  else { if (grouped) TL_STATIC_LAUNCH(1, true); else TL_STATIC_LAUNCH(1, false); }
#undef TL_STATIC_LAUNCH
}
}  // namespace

extern "C" int32_t tl_qgemv_nt_static_scratch(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed,
                                              const void* scales, void* out, int32_t out_dtype, int32_t m, int64_t n,
                                              int64_t k, const tl_quant_desc* qdesc, float alpha,
                                              const tl_epilogue* epilogue) {
  TL_CHECK_CTX(ctx);
  int32_t rc = tl_check_qargs(ctx, "tl_qgemv_nt_static_scratch", a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc);
  if (rc != TL_OK) return rc;
  if (m < 1 || m > 16)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_static_scratch: m=%d outside the GEMV range [1,16]", m);
  if (n == 0) return TL_OK;
  if ((a_dtype != TL_F16 && a_dtype != TL_BF16) || k % 128 != 0 || qdesc->group_size % 64 != 0)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED,
                        "tl_qgemv_nt_static_scratch: needs f16/bf16 activations, K %% 128 == 0 and groupSize %% 64 == 0 "
                        "(got %s, K=%lld, G=%d)", tl_dtype_name(a_dtype), (long long)k, qdesc->group_size);
  if ((reinterpret_cast<uintptr_t>(packed) & 15) || (reinterpret_cast<uintptr_t>(a) & 15))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_static_scratch: weight and activation pointers must be 16-byte aligned");
  const int64_t bands = (n + kTmaBoxRows - 1) / kTmaBoxRows;
  const size_t sbytes = size_t(m) * size_t(n) * sizeof(float);
  const size_t need = sbytes + size_t(bands) * kTmaConsumerWarps * sizeof(unsigned);
  if (need > TL_STATIC_SCRATCH_BYTES)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED,
                        "tl_qgemv_nt_static_scratch: m=%d n=%lld needs %zu bytes of scratch, the built-in array holds %u; "
                        "use tl_qgemv_nt", m, (long long)n, need, unsigned(TL_STATIC_SCRATCH_BYTES));
  EpiParams epi;
  bool has_ops = false;
  rc = tl_make_epi(ctx, epilogue, alpha, &epi, &has_ops);
  if (rc != TL_OK) return rc;
  if (ctx->device < 0 || ctx->device >= kStaticMaxDevices)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_nt_static_scratch: device ordinal %d not supported", ctx->device);
  DeviceGuard guard(ctx->device);
  if (!g_static_scratch_ptr[ctx->device]) {
    // once per device, with that device current: the symbol's address on THIS device
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, tl_static_scratch);
    if (e != cudaSuccess || !ptr) {
      cudaGetLastError();
      return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_nt_static_scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    }
    g_static_scratch_ptr[ctx->device] = ptr;
  }
  uint8_t* base = reinterpret_cast<uint8_t*>(g_static_scratch_ptr[ctx->device]);
  // the array keeps the previous call's contents: zero the part this call accumulates into
  TL_CUDA(ctx, cudaMemsetAsync(base, 0, need, ctx->stream));

  GemvArgs p{};
  p.a = a; p.packed = reinterpret_cast<const uint32_t*>(packed); p.scales = scales; p.out = out;
  p.m = m; p.n = int32_t(n); p.k = int32_t(k);
  p.group = qdesc->group_size; p.groups_per_row = int32_t(k / qdesc->group_size);
  p.scales_dtype = qdesc->scales_dtype; p.out_dtype = out_dtype;
  p.wscale = qdesc->scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
  p.row0 = 0; p.m_total = m;
  TmaArgs ta{};
  ta.scratch = reinterpret_cast<float*>(base);
  ta.counters = reinterpret_cast<unsigned*>(base + sbytes);
  ta.status = ctx->dev_status;
  ta.spb = int32_t(k / kTmaBoxBytes);
  ta.total_stages = int32_t(bands * ta.spb);
  const int grid = int(std::min<int64_t>(ctx->sm_count, ta.total_stages));
  const int block = (kTmaConsumerWarps + 1) * 32;
  const size_t smem = size_t(6) * kTmaStageBytes + 1024;
  CUtensorMap wmap;
  if (!tl_encode_tmap_2d(&wmap, 1, packed, uint64_t(k), uint64_t(n), uint64_t(k), kTmaBoxBytes, kTmaBoxRows, 3))
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_nt_static_scratch: cuTensorMapEncodeTiled failed");
  const bool grouped = qdesc->group_size != k;
  if (a_dtype == TL_F16) launch_tma_static<__half>(m > 8, grouped, grid, block, smem, ctx->stream, wmap, p, epi, ta);
  else launch_tma_static<__nv_bfloat16>(m > 8, grouped, grid, block, smem, ctx->stream, wmap, p, epi, ta);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  ctx->counters[TL_COUNTER_QGEMV]++;
  if (has_ops) ctx->counters[TL_COUNTER_QGEMV_EPILOGUE]++;
  return TL_OK;
}


// ---------------------------------------------------------------------------
// tl_qgemv_nt_batched: several small-batch projections over the same activations in one launch.
// ---------------------------------------------------------------------------
namespace {
template <typename AT, int NT, bool GROUPED, int S>
void launch_ring_batched(int grid, int block, cudaStream_t s, const RingBatchArgs& b) {
  const size_t smem = size_t(S) * 2 * block * 16 + size_t(block / 32) * NT * 128 * 4;
  auto kern = qgemv_ring_batched_kernel<AT, NT, GROUPED, S>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, b);
}
template <typename AT, int NT, bool GROUPED, int S>
void launch_ring2_batched(int grid, int block, cudaStream_t s, const RingBatchArgs& b) {
  const size_t smem = ring2_smem_bytes(block / 32, S, NT == 2);
  auto kern = qgemv_ring2_batched_kernel<AT, NT, GROUPED, S>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, b);
}
template <typename AT>
void launch_ring2_batched_at(bool two, bool grouped, int depth, int grid, int block, cudaStream_t s, const RingBatchArgs& b) {
#define TL_R2B(NT_, G_) { if (depth >= 4) launch_ring2_batched<AT, NT_, G_, 4>(grid, block, s, b); else launch_ring2_batched<AT, NT_, G_, 2>(grid, block, s, b); }
  if (two) { if (grouped) TL_R2B(2, true) else TL_R2B(2, false) }
  else { if (grouped) TL_R2B(1, true) else TL_R2B(1, false) }
#undef TL_R2B
}
template <typename AT, int NT, bool GROUPED>
void launch_ring_batched_s(int depth, int grid, int block, cudaStream_t s, const RingBatchArgs& b) {
  if (depth >= 8) launch_ring_batched<AT, NT, GROUPED, 8>(grid, block, s, b);
  else if (depth >= 6) launch_ring_batched<AT, NT, GROUPED, 6>(grid, block, s, b);
  else if (depth >= 4) launch_ring_batched<AT, NT, GROUPED, 4>(grid, block, s, b);
  else launch_ring_batched<AT, NT, GROUPED, 2>(grid, block, s, b);
}
template <typename AT>
void launch_ring_batched_at(bool two, bool grouped, int depth, int grid, int block, cudaStream_t s, const RingBatchArgs& b) {
  if (two) { if (grouped) launch_ring_batched_s<AT, 2, true>(depth, grid, block, s, b); else launch_ring_batched_s<AT, 2, false>(depth, grid, block, s, b); }
  else { if (grouped) launch_ring_batched_s<AT, 1, true>(depth, grid, block, s, b); else launch_ring_batched_s<AT, 1, false>(depth, grid, block, s, b); }
}
}  // namespace

extern "C" int32_t tl_qgemv_nt_batched(tl_ctx* ctx, const void* a, int32_t a_dtype, const tl_qgemv_item* items,
                                       int32_t n_items, int32_t out_dtype, int32_t m, int64_t k,
                                       const tl_quant_desc* qdesc) {
  TL_CHECK_CTX(ctx);
  if (!items || n_items < 1 || n_items > kMaxBatchItems)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_batched: 1..%d items (got %d)", kMaxBatchItems, n_items);
  if (m < 1 || m > 16) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_batched: m=%d outside the GEMV range [1,16]", m);
  bool fused_ok = qdesc && (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 64 == 0 && qdesc->group_size > 0 &&
                  qdesc->group_size % 64 == 0 && !(reinterpret_cast<uintptr_t>(a) & 15);
  for (int i = 0; i < n_items; ++i) {
    int32_t rc = tl_check_qargs(ctx, "tl_qgemv_nt_batched", a, a_dtype, items[i].packed, items[i].scales, items[i].out,
                                out_dtype, m, items[i].n, k, qdesc);
    if (rc != TL_OK) return rc;
    if (items[i].n == 0 || (reinterpret_cast<uintptr_t>(items[i].packed) & 15)) fused_ok = false;
  }
  if (!fused_ok) {
    // shapes the fused kernel does not take: one ordinary call per item, same results
    for (int i = 0; i < n_items; ++i) {
      int32_t rc = tl_qgemv_nt(ctx, a, a_dtype, items[i].packed, items[i].scales, items[i].out, out_dtype, m, items[i].n, k,
                               qdesc, items[i].alpha, items[i].epilogue);
      if (rc != TL_OK) return rc;
    }
    return TL_OK;
  }
  RingBatchArgs b{};
  int64_t tiles = 0;
  int n_epi = 0;
  for (int i = 0; i < kMaxBatchItems; ++i) {
    b.tile_start[i] = int32_t(tiles);
    if (i >= n_items) continue;
    bool has_ops = false;
    int32_t rc = tl_make_epi(ctx, items[i].epilogue, items[i].alpha, &b.e[i], &has_ops);
    if (rc != TL_OK) return rc;
    n_epi += has_ops ? 1 : 0;
    GemvArgs& p = b.p[i];
    p.a = a; p.packed = reinterpret_cast<const uint32_t*>(items[i].packed); p.scales = items[i].scales; p.out = items[i].out;
    p.m = m; p.n = int32_t(items[i].n); p.k = int32_t(k);
    p.group = qdesc->group_size; p.groups_per_row = int32_t(k / qdesc->group_size);
    p.scales_dtype = qdesc->scales_dtype; p.out_dtype = out_dtype;
    p.wscale = qdesc->scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
    p.row0 = 0; p.m_total = m;
    tiles += (items[i].n + 15) / 16;
  }
  b.tile_start[kMaxBatchItems] = int32_t(tiles);
  if (ctx->push_pending) {
    if (!tl_push_matches(ctx, a, a_dtype, m, k))
      return tl_set_error(ctx, TL_ERR_INVALID_ARG,
                          "tl_qgemv_nt_batched: a pushed partial sum is pending; this launch must read it as its activations "
                          "([m, k] = [%d, %lld]), or call tl_reduce_pending first", ctx->push_m, (long long)ctx->push_n);
    DeviceGuard guard(ctx->device);
    int32_t rc = tl_launch_qgemv_rin(ctx, a, a_dtype, b.p, b.e, n_items, m, k, qdesc->group_size != k);
    if (rc != TL_OK) return rc;
    ctx->counters[TL_COUNTER_QGEMV] += n_items;
    ctx->counters[TL_COUNTER_QGEMV_EPILOGUE] += n_epi;
    return TL_OK;
  }
  for (int i = n_items; i < kMaxBatchItems; ++i) b.tile_start[i] = int32_t(tiles);  // unused items are empty ranges
  // the single-matrix shape rule (one wave if possible); a forced or tuned ring variant (keyed on
  // the summed N) overrides it
  int64_t n_total = 0;
  for (int i = 0; i < n_items; ++i) n_total += items[i].n;
  DeviceGuard guard(ctx->device);
  int warps = 4, depth = 2, wide = 0;
  ring_pick_shape(ctx, true, a_dtype, m, qdesc->group_size != k, tiles, k, &warps, &depth, &wide);
  tl_variant tv{};
  if (ctx->has_forced && ctx->forced.family == TL_FAMILY_QGEMV && ctx->forced.kernel == kRing) {
    warps = ctx->forced.p0; depth = ctx->forced.p1; wide = ctx->forced.p2 == 2;
  } else if (tl_lookup_tuned(ctx, m, n_total, k, a_dtype, *qdesc, &tv) && tv.family == TL_FAMILY_QGEMV && tv.kernel == kRing) {
    warps = tv.p0; depth = tv.p1; wide = tv.p2 == 2;
  }
  if (warps != 2 && warps != 4 && warps != 8 && warps != 16)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_nt_batched: ring variant with %d warps", warps);
  if (wide) {  // 32-row tiles: the items' tile ranges are counted in those
    tiles = 0;
    for (int i = 0; i < kMaxBatchItems; ++i) {
      b.tile_start[i] = int32_t(tiles);
      if (i < n_items) tiles += (items[i].n + 31) / 32;
    }
    b.tile_start[kMaxBatchItems] = int32_t(tiles);
    depth = depth >= 4 ? 4 : 2;
  }
  const int block = warps * 32, grid = int(tiles);
  const bool grouped = qdesc->group_size != k;
  if (wide) {
    if (a_dtype == TL_F16) launch_ring2_batched_at<__half>(m > 8, grouped, depth, grid, block, ctx->stream, b);
    else launch_ring2_batched_at<__nv_bfloat16>(m > 8, grouped, depth, grid, block, ctx->stream, b);
  } else if (a_dtype == TL_F16) launch_ring_batched_at<__half>(m > 8, grouped, depth, grid, block, ctx->stream, b);
  else launch_ring_batched_at<__nv_bfloat16>(m > 8, grouped, depth, grid, block, ctx->stream, b);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  ctx->counters[TL_COUNTER_QGEMV] += n_items;
  ctx->counters[TL_COUNTER_QGEMV_EPILOGUE] += n_epi;
  return TL_OK;
}

// ---------------------------------------------------------------------------
// Persistent chain ("vertical fusion"): a whole sequence of dependent small-batch
// products -- the decode step of a layer stack -- in ONE cooperative launch.
//
// Launch boundaries are what a stream of single GEMVs loses most of its time to: every
// kernel ramps its loads up from nothing and drains them at the end (about 4 us per launch
// against 2.7-16 us of streaming for the decode projections).  Here the weight stream never
// stops.  Every CTA owns a flat sequence of 16-row tiles that runs through ALL phases
// (phase = up to four projections that read the same activations), and every thread keeps
// S 16-byte cp.async copies per row in flight along that sequence -- the prefetch cursor
// simply walks on into the next tile, and the next phase, because weight addresses never
// depend on results.  Only the consumer side is phase-ordered: before a CTA reads the
// activations of phase p it waits until all CTAs with tiles in phase p-1 have stored theirs
// (one arrival counter per phase in global memory, release/acquire at GPU scope).  While it
// waits, its prefetched next-phase weights keep landing, so HBM stays busy across the barrier.
//
// The sequence of a CTA is a table the host writes once (ChainTile records, in execution
// order, everything a tile needs in 80 bytes): walking it is one broadcast load per tile,
// issued a tile ahead, never a chain of dependent descriptor loads.  (A first version walked
// phase descriptors on the device; their cold-miss latency, 3-6 us per tile, sat inside the
// k loop and made the chain slower than separate launches.)
//
// The tile arithmetic (fragment mapping, W warps interleaved over 64-wide k blocks, summation
// order) is the ring kernel's, so a chain gives the same bits as ring launches with W warps.
// Shape: W = 8 warps per tile and S = 12 k blocks in flight per thread, two CTAs per SM, so
// that a CTA's ring (W*S KB = 96 KB) holds more than one 16 x 4096 tile.
//
// Standing: correct (bit-identical to ring launches) but NOT yet faster than a replayed graph
// of ring launches on the Qwen3-8B stack (2.3-2.6 ms against 1.8-2.0 ms per step).  Device
// traces show why: the weight wait is zero (the prefetch does run ahead), but one k-block
// iteration of a warp takes 0.3 us at batch 1 and 0.6 us at batch 8 -- with one or two tiles
// per CTA and phase every activation line is touched about once per SM, so the activation
// loads miss L1 and cost an L2 round trip per iteration that a short register queue cannot
// hide, and 16-24 warps per SM are too few to cover it; phases whose tile count is not a
// multiple of the grid add a 5-6 us wait at the next gate.  It is kept as an explicit entry
// point and is not what tl_qgemv_nt or the benchmark's default path run.
// Tiles of a phase are dealt round-robin starting at a rotating CTA, which balances the
// cumulative load.  All CTAs are co-resident (cooperative launch).  Every spin is bounded; a
// wait that runs out raises the status word and a global abort word that ends everybody's.
// ---------------------------------------------------------------------------
namespace {

constexpr int kChainMaxItems = 4;
constexpr unsigned kChainSpinLimit = 1u << 20;

struct alignas(16) ChainTile {
  const uint8_t* w;      // first weight row of the tile
  const void* a;         // activations [m, k] of the phase
  const void* scales;    // the item's scales
  void* out;             // the item's output [m, n]
  const EpiParams* epi;  // the item's epilogue
  uint64_t pad_;
  int32_t k, n, tile_row, phase;             // k == 0 ends the list
  int32_t group, out_dtype, wait_for, arrive;  // wait_for: arrivals of phase-1 to see first (0: none);
                                               // arrive: this is the CTA's last tile of its phase
};
static_assert(sizeof(ChainTile) == 80, "record layout");

struct ChainArgs {
  const ChainTile* sched;  // [grid][stride]
  unsigned* bar;           // [n_phases] arrival counters, then one abort word; all zero at launch
  int* status;
  int32_t stride, n_phases, m, scales_dtype;
  float wscale;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_act128(const void* p) {
  // Activations are written by other CTAs of this same launch, so never the non-coherent path
  // (ld.global.nc / __ldg).  An ordinary cached load is correct here: it is ordered after the
  // acquire on the phase counter (thread 0) and the CTA barrier that follows it, exactly the
  // pattern of a grid-wide barrier, and L1 reuse across the CTAs of an SM is what keeps the
  // activation traffic off L2.
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// The part of a record the prefetch cursor needs.
struct ChainFetchRec {
  const uint8_t* w;
  int32_t k, n, tile_row;
};
// Schedule records are read with volatile asm loads: an ordinary load may be sunk by the compiler
// to its first use, a whole tile later, which puts the miss latency back on the critical path.
__device__ __forceinline__ int4 ld_sched128(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint64_t ptr_of(int lo, int hi) { return (uint64_t(uint32_t(hi)) << 32) | uint32_t(lo); }
__device__ __forceinline__ ChainFetchRec chain_load_fetch(const ChainTile* t) {
  ChainFetchRec r;
  const int4 p0 = ld_sched128(&t->w);  // w, a
  const int4 v = ld_sched128(&t->k);
  r.w = reinterpret_cast<const uint8_t*>(ptr_of(p0.x, p0.y));
  r.k = v.x; r.n = v.y; r.tile_row = v.z;
  return r;
}


// A whole record, for the consumer side (five 16-byte broadcast loads).
struct ChainRec {
  const void* a;
  const void* scales;
  void* out;
  const EpiParams* epi;
  int32_t k, n, tile_row, phase, group, out_dtype, wait_for, arrive;
};
__device__ __forceinline__ ChainRec chain_load_rec(const ChainTile* t) {
  const int4 p0 = ld_sched128(&t->w);       // w, a
  const int4 p1 = ld_sched128(&t->scales);  // scales, out
  const int4 p2 = ld_sched128(&t->epi);     // epi, pad
  const int4 i0 = ld_sched128(&t->k);
  const int4 i1 = ld_sched128(&t->group);
  ChainRec r;
  r.a = reinterpret_cast<const void*>(ptr_of(p0.z, p0.w));
  r.scales = reinterpret_cast<const void*>(ptr_of(p1.x, p1.y));
  r.out = reinterpret_cast<void*>(ptr_of(p1.z, p1.w));
  r.epi = reinterpret_cast<const EpiParams*>(ptr_of(p2.x, p2.y));
  r.k = i0.x; r.n = i0.y; r.tile_row = i0.z; r.phase = i0.w;
  r.group = i1.x; r.out_dtype = i1.y; r.wait_for = i1.z; r.arrive = i1.w;
  return r;
}

template <typename AT, int NT, bool GROUPED, int W, int S, int MINB>
__global__ void __launch_bounds__(W * 32, MINB) qgemv_chain_kernel(const ChainArgs c) {
  constexpr int kThreads = W * 32;
  extern __shared__ __align__(16) uint8_t chain_smem[];
  uint4* ring = reinterpret_cast<uint4*>(chain_smem);                               // [S][2][threads]
  float* red = reinterpret_cast<float*>(chain_smem + size_t(S) * 2 * kThreads * 16);  // [W][NT][4][32]
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const uint32_t ring_base = uint32_t(__cvta_generic_to_shared(ring)) + uint32_t(tid) * 16u;
  constexpr uint32_t kSlotBytes = kThreads * 16u;
  const ChainTile* my = c.sched + size_t(blockIdx.x) * size_t(c.stride);
  unsigned* abort_word = c.bar + c.n_phases;
  if (tid == 0) s_abort = 0;

  // ---- prefetch cursor: S k blocks ahead of the consumer, along the same flat sequence ----
  int fj = 0, left = 0;
  bool fend = false;
  const uint8_t *w_lo = nullptr, *w_hi = nullptr;
  ChainFetchRec fcur = chain_load_fetch(my), fnxt = chain_load_fetch(my + 1);
  auto fetch_open = [&]() {
    // settle on the next record that has k blocks for this warp, or on the end of the list
    while (true) {
      if (fcur.k == 0) { fend = true; left = 0; return; }
      left = ((fcur.k >> 6) - warp + W - 1) / W;
      if (left > 0) break;
      fcur = fnxt;
      ++fj;
      fnxt = chain_load_fetch(my + fj + 1);
    }
    const int last = fcur.n - 1 - fcur.tile_row;  // last valid row of the tile (clamped like the ring kernel)
    w_lo = fcur.w + int64_t(min(g, last)) * fcur.k + 16 * t + warp * 64;
    w_hi = fcur.w + int64_t(min(g + 8, last)) * fcur.k + 16 * t + warp * 64;
  };
  fetch_open();
  auto fetch_into = [&](int slot) {
    if (!fend) {
      cp_async16(ring_base + uint32_t(2 * slot) * kSlotBytes, w_lo);
      cp_async16(ring_base + uint32_t(2 * slot + 1) * kSlotBytes, w_hi);
      w_lo += W * 64;
      w_hi += W * 64;
      if (--left == 0) {
        fcur = fnxt;
        ++fj;
        fnxt = chain_load_fetch(my + fj + 1);  // needed a whole tile from now
        fetch_open();
      }
    }
    cp_async_commit();  // one group per step, empty or not, keeps wait_group's count uniform
  };
#pragma unroll 1
  for (int s = 0; s < S; ++s) fetch_into(s);
  __syncthreads();

  int slot = 0, cj = 0;
  ChainRec cur = chain_load_rec(my);
  while (cur.k != 0) {
    const ChainRec nxt = chain_load_rec(my + cj + 1);  // used at the end of this tile
    // ---- gate: the activations of this phase are the stores of the phases before it ----
    if (cur.wait_for > 0) {
      if (tid == 0) {
        const unsigned want = unsigned(cur.wait_for);
        unsigned spins = 0;
        while (ld_acquire_gpu(c.bar + (cur.phase - 1)) < want) {
          if (++spins > kChainSpinLimit || ld_acquire_gpu(abort_word) != 0u) {
            if (spins > kChainSpinLimit) { atomicExch(c.status, TL_DEV_TIMEOUT_FULL); atomicExch(abort_word, 1u); }
            s_abort = 1;
            break;
          }
          __nanosleep(20);
        }
      }
      __syncthreads();
      if (s_abort) break;
      __threadfence();
    }
    const int k = cur.k, n = cur.n;
    const int64_t tile_row = cur.tile_row;
    const AT* a = reinterpret_cast<const AT*>(cur.a);
    const AT* a_col[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) a_col[nt] = a + int64_t(min(g + 8 * nt, c.m - 1)) * k + 16 * t + warp * 64;
    const int nkb = ((k >> 6) - warp + W - 1) / W;
    const void* scales = cur.scales;
    const int group = GROUPED ? cur.group : 0, gpr = GROUPED ? k / cur.group : 0;
    const int64_t r_lo = min(tile_row + g, int64_t(n) - 1), r_hi = min(tile_row + g + 8, int64_t(n) - 1);

    // What the epilogue will need comes from global memory: ask for it now, so that the latency
    // hides behind the k loop instead of following it.
    constexpr int kOutPerThread = (NT * 128 + kThreads - 1) / kThreads;
    float pre_scale[kOutPerThread], pre_bias[kOutPerThread];
    const EpiParams& epi = *cur.epi;
    const int epi_fast = __ldg(&epi.fast), epi_unary = __ldg(&epi.fast_unary);
    const float epi_alpha = __ldg(&epi.alpha);
    const float* epi_bias = reinterpret_cast<const float*>(__ldg(reinterpret_cast<const unsigned long long*>(&epi.fast_bias)));
#pragma unroll
    for (int u = 0; u < kOutPerThread; ++u) {
      const int o = tid + u * kThreads;
      const int64_t row = tile_row + ((o & 31) >> 2) + (((o >> 5) & 2) ? 8 : 0);
      const bool live = o < NT * 128 && row < n;
      pre_scale[u] = (!GROUPED && live) ? tl_load_scale(scales, c.scales_dtype, row) : 1.f;
      pre_bias[u] = (live && epi_fast && epi_bias) ? __ldg(epi_bias + row) : 0.f;
    }

    float total[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) total[nt][i] = 0.f;

    // Activations are loaded PD k blocks ahead into a register queue.  With one or two tiles per
    // CTA and phase, every activation line is touched about once per SM, so these loads mostly
    // miss L1: an L2 round trip (~0.4 us) per k block unless it is issued well ahead.  The queue
    // is indexed statically (the loop is unrolled PD-fold): shifting it with moves would make
    // every move wait for the load still in flight to its source register.
    constexpr int PD = (W * 32 * MINB > 512) ? (NT == 1 ? 2 : 1) : (NT == 1 ? 3 : 2);
    uint4 bq[PD][NT][2];
#pragma unroll
    for (int d = 0; d < PD; ++d)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const AT* src = a_col[nt] + int64_t(d) * (W * 64);
        bq[d][nt][0] = d < nkb ? ld_act128(src) : make_uint4(0, 0, 0, 0);
        bq[d][nt][1] = d < nkb ? ld_act128(src + 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll 1
    for (int i0 = 0; i0 < nkb; i0 += PD) {
#pragma unroll
      for (int d = 0; d < PD; ++d) {
        const int i = i0 + d;
        if (i >= nkb) break;
        uint4 bx[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          bx[nt][0] = bq[d][nt][0];
          bx[nt][1] = bq[d][nt][1];
          if (i + PD < nkb) {
            const AT* src = a_col[nt] + int64_t(i + PD) * (W * 64);
            bq[d][nt][0] = ld_act128(src);
            bq[d][nt][1] = ld_act128(src + 8);
          }
        }
        cp_async_wait<S - 1>();
        const uint4 wl = ring[(2 * slot) * kThreads + tid];
        const uint4 wh = ring[(2 * slot + 1) * kThreads + tid];
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[nt][e] = GROUPED ? 0.f : total[nt][e];
        const uint32_t wlo[4] = {wl.x, wl.y, wl.z, wl.w};
        const uint32_t whi[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a0, a1, a2, a3;
          MmaOps<AT>::cvt(wlo[j], a0, a2);
          MmaOps<AT>::cvt(whi[j], a1, a3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 v = bx[nt][j >> 1];
            const uint32_t b0 = (j & 1) ? v.z : v.x, b1 = (j & 1) ? v.w : v.y;
            MmaOps<AT>::mma(acc[nt], a0, a1, a2, a3, b0, b1);
          }
        }
        fetch_into(slot);  // the slot's words are in registers and consumed: refill it
        slot = slot + 1 == S ? 0 : slot + 1;
        if (GROUPED) {
          const int gi = ((warp + i * W) * 64) / group;
          const float s_lo = tl_load_scale(scales, c.scales_dtype, r_lo * gpr + gi);
          const float s_hi = tl_load_scale(scales, c.scales_dtype, r_hi * gpr + gi);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            total[nt][0] = fmaf(s_lo, acc[nt][0], total[nt][0]);
            total[nt][1] = fmaf(s_lo, acc[nt][1], total[nt][1]);
            total[nt][2] = fmaf(s_hi, acc[nt][2], total[nt][2]);
            total[nt][3] = fmaf(s_hi, acc[nt][3], total[nt][3]);
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) total[nt][e] = acc[nt][e];
        }
      }
    }

    // ---- the W warps' partial tiles meet in shared memory; scale, epilogue, store ----
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[((warp * NT + nt) * 4 + i) * 32 + lane] = total[nt][i];
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kOutPerThread; ++u) {
      const int o = tid + u * kThreads;
      if (o >= NT * 128) break;
      const int nt = o >> 7, i = (o >> 5) & 3, ln = o & 31;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) v += red[((w * NT + nt) * 4 + i) * 32 + ln];
      const int gg = ln >> 2, tt = ln & 3;
      const int64_t row = tile_row + gg + ((i & 2) ? 8 : 0);
      const int col = 8 * nt + 2 * tt + (i & 1);
      if (row < n && col < c.m) {
        const float vs = v * (c.wscale * pre_scale[u]);
        float r;
        if (epi_fast) {
          // [bias][unary] chain, evaluated in the op interpreter's order and rounding
          r = __fmul_rn(vs, epi_alpha);
          if (epi_bias) r = __fadd_rn(r, pre_bias[u]);
          if (epi_unary) r = tl_unary(epi_unary, r);
        } else {
          r = tl_apply_epilogue(epi, vs, col, row, n);
        }
        tl_store_out(cur.out, cur.out_dtype, int64_t(col) * n + row, r);
      }
    }
    __syncthreads();  // the stores above are done, and `red` may be overwritten
    // ---- leaving a phase = one arrival on its counter ----
    if (cur.arrive && tid == 0) {
      __threadfence();
      atomicAdd(c.bar + cur.phase, 1u);
    }
    cur = nxt;
    ++cj;
  }
  cp_async_wait<0>();  // nothing of ours may still be landing when the CTA leaves
}

}  // namespace

struct tl_chain {
  ChainTile* d_sched = nullptr;
  EpiParams* d_epi = nullptr;
  unsigned* d_bar = nullptr;
  int32_t n_phases = 0, m = 0, a_dtype = 0, scales_dtype = 0, stride = 0;
  float wscale = 1.f;
  bool grouped = false;
  int32_t n_items = 0, n_epi = 0;
  int grid = 0, threads = 0, warps = 0, depth = 0;
  size_t smem = 0;
  const void* kernel = nullptr;
};

namespace {
// CTA shapes of the chain kernel: warps per tile x prefetch depth (k blocks in flight per thread),
// with the resident CTAs per SM the launch bounds ask for.
template <typename AT, int NT, bool GROUPED, int W, int S, int MINB>
void chain_set(tl_chain* ch) {
  ch->kernel = reinterpret_cast<const void*>(&qgemv_chain_kernel<AT, NT, GROUPED, W, S, MINB>);
  ch->threads = W * 32;
  ch->smem = size_t(S) * 2 * (W * 32) * 16 + size_t(W) * NT * 128 * sizeof(float);
}
template <typename AT, int NT, bool GROUPED>
bool chain_pick_shape(tl_chain* ch, int warps, int depth) {
  if (warps == 8 && depth == 12) { chain_set<AT, NT, GROUPED, 8, 12, 2>(ch); return true; }
  if (warps == 8 && depth == 8) { chain_set<AT, NT, GROUPED, 8, 8, 3>(ch); return true; }
  if (warps == 4 && depth == 12) { chain_set<AT, NT, GROUPED, 4, 12, 6>(ch); return true; }
  if (warps == 16 && depth == 12) { chain_set<AT, NT, GROUPED, 16, 12, 1>(ch); return true; }
  return false;
}
template <typename AT>
bool chain_pick_at(tl_chain* ch, int warps, int depth) {
  if (ch->m > 8) return ch->grouped ? chain_pick_shape<AT, 2, true>(ch, warps, depth) : chain_pick_shape<AT, 2, false>(ch, warps, depth);
  return ch->grouped ? chain_pick_shape<AT, 1, true>(ch, warps, depth) : chain_pick_shape<AT, 1, false>(ch, warps, depth);
}
}  // namespace

extern "C" int32_t tl_qgemv_chain_destroy(tl_ctx* ctx, tl_chain* chain) {
  TL_CHECK_CTX(ctx);
  if (!chain) return TL_OK;
  DeviceGuard guard(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (chain->d_sched) cudaFree(chain->d_sched);
  if (chain->d_epi) cudaFree(chain->d_epi);
  if (chain->d_bar) cudaFree(chain->d_bar);
  delete chain;
  return TL_OK;
}

extern "C" int32_t tl_qgemv_chain_create(tl_ctx* ctx, const tl_chain_phase* phases, int32_t n_phases, int32_t a_dtype,
                                         int32_t m, int32_t scales_dtype, int32_t scale_convention, tl_chain** out) {
  TL_CHECK_CTX(ctx);
  if (!out) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_chain_create: null output");
  *out = nullptr;
  if (!phases || n_phases < 1 || n_phases > 4096)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_chain_create: 1..4096 phases (got %d)", n_phases);
  if (m < 1 || m > 16) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_chain_create: m=%d outside the GEMV range [1,16]", m);
  if (a_dtype != TL_F16 && a_dtype != TL_BF16)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_chain_create: activations must be f16 or bf16");
  DeviceGuard guard(ctx->device);
  tl_chain* ch = new tl_chain();
  ch->n_phases = n_phases; ch->m = m; ch->a_dtype = a_dtype; ch->scales_dtype = scales_dtype;
  ch->wscale = scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;

  // ---- validate, flatten the epilogues ----
  std::vector<EpiParams> epis;
  for (int p = 0; p < n_phases; ++p) {
    const tl_chain_phase& src = phases[p];
    if (src.n_items < 1 || src.n_items > kChainMaxItems || src.k < 64 || src.k % 64 != 0 || src.k > (int64_t(1) << 30) ||
        src.group_size < 64 || src.group_size % 64 != 0 || src.k % src.group_size != 0 ||
        (reinterpret_cast<uintptr_t>(src.a) & 15)) {
      delete ch;
      return tl_set_error(ctx, TL_ERR_UNSUPPORTED,
                          "tl_qgemv_chain_create: phase %d: needs 1..4 items, K %% 64 == 0, group %% 64 == 0 dividing K, "
                          "16-byte aligned activations", p);
    }
    tl_quant_desc q{TL_SCHEME_INT8_GROUPED, src.group_size, scales_dtype, scale_convention};
    if (src.group_size != src.k) ch->grouped = true;
    for (int i = 0; i < src.n_items; ++i) {
      const tl_qgemv_item& si = src.items[i];
      int32_t rc = tl_check_qargs(ctx, "tl_qgemv_chain_create", src.a, a_dtype, si.packed, si.scales, si.out, src.out_dtype,
                                  m, si.n, src.k, &q);
      bool has_ops = false;
      EpiParams e{};
      if (rc == TL_OK) rc = tl_make_epi(ctx, si.epilogue, si.alpha, &e, &has_ops);
      if (rc == TL_OK && (si.n < 1 || si.n > (int64_t(1) << 30) || (reinterpret_cast<uintptr_t>(si.packed) & 15) || si.out == src.a))
        rc = tl_set_error(ctx, TL_ERR_INVALID_ARG,
                          "tl_qgemv_chain_create: phase %d item %d: n >= 1, 16-byte aligned weights, out != a", p, i);
      if (rc != TL_OK) { delete ch; return rc; }
      epis.push_back(e);
      ch->n_items++;
      ch->n_epi += has_ops ? 1 : 0;
    }
  }

  // ---- kernel shape and grid ----
  // a forced variant {TL_FAMILY_QGEMV, kernel 7 "chain", warps, depth} overrides the default shape
  ch->warps = 8; ch->depth = 12;
  if (ctx->has_forced && ctx->forced.family == TL_FAMILY_QGEMV && ctx->forced.kernel == kChain) {
    ch->warps = ctx->forced.p0; ch->depth = ctx->forced.p1;
  }
  if (!(a_dtype == TL_F16 ? chain_pick_at<__half>(ch, ch->warps, ch->depth) : chain_pick_at<__nv_bfloat16>(ch, ch->warps, ch->depth))) {
    const int w = ch->warps, d = ch->depth;
    delete ch;
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_chain_create: no chain kernel with %d warps x depth %d", w, d);
  }
  cudaError_t e = cudaFuncSetAttribute(ch->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ch->smem));
  int per_sm = 0;
  if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ch->kernel, ch->threads, ch->smem);
  if (e != cudaSuccess || per_sm < 1) {
    delete ch;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_chain_create: occupancy query failed: %s", cudaGetErrorString(e));
  }
  ch->grid = ctx->sm_count * per_sm;  // all of them co-resident: the launch is cooperative
  e = cudaMalloc(&ch->d_epi, epis.size() * sizeof(EpiParams));
  if (e == cudaSuccess) e = cudaMemcpy(ch->d_epi, epis.data(), epis.size() * sizeof(EpiParams), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    tl_qgemv_chain_destroy(ctx, ch);
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_chain_create: %s", cudaGetErrorString(e));
  }

  // ---- the schedule: tiles of successive phases dealt round-robin, each phase starting at the
  // CTA after the one the previous phase stopped at; one list of records per CTA ----
  std::vector<std::vector<ChainTile>> lists;
  lists.resize(size_t(ch->grid));
  int64_t start = 0;
  int64_t prev_tiles = 0;
  size_t epi_index = 0;
  for (int p = 0; p < n_phases; ++p) {
    const tl_chain_phase& src = phases[p];
    const int32_t wait_for = p == 0 ? 0 : int32_t(std::min<int64_t>(ch->grid, prev_tiles));
    std::vector<size_t> first_of_cta(size_t(ch->grid), size_t(-1));
    int64_t t = 0;
    for (int i = 0; i < src.n_items; ++i, ++epi_index) {
      const tl_qgemv_item& si = src.items[i];
      for (int64_t row = 0; row < si.n; row += 16, ++t) {
        const size_t cta = size_t((start + t) % ch->grid);
        ChainTile rec{};
        rec.w = reinterpret_cast<const uint8_t*>(si.packed) + row * src.k;
        rec.a = src.a; rec.scales = si.scales; rec.out = si.out; rec.epi = ch->d_epi + epi_index;
        rec.k = int32_t(src.k); rec.n = int32_t(si.n); rec.tile_row = int32_t(row); rec.phase = p;
        rec.group = src.group_size; rec.out_dtype = src.out_dtype;
        rec.wait_for = 0; rec.arrive = 0;
        auto& list = lists[cta];
        if (first_of_cta[cta] == size_t(-1)) {
          first_of_cta[cta] = list.size();
          rec.wait_for = wait_for;
        }
        list.push_back(rec);
      }
    }
    for (size_t cta = 0; cta < lists.size(); ++cta)
      if (first_of_cta[cta] != size_t(-1)) lists[cta].back().arrive = 1;  // its last tile of this phase
    start += t;
    prev_tiles = t;
  }
  size_t longest = 0;
  for (const auto& l : lists) longest = std::max(longest, l.size());
  ch->stride = int32_t(longest + 2);  // the list ends with an all-zero record, and the walk reads one past it
  std::vector<ChainTile> flat;
  flat.resize(lists.size() * size_t(ch->stride));
  for (size_t cta = 0; cta < lists.size(); ++cta)
    std::copy(lists[cta].begin(), lists[cta].end(), flat.begin() + cta * size_t(ch->stride));
  e = cudaMalloc(&ch->d_sched, flat.size() * sizeof(ChainTile));
  if (e == cudaSuccess) e = cudaMalloc(&ch->d_bar, size_t(n_phases + 1) * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemcpy(ch->d_sched, flat.data(), flat.size() * sizeof(ChainTile), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    tl_qgemv_chain_destroy(ctx, ch);
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_chain_create: %s", cudaGetErrorString(e));
  }
  *out = ch;
  return TL_OK;
}

extern "C" int32_t tl_qgemv_chain_launch(tl_ctx* ctx, tl_chain* chain) {
  TL_CHECK_CTX(ctx);
  if (!chain) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_chain_launch: null chain");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaMemsetAsync(chain->d_bar, 0, size_t(chain->n_phases + 1) * sizeof(unsigned), ctx->stream));
  ChainArgs args{};
  args.sched = chain->d_sched; args.bar = chain->d_bar; args.status = ctx->dev_status;
  args.stride = chain->stride; args.n_phases = chain->n_phases; args.m = chain->m;
  args.scales_dtype = chain->scales_dtype; args.wscale = chain->wscale;
  void* kargs[] = {&args};
  cudaError_t e = cudaLaunchCooperativeKernel(chain->kernel, dim3(unsigned(chain->grid)), dim3(unsigned(chain->threads)), kargs,
                                              chain->smem, ctx->stream);
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_chain_launch: %s", cudaGetErrorString(e));
  }
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  ctx->counters[TL_COUNTER_QGEMV] += chain->n_items;
  ctx->counters[TL_COUNTER_QGEMV_EPILOGUE] += chain->n_epi;
  return TL_OK;
}


// ---------------------------------------------------------------------------
// Fused row-parallel GEMV + all-reduce (host side)
// ---------------------------------------------------------------------------
namespace {
template <typename AT, int NT, bool GROUPED>
cudaError_t launch_ring_allreduce(int grid, int block, cudaStream_t s, const GemvArgs& p, const EpiParams& e, const PushArgs& q) {
  constexpr int S = 4;
  const size_t smem = size_t(S) * 2 * block * 16 + size_t(block / 32) * NT * 128 * 4;
  auto kern = qgemv_ring_allreduce_kernel<AT, NT, GROUPED, S>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p, e, q);
}
template <typename AT>
cudaError_t launch_ring_allreduce_at(bool two, bool grouped, int grid, int block, cudaStream_t s, const GemvArgs& p,
                                     const EpiParams& e, const PushArgs& q) {
  if (two) return grouped ? launch_ring_allreduce<AT, 2, true>(grid, block, s, p, e, q) : launch_ring_allreduce<AT, 2, false>(grid, block, s, p, e, q);
  return grouped ? launch_ring_allreduce<AT, 1, true>(grid, block, s, p, e, q) : launch_ring_allreduce<AT, 1, false>(grid, block, s, p, e, q);
}
}  // namespace

extern "C" int32_t tl_qgemv_nt_allreduce(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed, const void* scales,
                                         void* out, int32_t out_dtype, int32_t m, int64_t n, int64_t k,
                                         const tl_quant_desc* qdesc, float alpha) {
  TL_CHECK_CTX(ctx);
  if (ctx->world <= 1)  // nothing to sum: the plain product
    return tl_qgemv_nt(ctx, a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc, alpha, nullptr);
  int32_t rc = tl_check_qargs(ctx, "tl_qgemv_nt_allreduce", a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc);
  if (rc != TL_OK) return rc;
  if (m < 1 || m > 16) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_allreduce: m=%d outside the GEMV range [1,16]", m);
  if (!ctx->p2p_attached) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_allreduce: peers not attached (tl_p2p_create / tl_p2p_attach)");
  if (!(a_dtype == TL_F16 || a_dtype == TL_BF16) || k % 64 != 0 || qdesc->group_size % 64 != 0 ||
      (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(packed) & 15))
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED,
                        "tl_qgemv_nt_allreduce: needs f16/bf16 activations, K %% 64 == 0, group %% 64 == 0, 16-byte aligned operands");
  const int64_t tiles = (n + 15) / 16;
  if (n < 1 || tiles > kP2PFusedMaxTiles)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_nt_allreduce: n=%lld outside [1, %d]", (long long)n, 16 * kP2PFusedMaxTiles);
  if (size_t(m) * size_t(n) * tl_dtype_size(out_dtype) > ctx->p2p_max_bytes)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_nt_allreduce: %zu bytes exceed the exchange buffer (%zu)",
                        size_t(m) * size_t(n) * tl_dtype_size(out_dtype), ctx->p2p_max_bytes);
  // The tile counters count uses, so every fused call on a context must cover the same tiles.
  if (ctx->fused_tiles != 0 && ctx->fused_tiles != tiles)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_nt_allreduce: every call on a context must have the same n (first call: %lld rows)",
                        (long long)ctx->fused_tiles * 16);
  EpiParams epi;
  bool has_ops = false;
  rc = tl_make_epi(ctx, nullptr, alpha, &epi, &has_ops);
  if (rc != TL_OK) return rc;
  DeviceGuard guard(ctx->device);
  GemvArgs p{};
  p.a = a; p.packed = reinterpret_cast<const uint32_t*>(packed); p.scales = scales; p.out = out;
  p.m = m; p.n = int32_t(n); p.k = int32_t(k);
  p.group = qdesc->group_size; p.groups_per_row = int32_t(k / qdesc->group_size);
  p.scales_dtype = qdesc->scales_dtype; p.out_dtype = out_dtype;
  p.wscale = qdesc->scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
  p.row0 = 0; p.m_total = m;
  PushArgs q{};
  for (int r = 0; r < ctx->world; ++r) q.base[r] = static_cast<uint8_t*>(ctx->p2p_peer[r]);
  q.rank = ctx->rank; q.world = ctx->world; q.max_bytes = ctx->p2p_max_bytes; q.dst = out; q.status = ctx->dev_status;
  q.spin_limit = ctx->wait_limit_polls < (1 << 22) ? ctx->wait_limit_polls : (1 << 22);
  // widest CTA that keeps the launch in one wave at two resident CTAs per SM
  int warps = 4;
  for (int w : {16, 8})
    if (tiles <= int64_t(ctx->sm_count) * (1024 / (w * 32))) { warps = w; break; }
  const int block = warps * 32, grid = int(tiles);
  const bool grouped = qdesc->group_size != k;
  cudaError_t e = a_dtype == TL_F16 ? launch_ring_allreduce_at<__half>(m > 8, grouped, grid, block, ctx->stream, p, epi, q)
                                    : launch_ring_allreduce_at<__nv_bfloat16>(m > 8, grouped, grid, block, ctx->stream, p, epi, q);
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_nt_allreduce: launch failed: %s", cudaGetErrorString(e));
  }
  ctx->fused_tiles = tiles;
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  ctx->counters[TL_COUNTER_QGEMV]++;
  return TL_OK;
}


// ---------------------------------------------------------------------------
// Push / reduce-on-read (host side)
// ---------------------------------------------------------------------------
namespace {
template <typename K, typename... Args>
cudaError_t launch_pdl_args(K kern, int grid, int block, size_t smem, cudaStream_t s, Args... args) {
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}
constexpr int kTpStages = 4;  // ring depth of the tensor-parallel launches (their k loops are short)
inline size_t tp_smem(int block, int nt) { return size_t(kTpStages) * 2 * block * 16 + size_t(block / 32) * nt * 128 * 4; }

#define TL_TP_GO(KERN_, NT_, ...)                                                                  \
  do {                                                                                            \
    auto kern = KERN_;                                                                            \
    const int block = tp_warps_for(ctx, kern, NT_, grid) * 32;                                    \
    return launch_pdl_args(kern, grid, block, tp_smem(block, NT_), ctx->stream, __VA_ARGS__);     \
  } while (0)
template <typename AT>
cudaError_t launch_push(tl_ctx* ctx, bool two, bool grouped, int grid, const GemvArgs& p, const EpiParams& e, const PushArgs& q) {
  if (two) {
    if (grouped) TL_TP_GO((qgemv_ring_push_kernel<AT, 2, true, kTpStages>), 2, p, e, q);
    TL_TP_GO((qgemv_ring_push_kernel<AT, 2, false, kTpStages>), 2, p, e, q);
  }
  if (grouped) TL_TP_GO((qgemv_ring_push_kernel<AT, 1, true, kTpStages>), 1, p, e, q);
  TL_TP_GO((qgemv_ring_push_kernel<AT, 1, false, kTpStages>), 1, p, e, q);
}
template <typename AT>
cudaError_t launch_rin(tl_ctx* ctx, bool two, bool grouped, int grid, const GemvArgs& p, const EpiParams& e, ReduceIn r) {
  r.nsum = std::min(grid, 32);
  if (two) {
    if (grouped) TL_TP_GO((qgemv_ring_rin_kernel<AT, 2, true, kTpStages>), 2, p, e, r);
    TL_TP_GO((qgemv_ring_rin_kernel<AT, 2, false, kTpStages>), 2, p, e, r);
  }
  if (grouped) TL_TP_GO((qgemv_ring_rin_kernel<AT, 1, true, kTpStages>), 1, p, e, r);
  TL_TP_GO((qgemv_ring_rin_kernel<AT, 1, false, kTpStages>), 1, p, e, r);
}
template <typename AT>
cudaError_t launch_rin_batched(tl_ctx* ctx, bool two, bool grouped, int grid, const RingBatchArgs& b, ReduceIn r) {
  r.nsum = std::min(grid, 32);
  if (two) {
    if (grouped) TL_TP_GO((qgemv_ring_rin_batched_kernel<AT, 2, true, kTpStages>), 2, b, r);
    TL_TP_GO((qgemv_ring_rin_batched_kernel<AT, 2, false, kTpStages>), 2, b, r);
  }
  if (grouped) TL_TP_GO((qgemv_ring_rin_batched_kernel<AT, 1, true, kTpStages>), 1, b, r);
  TL_TP_GO((qgemv_ring_rin_batched_kernel<AT, 1, false, kTpStages>), 1, b, r);
}
#undef TL_TP_GO

// stand-alone form of the consumer's prologue (tl_reduce_pending)
__global__ void __launch_bounds__(256) reduce_pending_kernel(const __grid_constant__ ReduceIn rin) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  reduce_in_prologue(rin);
}

// CTA width of a tensor-parallel launch: the widest CTA whose whole launch is resident at once (one
// wave), asked of the occupancy calculator for the kernel that will actually run.
template <typename K>
int tp_warps_for(tl_ctx* ctx, K kern, int nt, int64_t tiles) {
  for (int w : {16, 8, 4}) {
    const size_t smem = tp_smem(w * 32, nt);
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, w * 32, smem) != cudaSuccess) { cudaGetLastError(); occ = 0; }
    if (int64_t(occ) * ctx->sm_count >= tiles) return w;
  }
  return 4;
}

ReduceIn make_reduce_in(tl_ctx* ctx, void* dst, int grid) {
  ReduceIn r{};
  r.base = static_cast<uint8_t*>(ctx->p2p_local);
  r.max_bytes = ctx->p2p_max_bytes;
  r.dst = dst;
  r.world = ctx->world;
  r.expected = 0;
  r.nsum = std::min(grid, 32);
  r.count_vec = int32_t(int64_t(ctx->push_m) * ctx->push_n * 2 / 16);
  r.dtype = ctx->push_dtype;
  r.status = ctx->dev_status;
  r.spin_limit = ctx->wait_limit_polls;
  r.poll_ranks = ctx->push_poll_ranks;
  return r;
}
}  // namespace

// Can the pending push be reduced by a launch that reads `a` as [m, k] activations of a_dtype?
bool tl_push_matches(tl_ctx* ctx, const void* a, int32_t a_dtype, int32_t m, int64_t k) {
  return ctx->push_pending && a == ctx->push_dst && a_dtype == ctx->push_dtype && m == ctx->push_m && k == ctx->push_n;
}

extern "C" int32_t tl_qgemv_nt_push(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed, const void* scales,
                                    void* out, int32_t out_dtype, int32_t m, int64_t n, int64_t k, const tl_quant_desc* qdesc,
                                    float alpha) {
  TL_CHECK_CTX(ctx);
  if (ctx->world <= 1 && !ctx->p2p_attached)  // nothing to sum: the plain product, straight into out
    return tl_qgemv_nt(ctx, a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc, alpha, nullptr);
  int32_t rc = tl_check_qargs(ctx, "tl_qgemv_nt_push", a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc);
  if (rc != TL_OK) return rc;
  if (m < 1 || m > 16) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_push: m=%d outside the GEMV range [1,16]", m);
  if (!ctx->p2p_attached) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_push: peers not attached (tl_p2p_create / tl_p2p_attach)");
  if (ctx->push_pending)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_qgemv_nt_push: the previous push has not been reduced yet (run the launch that reads it, or tl_reduce_pending)");
  if (!(a_dtype == TL_F16 || a_dtype == TL_BF16) || !(out_dtype == TL_F16 || out_dtype == TL_BF16) || k % 64 != 0 ||
      qdesc->group_size % 64 != 0 || n % 16 != 0 || n < 16 || (reinterpret_cast<uintptr_t>(a) & 15) ||
      (reinterpret_cast<uintptr_t>(packed) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED,
                        "tl_qgemv_nt_push: needs f16/bf16 activations and outputs, K %% 64 == 0, group %% 64 == 0, N %% 16 == 0, 16-byte aligned operands");
  if (size_t(m) * size_t(n) * 4 > ctx->p2p_max_bytes)  // two 24-bit partial sums and a 16-bit tag per 8-byte word
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_qgemv_nt_push: %zu bytes exceed the exchange buffer (%zu)", size_t(m) * size_t(n) * 4,
                        ctx->p2p_max_bytes);
  EpiParams epi;
  bool has_ops = false;
  rc = tl_make_epi(ctx, nullptr, alpha, &epi, &has_ops);
  if (rc != TL_OK) return rc;
  DeviceGuard guard(ctx->device);
  GemvArgs p{};
  p.a = a; p.packed = reinterpret_cast<const uint32_t*>(packed); p.scales = scales; p.out = out;
  p.m = m; p.n = int32_t(n); p.k = int32_t(k);
  p.group = qdesc->group_size; p.groups_per_row = int32_t(k / qdesc->group_size);
  p.scales_dtype = qdesc->scales_dtype; p.out_dtype = out_dtype;
  p.wscale = qdesc->scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
  p.row0 = 0; p.m_total = m;
  PushArgs q{};
  for (int r = 0; r < ctx->world; ++r) q.base[r] = static_cast<uint8_t*>(ctx->p2p_peer[r]);
  q.rank = ctx->rank; q.world = ctx->world; q.max_bytes = ctx->p2p_max_bytes; q.dst = out; q.status = ctx->dev_status;
  q.spin_limit = ctx->wait_limit_polls;
  const int64_t tiles = n / 16;
  const int grid = int(tiles);
  const bool grouped = qdesc->group_size != k;
  cudaError_t e = a_dtype == TL_F16 ? launch_push<__half>(ctx, m > 8, grouped, grid, p, epi, q)
                                    : launch_push<__nv_bfloat16>(ctx, m > 8, grouped, grid, p, epi, q);
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_qgemv_nt_push: launch failed: %s", cudaGetErrorString(e));
  }
  ctx->push_pending = true;
  ctx->push_dst = out; ctx->push_m = m; ctx->push_n = n; ctx->push_tiles = tiles; ctx->push_dtype = out_dtype;
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  ctx->counters[TL_COUNTER_QGEMV]++;
  return TL_OK;
}

extern "C" int32_t tl_reduce_pending(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  if (!ctx->push_pending) return TL_OK;
  DeviceGuard guard(ctx->device);
  const int grid = 16;
  const ReduceIn r = make_reduce_in(ctx, ctx->push_dst, grid);
  cudaError_t e = launch_pdl_args(reduce_pending_kernel, grid, 256, 0, ctx->stream, r);
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_reduce_pending: launch failed: %s", cudaGetErrorString(e));
  }
  ctx->push_pending = false;
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

// One launch that reduces the pending push into `a` and then runs up to four products over it.
int32_t tl_launch_qgemv_rin(tl_ctx* ctx, const void* a, int32_t a_dtype, const GemvArgs* items, const EpiParams* epis, int n_items,
                            int32_t m, int64_t k, bool grouped) {
  int64_t tiles = 0;
  RingBatchArgs b{};
  for (int i = 0; i < kMaxBatchItems; ++i) {
    b.tile_start[i] = int32_t(tiles);
    if (i >= n_items) continue;
    b.p[i] = items[i];
    b.e[i] = epis[i];
    tiles += (items[i].n + 15) / 16;
  }
  b.tile_start[kMaxBatchItems] = int32_t(tiles);
  const int grid = int(tiles);
  const ReduceIn r = make_reduce_in(ctx, const_cast<void*>(a), grid);
  cudaError_t e;
  if (n_items == 1)
    e = a_dtype == TL_F16 ? launch_rin<__half>(ctx, m > 8, grouped, grid, items[0], epis[0], r)
                          : launch_rin<__nv_bfloat16>(ctx, m > 8, grouped, grid, items[0], epis[0], r);
  else
    e = a_dtype == TL_F16 ? launch_rin_batched<__half>(ctx, m > 8, grouped, grid, b, r)
                          : launch_rin_batched<__nv_bfloat16>(ctx, m > 8, grouped, grid, b, r);
  if (e != cudaSuccess) {
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_CUDA, "qgemv: reduce-on-read launch failed: %s", cudaGetErrorString(e));
  }
  ctx->push_pending = false;
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}
