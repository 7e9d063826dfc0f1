// int4-grouped: the second weight-only scheme, which the reference plans but does not implement
// (docs/quantization-design.md:69-75, 386-396: "8 int4 per u32 word, packed 8-along-K into [N, K/8] u32,
// ... unpacks a nibble ((word >> (4*j)) & 0xF, sign-extend from 4 bits)"; "a new VALUE on the format
// axis: a scheme entry + unpackInt4 in the kernel", reusing the seam).  Everything here follows the int8
// path with the range [-7, 7]: scales are the f16 bits of the group abs-max (w = (q / 7) * scale), or
// f32 "direct" scales (w = q * s).
//
//   host quantizer        tl_quantize_linear_weight_int4 (same arithmetic as the int8 quantizer)
//   explicit dequant      tl_dequant_int4 (f64 through a 16-entry table, one rounding: bit-exact)
//   small batch, m <= 16  qgemv_int4_mma_kernel (f16 / bf16 activations, K and the group multiples of
//                         128): mma.sync with the nibbles converted pairwise, see below; else
//                         qgemv_int4_kernel: warp per R rows, one packed word (8 weights) per lane and
//                         step -- a warp reads 128 contiguous bytes of each row per step -- nibbles to
//                         f32 by exponent stuffing, f32 FMA, group scale applied to the group's partial
//                         sum, warp-shuffle reduction, the common epilogue.  HBM-bound at m <= 2
//                         (0.5 byte per weight against 3 ALU ops per weight and one FMA per batch
//                         row); FMA-bound above that.
//   m > 16                explicit dequant into library scratch in the activation type, then the dense
//                         matmul (tl_matmul: tcgen05 when it applies) -- the reference's fallback for
//                         every m > 1 (src/backend/webgpu/ops/matmul-ops.ts:163-181).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "tl_common.cuh"
#include "tl_mma_frag.cuh"

namespace {

inline double round_half_up(double x) {  // JS Math.round
  const double f = std::floor(x);
  return (x - f >= 0.5) ? f + 1.0 : f;
}

void quantize_rows_int4(const float* weight, int64_t row0, int64_t row1, int64_t k, int32_t group, uint32_t* packed,
                        uint16_t* scales) {
  const int64_t groups = k / group, words = k / 8;
  for (int64_t row = row0; row < row1; ++row) {
    const float* w = weight + row * k;
    uint32_t* pw = packed + row * words;
    std::memset(pw, 0, size_t(words) * 4);
    for (int64_t g = 0; g < groups; ++g) {
      const float* wg = w + g * group;
      float amax = 0.f;
      for (int32_t j = 0; j < group; ++j) amax = std::max(amax, std::fabs(wg[j]));
      const uint32_t sbits = tl_f32_to_f16_bits(amax);
      scales[row * groups + g] = uint16_t(sbits);
      // the scale that is stored is the scale that quantizes: widen the f16 bits back exactly
      const double s = double(tl_f16_bits_to_f32(sbits));
      const double inv = s > 0 ? 7.0 / s : 0.0;
      for (int32_t j = 0; j < group; ++j) {
        double q = round_half_up(double(wg[j]) * inv);
        q = std::isnan(q) ? 0.0 : std::max(-7.0, std::min(7.0, q));
        const int64_t kk = g * group + j;
        pw[kk >> 3] |= (uint32_t(int32_t(q)) & 0xfu) << ((kk & 7) * 4);
      }
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(256)
dequant_int4_kernel(const uint32_t* __restrict__ packed, const void* __restrict__ scales, OutT* __restrict__ out, int64_t n_words,
                    int32_t words_per_row, int32_t group, int32_t groups_per_row, int32_t scales_dtype, int32_t convention) {
  __shared__ double lut[16];  // q/7 (snorm) or q (direct), indexed by the raw nibble
  if (threadIdx.x < 16) {
    const int q = threadIdx.x >= 8 ? int(threadIdx.x) - 16 : int(threadIdx.x);
    lut[threadIdx.x] = convention == TL_SCALE_SNORM127 ? double(q) / 7.0 : double(q);
  }
  __syncthreads();
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t wi = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; wi < n_words; wi += stride) {
    const int64_t row = wi / words_per_row;
    const int32_t k0 = int32_t(wi - row * words_per_row) * 8;
    const uint32_t word = __ldg(packed + wi);
    OutT* o = out + wi * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const double s = double(tl_load_scale(scales, scales_dtype, row * groups_per_row + (k0 + j) / group));
      o[j] = DT<OutT>::from_f32(float(lut[(word >> (4 * j)) & 0xfu] * s));
    }
  }
}

__global__ void __launch_bounds__(256) unpack_int4_kernel(const uint32_t* __restrict__ packed, int8_t* __restrict__ out, int64_t n_words) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t wi = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; wi < n_words; wi += stride) {
    const uint32_t w = __ldg(packed + wi);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= (uint32_t(int32_t(w << (28 - 4 * j)) >> 28) & 0xffu) << (8 * j);
      hi |= (uint32_t(int32_t(w << (12 - 4 * j)) >> 28) & 0xffu) << (8 * j);
    }
    reinterpret_cast<uint2*>(out)[wi] = make_uint2(lo, hi);
  }
}

struct Int4Args {
  const void* a;
  const uint32_t* packed;
  const void* scales;
  void* out;
  int32_t m, n, k, row0;     // this launch's batch rows are [row0, row0 + m)
  int32_t group, groups_per_row, scales_dtype, out_dtype;
  float wscale;              // 1/7 for the abs-max convention, 1 for direct scales
};

template <typename AT> __device__ __forceinline__ void load8(const AT* p, float (&x)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&x)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float (&x)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    x[2 * i] = f.x; x[2 * i + 1] = f.y;
  }
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { x[2 * i] = __uint_as_float(w[i] << 16); x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}

// warp per R rows; lane per packed word (8 weights, one group: group % 8 == 0)
template <typename AT, int MT, int R>
__global__ void __launch_bounds__(256) qgemv_int4_kernel(Int4Args p, EpiParams epi) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_base = (int64_t(blockIdx.x) * warps + (threadIdx.x >> 5)) * R;
  if (row_base >= p.n) return;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const int words = p.k >> 3;
  int64_t rows[R];
#pragma unroll
  for (int r = 0; r < R; ++r) rows[r] = min(row_base + r, int64_t(p.n) - 1);  // tail rows clamp, stores mask
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[r][i] = 0.f;
  for (int c = lane; c < words; c += 32) {
    uint32_t wv[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wv[r] = __ldg(p.packed + rows[r] * words + c);
    float x[MT][8];
#pragma unroll
    for (int i = 0; i < MT; ++i) load8<AT>(a + int64_t(i) * p.k + int64_t(c) * 8, x[i]);
    const int grp = (c * 8) / p.group;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t u = wv[r] ^ 0x88888888u;  // two's complement nibble -> q + 8
      float part[MT];
#pragma unroll
      for (int i = 0; i < MT; ++i) part[i] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // (q + 8) into the mantissa of 2^23, minus (2^23 + 8): q exactly
        const float q = __uint_as_float(((u >> (4 * j)) & 0xfu) | 0x4B000000u) - 8388616.f;
#pragma unroll
        for (int i = 0; i < MT; ++i) part[i] = fmaf(q, x[i][j], part[i]);
      }
      const float s = tl_load_scale(p.scales, p.scales_dtype, rows[r] * p.groups_per_row + grp);
#pragma unroll
      for (int i = 0; i < MT; ++i) acc[r][i] = fmaf(s, part[i], acc[r][i]);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int64_t row = row_base + r;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      float v = acc[r][i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && row < p.n) {
        const float o = tl_apply_epilogue(epi, v * p.wscale, p.row0 + i, row, p.n);
        tl_store_out(p.out, p.out_dtype, int64_t(p.row0 + i) * p.n + row, o);
      }
    }
  }
}

template <typename AT, int MT>
void launch_int4(tl_ctx* ctx, const Int4Args& p, const EpiParams& e) {
  constexpr int R = MT >= 4 ? 2 : 4;
  const int warps = 8;
  const int64_t rows_per_cta = int64_t(warps) * R;
  const int grid = int((p.n + rows_per_cta - 1) / rows_per_cta);
  qgemv_int4_kernel<AT, MT, R><<<grid, warps * 32, 0, ctx->stream>>>(p, e);
}

template <typename AT>
void launch_int4_m(tl_ctx* ctx, Int4Args p, const EpiParams& epi, int m) {
  const uint8_t* a0 = static_cast<const uint8_t*>(p.a);
  // column tiles of 4, 2 and 1 batch rows (each launch re-reads the weights: FMA-bound territory anyway)
  for (int m0 = 0; m0 < m;) {
    const int mt = m - m0 >= 4 ? 4 : m - m0 >= 2 ? 2 : 1;
    p.a = a0 + size_t(m0) * p.k * sizeof(AT);
    p.row0 = m0; p.m = mt;
    if (mt == 4) launch_int4<AT, 4>(ctx, p, epi);
    else if (mt == 2) launch_int4<AT, 2>(ctx, p, epi);
    else launch_int4<AT, 1>(ctx, p, epi);
    ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
    m0 += mt;
  }
}

// ---------------------------------------------------------------------------
// Tensor-core form (f16 / bf16 activations, K % 128 == 0, group % 128 == 0): CTA per 16 weight rows,
// warps interleaved over 128-wide k blocks.  Lane (g, t) loads 16 bytes = 32 nibbles of rows g and
// g + 8 and the matching 32 activations of batch row g.  (w ^ 0x88888888) turns every nibble into
// q + 8; a mask and a magic exponent make the pair (q_x + 8, q_{x+4} + 8) 16-bit floats 1024 + .
// (f16) or 128 + . (bf16), and one subtraction -- or, for the nibbles taken at bits 4-7, one fused
// multiply-add -- gives (q_x, q_{x+4}) exactly (Nib::quad).  A word of eight
// nibbles feeds two mma.sync.m16n8k16; the activations are paired the same way with two byte
// permutes per MMA.  One group per k block: the block's accumulators are folded into the totals
// with the rows' scales (per-channel scales once at the end).
// ---------------------------------------------------------------------------
// quad(u, v): the four MMA operand registers of one word u (nibbles already q + 8):
//   v[0] = (q0, q4), v[1] = (q1, q5), v[2] = (q2, q6), v[3] = (q3, q7)
template <typename AT> struct Nib;
template <> struct Nib<__half> {
  // ONE shift per word: nibbles at bits 0-3 give 1024 + n, nibbles at bits 4-7 give 1024 + 16 n, which
  // one fused multiply-add turns into n - 8 exactly ((1024 + 16 n) / 16 - 72); the upper half of the
  // word goes through the same two masks after a shift by 8.
  __device__ static void quad(uint32_t u, uint32_t (&v)[4]) {
    const __half2 k1032 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
    const __half2 k16th = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));   // 1/16
    const __half2 km72 = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));    // -72
    const uint32_t u8 = u >> 8;
    const uint32_t a = (u & 0x000F000Fu) | 0x64006400u, b = (u & 0x00F000F0u) | 0x64006400u;
    const uint32_t c = (u8 & 0x000F000Fu) | 0x64006400u, d = (u8 & 0x00F000F0u) | 0x64006400u;
    const __half2 r0 = __hsub2(*reinterpret_cast<const __half2*>(&a), k1032);
    const __half2 r1 = __hfma2(*reinterpret_cast<const __half2*>(&b), k16th, km72);
    const __half2 r2 = __hsub2(*reinterpret_cast<const __half2*>(&c), k1032);
    const __half2 r3 = __hfma2(*reinterpret_cast<const __half2*>(&d), k16th, km72);
    v[0] = *reinterpret_cast<const uint32_t*>(&r0); v[1] = *reinterpret_cast<const uint32_t*>(&r1);
    v[2] = *reinterpret_cast<const uint32_t*>(&r2); v[3] = *reinterpret_cast<const uint32_t*>(&r3);
  }
};
template <> struct Nib<__nv_bfloat16> {
  // seven mantissa bits hold 128 + n only for a nibble at bits 0-3: one shift per pair
  __device__ static void quad(uint32_t u, uint32_t (&v)[4]) {
    const uint32_t m = 0x43084308u;  // 136 | 136
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const uint32_t w = ((u >> (4 * x)) & 0x000F000Fu) | 0x43004300u;
      const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&w), *reinterpret_cast<const __nv_bfloat162*>(&m));
      v[x] = *reinterpret_cast<const uint32_t*>(&r);
    }
  }
};

template <typename AT, int NT, bool GROUPED>
__global__ void __launch_bounds__(512) qgemv_int4_mma_kernel(Int4Args p, EpiParams epi) {
  extern __shared__ float red4[];  // [warps][NT][4][32]
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t tile_row = int64_t(blockIdx.x) * 16;
  const int64_t r_lo = min(tile_row + g, int64_t(p.n) - 1), r_hi = min(tile_row + g + 8, int64_t(p.n) - 1);
  const uint8_t* wb = reinterpret_cast<const uint8_t*>(p.packed);
  const int64_t row_bytes = p.k >> 1;
  const uint8_t* w_lo = wb + r_lo * row_bytes + 16 * t;
  const uint8_t* w_hi = wb + r_hi * row_bytes + 16 * t;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const AT* x_row[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) x_row[nt] = a + int64_t(min(g + 8 * nt, p.m - 1)) * p.k + 32 * t;
  float total[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) total[nt][i] = 0.f;
  const int kblocks = p.k >> 7;
  // one 128-wide k block: 8 MMAs per batch tile, on two accumulators so that only four are dependent
  auto block = [&](const uint4& wl4, const uint4& wh4, float s_lo, float s_hi, int kb) {
    const uint32_t wl[4] = {wl4.x ^ 0x88888888u, wl4.y ^ 0x88888888u, wl4.z ^ 0x88888888u, wl4.w ^ 0x88888888u};
    const uint32_t wh[4] = {wh4.x ^ 0x88888888u, wh4.y ^ 0x88888888u, wh4.z ^ 0x88888888u, wh4.w ^ 0x88888888u};
    float c[NT][4], d[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) { c[nt][i] = GROUPED ? 0.f : total[nt][i]; d[nt][i] = 0.f; }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t lo[4], hi[4];
      Nib<AT>::quad(wl[j], lo);
      Nib<AT>::quad(wh[j], hi);
      const uint32_t a00 = lo[0], a01 = hi[0], a02 = lo[1], a03 = hi[1];
      const uint32_t a10 = lo[2], a11 = hi[2], a12 = lo[3], a13 = hi[3];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x_row[nt] + int64_t(kb) * 128) + j);  // x0..x7 of this word
        MmaOps<AT>::mma(c[nt], a00, a01, a02, a03, __byte_perm(xv.x, xv.z, 0x5410), __byte_perm(xv.x, xv.z, 0x7632));
        MmaOps<AT>::mma(d[nt], a10, a11, a12, a13, __byte_perm(xv.y, xv.w, 0x5410), __byte_perm(xv.y, xv.w, 0x7632));
      }
    }
    if (GROUPED) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        total[nt][0] = fmaf(s_lo, c[nt][0] + d[nt][0], total[nt][0]); total[nt][1] = fmaf(s_lo, c[nt][1] + d[nt][1], total[nt][1]);
        total[nt][2] = fmaf(s_hi, c[nt][2] + d[nt][2], total[nt][2]); total[nt][3] = fmaf(s_hi, c[nt][3] + d[nt][3], total[nt][3]);
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[nt][i] = c[nt][i] + d[nt][i];
    }
  };
  // Two blocks' weights (and their scales) are always in flight.  (Programmatic dependent launch with
  // the first loads ahead of griddepcontrol.wait measured slightly slower here, 17.8 against 16.6 us.)
  // the rows' group scales of a block travel with its weights (loaded in the loop they cost an
  // exposed L2 / DRAM round trip per block: the scale array is read once, like the weights)
  const int shift = 31 - __clz(p.group >> 7);  // group = 128 << shift when GROUPED takes this kernel's power-of-two path
  const bool pow2 = (p.group & (p.group - 1)) == 0;
  auto scale_of = [&](int64_t row, int kblk) -> float {
    if (!GROUPED) return 1.f;
    const int grp = pow2 ? (kblk >> shift) : (kblk * 128) / p.group;
    return tl_load_scale(p.scales, p.scales_dtype, row * p.groups_per_row + grp);
  };
  int kb = warp;
  bool have0 = kb < kblocks, have1 = kb + warps < kblocks;
  uint4 l0 = make_uint4(0, 0, 0, 0), h0 = l0, l1 = l0, h1 = l0;
  float sl0 = 0.f, sh0 = 0.f, sl1 = 0.f, sh1 = 0.f;
  if (have0) {
    l0 = __ldg(reinterpret_cast<const uint4*>(w_lo + int64_t(kb) * 64));
    h0 = __ldg(reinterpret_cast<const uint4*>(w_hi + int64_t(kb) * 64));
    sl0 = scale_of(r_lo, kb); sh0 = scale_of(r_hi, kb);
  }
  if (have1) {
    l1 = __ldg(reinterpret_cast<const uint4*>(w_lo + int64_t(kb + warps) * 64));
    h1 = __ldg(reinterpret_cast<const uint4*>(w_hi + int64_t(kb + warps) * 64));
    sl1 = scale_of(r_lo, kb + warps); sh1 = scale_of(r_hi, kb + warps);
  }
  while (have0) {
    const uint4 cl0 = l0, ch0 = h0, cl1 = l1, ch1 = h1;
    const float csl0 = sl0, csh0 = sh0, csl1 = sl1, csh1 = sh1;
    const int kb0 = kb;
    const bool run1 = have1;
    kb += 2 * warps;
    have0 = kb < kblocks;
    have1 = kb + warps < kblocks;
    if (have0) {
      l0 = __ldg(reinterpret_cast<const uint4*>(w_lo + int64_t(kb) * 64));
      h0 = __ldg(reinterpret_cast<const uint4*>(w_hi + int64_t(kb) * 64));
      sl0 = scale_of(r_lo, kb); sh0 = scale_of(r_hi, kb);
    }
    if (have1) {
      l1 = __ldg(reinterpret_cast<const uint4*>(w_lo + int64_t(kb + warps) * 64));
      h1 = __ldg(reinterpret_cast<const uint4*>(w_hi + int64_t(kb + warps) * 64));
      sl1 = scale_of(r_lo, kb + warps); sh1 = scale_of(r_hi, kb + warps);
    }
    block(cl0, ch0, csl0, csh0, kb0);
    if (run1) block(cl1, ch1, csl1, csh1, kb0 + warps);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) red4[((warp * NT + nt) * 4 + i) * 32 + lane] = total[nt][i];
  __syncthreads();
  for (int o = threadIdx.x; o < NT * 128; o += blockDim.x) {
    const int nt = o >> 7, i = (o >> 5) & 3, ln = o & 31;
    float v = 0.f;
    for (int w = 0; w < warps; ++w) v += red4[((w * NT + nt) * 4 + i) * 32 + ln];
    const int64_t row = tile_row + (ln >> 2) + ((i & 2) ? 8 : 0);
    const int col = 8 * nt + 2 * (ln & 3) + (i & 1);
    if (row < p.n && col < p.m) {
      float sc = p.wscale;
      if (!GROUPED) sc *= tl_load_scale(p.scales, p.scales_dtype, row);
      const float r = tl_apply_epilogue(epi, v * sc, col, row, p.n);
      tl_store_out(p.out, p.out_dtype, int64_t(col) * p.n + row, r);
    }
  }
}

template <typename AT>
void launch_int4_mma(tl_ctx* ctx, const Int4Args& p, const EpiParams& e, bool grouped) {
  const int kblocks = p.k >> 7;
  int warps = kblocks >= 8 ? 8 : kblocks >= 4 ? 4 : kblocks >= 2 ? 2 : 1;  // 8 measured best or equal at m = 1, 8, 16
  // A/B hook: {TL_FAMILY_QGEMV, 9, warps} forces the CTA width
  if (ctx->has_forced && ctx->forced.family == TL_FAMILY_QGEMV && ctx->forced.kernel == 9 && ctx->forced.p0 >= 1 && ctx->forced.p0 <= 16 &&
      (ctx->forced.p0 & (ctx->forced.p0 - 1)) == 0)
    warps = ctx->forced.p0;
  const int grid = (p.n + 15) / 16, nt = p.m > 8 ? 2 : 1;
  const size_t smem = size_t(warps) * nt * 128 * sizeof(float);
  if (nt == 2) {
    if (grouped) qgemv_int4_mma_kernel<AT, 2, true><<<grid, warps * 32, smem, ctx->stream>>>(p, e);
    else qgemv_int4_mma_kernel<AT, 2, false><<<grid, warps * 32, smem, ctx->stream>>>(p, e);
  } else {
    if (grouped) qgemv_int4_mma_kernel<AT, 1, true><<<grid, warps * 32, smem, ctx->stream>>>(p, e);
    else qgemv_int4_mma_kernel<AT, 1, false><<<grid, warps * 32, smem, ctx->stream>>>(p, e);
  }
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
}

int32_t check_int4(tl_ctx* ctx, const char* who, const void* packed, const void* scales, int64_t n, int64_t k, const tl_quant_desc* q) {
  if (!packed || !scales) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: missing packing/scales on B operand", who);
  if (n < 0 || k < 0 || n > 0x7fffffffLL || k > 0x7fffffffLL) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: bad shape n=%lld k=%lld", who, (long long)n, (long long)k);
  if (k % 8 != 0) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: K=%lld must be divisible by 8 (eight int4 per word)", who, (long long)k);
  if (q->group_size <= 0 || q->group_size % 8 != 0 || (k > 0 && k % q->group_size != 0))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: K=%lld must be divisible by groupSize=%d, itself a multiple of 8", who, (long long)k, q->group_size);
  if (q->scales_dtype != TL_F16 && q->scales_dtype != TL_F32) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: scales dtype must be f16 or f32", who);
  if (q->scale_convention != TL_SCALE_SNORM127 && q->scale_convention != TL_SCALE_DIRECT)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: unknown scale convention %d", who, q->scale_convention);
  if ((reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(scales) & (tl_dtype_size(q->scales_dtype) - 1)))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: misaligned weight or scales pointer", who);
  return TL_OK;
}

}  // namespace

extern "C" {

int32_t tl_quantize_linear_weight_int4(const float* weight, int64_t n, int64_t k, int32_t group_size, uint32_t* packed, uint16_t* scales) {
  if (!weight || !packed || !scales) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize int4: null pointer");
  if (n < 0 || k < 0) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize int4: negative shape");
  if (k % 8 != 0) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize int4: K=%lld must be divisible by 8", (long long)k);
  if (group_size <= 0 || k % group_size != 0)
    return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize int4: K=%lld must be divisible by groupSize=%d", (long long)k, group_size);
  if (n == 0 || k == 0) return TL_OK;
  const unsigned hw = std::thread::hardware_concurrency();
  int64_t nthreads = std::max<int64_t>(1, std::min<int64_t>(hw ? hw : 1, (n * k) / (1 << 16)));
  nthreads = std::min<int64_t>(nthreads, n);
  if (nthreads <= 1) {
    quantize_rows_int4(weight, 0, n, k, group_size, packed, scales);
    return TL_OK;
  }
  std::vector<std::thread> pool;
  const int64_t per = (n + nthreads - 1) / nthreads;
  for (int64_t t = 0; t < nthreads; ++t) {
    const int64_t r0 = t * per, r1 = std::min(n, r0 + per);
    if (r0 >= r1) break;
    pool.emplace_back(quantize_rows_int4, weight, r0, r1, k, group_size, packed, scales);
  }
  for (auto& th : pool) th.join();
  return TL_OK;
}

int32_t tl_dequant_int4(tl_ctx* ctx, const void* packed, const void* scales, void* out, int32_t out_dtype, int64_t n, int64_t k,
                        const tl_quant_desc* qdesc) {
  TL_CHECK_CTX(ctx);
  if (!qdesc || qdesc->scheme != TL_SCHEME_INT4_GROUPED) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_dequant_int4: the descriptor's scheme must be int4-grouped");
  int32_t rc = check_int4(ctx, "tl_dequant_int4", packed, scales, n, k, qdesc);
  if (rc != TL_OK) return rc;
  if (!out || !tl_dtype_valid(out_dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_dequant_int4: null output or unknown dtype");
  ctx->counters[TL_COUNTER_DEQUANT]++;
  const int64_t n_words = n * (k / 8);
  if (n_words == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  const int grid = int(std::min<int64_t>((n_words + 255) / 256, int64_t(ctx->sm_count) * 16));
  const int32_t wpr = int32_t(k / 8), gpr = int32_t(k / qdesc->group_size);
  const uint32_t* pk = static_cast<const uint32_t*>(packed);
  if (out_dtype == TL_F32)
    dequant_int4_kernel<float><<<grid, 256, 0, ctx->stream>>>(pk, scales, static_cast<float*>(out), n_words, wpr, qdesc->group_size, gpr, qdesc->scales_dtype, qdesc->scale_convention);
  else if (out_dtype == TL_F16)
    dequant_int4_kernel<__half><<<grid, 256, 0, ctx->stream>>>(pk, scales, static_cast<__half*>(out), n_words, wpr, qdesc->group_size, gpr, qdesc->scales_dtype, qdesc->scale_convention);
  else
    dequant_int4_kernel<__nv_bfloat16><<<grid, 256, 0, ctx->stream>>>(pk, scales, static_cast<__nv_bfloat16*>(out), n_words, wpr, qdesc->group_size, gpr, qdesc->scales_dtype, qdesc->scale_convention);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_unpack_int4(tl_ctx* ctx, const void* packed, void* out_i8, int64_t n, int64_t k) {
  TL_CHECK_CTX(ctx);
  if (!packed || !out_i8 || n < 0 || k < 0 || k % 8 != 0 || (reinterpret_cast<uintptr_t>(out_i8) & 7))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_unpack_int4: null pointer, K %% 8 != 0 or an output not 8-byte aligned");
  const int64_t n_words = n * (k / 8);
  if (n_words == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  const int grid = int(std::min<int64_t>((n_words + 255) / 256, int64_t(ctx->sm_count) * 16));
  unpack_int4_kernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const uint32_t*>(packed), static_cast<int8_t*>(out_i8), n_words);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

}  // extern "C"

// The seam's int4 branch (tl_qmatmul_nt / tl_qgemv_nt / tl_qgemm_nt with an int4 descriptor).
// route: 0 by m, 1 GEMV only, 2 dequant + dense only.
int32_t tl_int4_matmul(tl_ctx* ctx, const char* who, int route, const void* a, int32_t a_dtype, const void* packed, const void* scales,
                       void* out, int32_t out_dtype, int64_t m, int64_t n, int64_t k, const tl_quant_desc* q, float alpha,
                       const tl_epilogue* epilogue, tl_plan_receipt* receipt_only) {
  int32_t rc = check_int4(ctx, who, receipt_only ? (const void*)16 : packed, receipt_only ? (const void*)16 : scales, n, k, q);
  if (rc != TL_OK) return rc;
  if (!tl_dtype_valid(a_dtype) || !tl_dtype_valid(out_dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: unknown dtype", who);
  if (m < 0) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: negative m", who);
  if (!receipt_only && ((m > 0 && !a) || !out)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: null activation or output", who);
  if (route == 1 && (m < 1 || m > 16)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: m=%lld outside the GEMV range [1,16]", who, (long long)m);
  EpiParams epi;
  bool has_ops = false;
  rc = tl_make_epi(ctx, epilogue, alpha, &epi, &has_ops);
  if (rc != TL_OK) return rc;
  const bool gemv = route == 1 || (route == 0 && m <= 16);
  // vector loads of the activations: 8 values per lane and step
  const bool a_aligned = receipt_only || (reinterpret_cast<uintptr_t>(a) & 15) == 0;
  if (receipt_only) {
    memset(receipt_only, 0, sizeof(*receipt_only));
    receipt_only->choice.family = gemv ? TL_FAMILY_QGEMV : TL_FAMILY_QGEMM;
    receipt_only->choice.kernel = gemv ? 9 : 2;  // "int4" / "dequant+dense"
    receipt_only->grid[0] = gemv ? int32_t((n + 15) / 16) : 0;
    receipt_only->block = gemv ? 256 : 0;
    receipt_only->split_k = 1;
    receipt_only->epilogue_engaged = has_ops ? 1 : 0;
    return TL_OK;
  }
  if (m == 0 || n == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  if (gemv) {
    if (!a_aligned) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: int4 GEMV needs 16-byte aligned activations", who);
    if ((size_t(k) * tl_dtype_size(a_dtype)) % 16 != 0) return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "%s: int4 GEMV needs activation rows of whole 16-byte vectors", who);
    Int4Args p{};
    p.a = a; p.packed = static_cast<const uint32_t*>(packed); p.scales = scales; p.out = out;
    p.n = int32_t(n); p.k = int32_t(k);
    p.group = q->group_size; p.groups_per_row = int32_t(k / q->group_size);
    p.scales_dtype = q->scales_dtype; p.out_dtype = out_dtype;
    p.wscale = q->scale_convention == TL_SCALE_SNORM127 ? 1.0f / 7.0f : 1.0f;
    // the tensor-core form when its layout conditions hold (and it is not switched off for A/B tests)
    const bool forced_simt = ctx->has_forced && ctx->forced.family == TL_FAMILY_QGEMV && ctx->forced.kernel == 1;
    const bool mma_ok = !forced_simt && a_dtype != TL_F32 && k % 128 == 0 && q->group_size % 128 == 0 &&
                        (reinterpret_cast<uintptr_t>(packed) & 15) == 0;
    p.m = int32_t(m); p.row0 = 0;
    if (mma_ok && a_dtype == TL_F16) launch_int4_mma<__half>(ctx, p, epi, q->group_size != k);
    else if (mma_ok) launch_int4_mma<__nv_bfloat16>(ctx, p, epi, q->group_size != k);
    else if (a_dtype == TL_F32) launch_int4_m<float>(ctx, p, epi, int(m));
    else if (a_dtype == TL_F16) launch_int4_m<__half>(ctx, p, epi, int(m));
    else launch_int4_m<__nv_bfloat16>(ctx, p, epi, int(m));
    TL_CUDA(ctx, cudaGetLastError());
    ctx->counters[TL_COUNTER_QGEMV]++;
    if (has_ops) ctx->counters[TL_COUNTER_QGEMV_EPILOGUE]++;
    return TL_OK;
  }
  // m > 16: dequantize [N, K] into scratch in the activation type, then the dense NT product
  void* wbuf = nullptr;
  rc = tl_ensure_scratch(ctx, size_t(n) * size_t(k) * tl_dtype_size(a_dtype) + (size_t(1) << 20), &wbuf);
  if (rc != TL_OK) return rc;
  // the dense kernel may want scratch of its own (operand transposition: not for NT) -- keep ours at the front
  rc = tl_dequant_int4(ctx, packed, scales, wbuf, a_dtype, n, k, q);
  if (rc != TL_OK) return rc;
  rc = tl_matmul(ctx, a, wbuf, out, m, n, k, 1, 0, 0, m * n, 0, 1, alpha, a_dtype, a_dtype, out_dtype, -1, -1, epilogue, nullptr);
  if (rc == TL_OK) ctx->counters[TL_COUNTER_QGEMM]++;
  return rc;
}
