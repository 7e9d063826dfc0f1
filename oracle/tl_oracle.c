/*
 * CPU oracle for the quantized-weight matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * torchlette's own CPU code for the path; it is the checker the GPU kernels are
 * compared with and the timed CPU baseline.  Nothing in the shipped library
 * links, loads or calls it.
 *
 * PARITY UNPINNED: the reference holds no golden vectors or known-answer values
 * for this path (its specs are same-input cross-path differentials) and the
 * TypeScript reference cannot be executed where this was written (no node).
 * The restatement is therefore pinned only procedurally: against IEEE facts
 * (numpy float16), against an independent numpy restatement, and against the
 * seeds / shapes / tolerances of the reference's own probes.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the torchlette repository root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* f32 <-> f16 bit converters: src/backend/quantize.ts:22-60                 */
/* ------------------------------------------------------------------------- */

/* src/backend/quantize.ts:22-47.  Normal range rounds to nearest even
 * (:39-46); the subnormal branch rounds half-up on bit 12 of the shifted
 * mantissa and ignores the sticky bits below (:30-37); exp < -10 flushes to a
 * signed zero (:32); exp >= 31 (inf, NaN and overflow alike) returns signed
 * infinity (:38). */
ORC_API uint32_t orc_f32_to_f16_bits(float val) {
  uint32_t x;
  memcpy(&x, &val, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xffu) - 127 + 15;
  uint32_t mant = x & 0x7fffffu;
  if (exp <= 0) {
    if (exp < -10) return sign;
    uint32_t m = (mant | 0x800000u) >> (1 - exp);
    uint32_t round = (m & 0x1000u) != 0 ? 1u : 0u;
    return (sign | ((m >> 13) + round)) & 0xffffu;
  }
  if (exp >= 0x1f) return sign | 0x7c00u;
  uint32_t half_mant = mant >> 13;
  uint32_t remainder = mant & 0x1fffu;
  uint32_t out = sign | ((uint32_t)exp << 10) | half_mant;
  if (remainder > 0x1000u || (remainder == 0x1000u && (half_mant & 1u) == 1u)) {
    out += 1;
  }
  return out & 0xffffu;
}

/* src/backend/quantize.ts:50-60.  Returned as double: the reference returns a
 * JS number; every f16 value is exactly representable in f32 and f64. */
ORC_API double orc_f16_bits_to_f64(uint32_t bits) {
  uint32_t sign = (bits >> 15) & 0x1u;
  uint32_t exp = (bits >> 10) & 0x1fu;
  uint32_t frac = bits & 0x3ffu;
  if (exp == 0) {
    if (frac == 0) return sign ? -0.0 : 0.0;
    return (sign ? -1.0 : 1.0) * ldexp(1.0, -14) * ((double)frac / 1024.0);
  }
  if (exp == 31) {
    if (frac == 0) return sign ? -INFINITY : INFINITY;
    return NAN;
  }
  return (sign ? -1.0 : 1.0) * ldexp(1.0, (int)exp - 15) * (1.0 + (double)frac / 1024.0);
}

ORC_API float orc_f16_bits_to_f32(uint32_t bits) { return (float)orc_f16_bits_to_f64(bits); }

/* JS Math.round: nearest integer, ties toward +infinity. */
static double js_math_round(double x) {
  if (isnan(x) || isinf(x)) return x;
  double r = floor(x);
  if (x - r >= 0.5) r += 1.0;
  return r;
}

/* ------------------------------------------------------------------------- */
/* Host quantizer: src/backend/quantize.ts:77-131                             */
/* ------------------------------------------------------------------------- */

/* weight [n,k] f32 row-major -> packed u32 [n,k/4] (byte lane = k&3, lowest k
 * in bits 0-7, two's complement) + scales u16 [n,k/G] holding the f16 bits of
 * the group abs-max.  Returns 0, or -1 for the argument errors the reference
 * throws on (:88-93). */
ORC_API int orc_quantize_linear_weight(const float* weight, int64_t n, int64_t k, int64_t group,
                                       uint32_t* packed, uint16_t* scales) {
  if (k % 4 != 0 || group <= 0 || k % group != 0) return -1;
  int64_t groups_per_row = k / group;
  int64_t words_per_row = k / 4;
  memset(packed, 0, (size_t)(n * words_per_row) * sizeof(uint32_t));
  for (int64_t row = 0; row < n; row++) {
    int64_t row_base = row * k;
    for (int64_t g = 0; g < groups_per_row; g++) {
      double abs_max = 0.0;
      int64_t g_base = row_base + g * group;
      for (int64_t j = 0; j < group; j++) {
        double a = fabs((double)weight[g_base + j]);
        if (a > abs_max) abs_max = a;
      }
      /* f32ToF16Bits stores val into a Float32Array first (:25); abs_max is an
       * f32 value already so that store is exact. */
      uint32_t scale_bits = orc_f32_to_f16_bits((float)abs_max);
      scales[row * groups_per_row + g] = (uint16_t)scale_bits;
      double scale = orc_f16_bits_to_f64(scale_bits);
      double inv = scale > 0 ? 127.0 / scale : 0.0;
      for (int64_t j = 0; j < group; j++) {
        double r = js_math_round((double)weight[g_base + j] * inv);
        /* Math.min / Math.max propagate NaN (C's fmin / fmax would drop it), and `NaN & 0xff`
         * is 0 (:121-126): a NaN weight, or Inf * 0 under an infinite group scale, packs 0. */
        double q = isnan(r) ? 0.0 : fmax(-127.0, fmin(127.0, r));
        int32_t qi = (int32_t)q;
        int64_t k_idx = g * group + j;
        int64_t word = row * words_per_row + (k_idx >> 2);
        int byte = (int)(k_idx & 3);
        packed[word] |= ((uint32_t)qi & 0xffu) << (byte * 8);
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* int4-grouped: the planned second scheme (docs/quantization-design.md:69-75)  */
/* ------------------------------------------------------------------------- */

/* The reference only DESCRIBES this scheme: "8 int4 per u32 word, packed 8-along-K into [N, K/8]
 * u32 ... unpacks a nibble ((word >> (4*j)) & 0xF, sign-extend from 4 bits)".  It holds no code and
 * no vectors for it, so this restatement follows the int8 quantizer above line for line with the
 * range [-7, 7] in place of [-127, 127] (symmetric, -8 never emitted) and nibble j = k & 7 in bits
 * 4j..4j+3; scales are the f16 bits of the group abs-max and w = (q / 7) * scale.  Parity for
 * int4 is therefore pinned to nothing but this text. */
ORC_API int orc_quantize_linear_weight_int4(const float* weight, int64_t n, int64_t k, int64_t group,
                                            uint32_t* packed, uint16_t* scales) {
  if (k % 8 != 0 || group <= 0 || k % group != 0) return -1;
  int64_t groups_per_row = k / group;
  int64_t words_per_row = k / 8;
  memset(packed, 0, (size_t)(n * words_per_row) * sizeof(uint32_t));
  for (int64_t row = 0; row < n; row++) {
    for (int64_t g = 0; g < groups_per_row; g++) {
      double abs_max = 0.0;
      int64_t g_base = row * k + g * group;
      for (int64_t j = 0; j < group; j++) {
        double a = fabs((double)weight[g_base + j]);
        if (a > abs_max) abs_max = a;
      }
      uint32_t scale_bits = orc_f32_to_f16_bits((float)abs_max);
      scales[row * groups_per_row + g] = (uint16_t)scale_bits;
      double scale = orc_f16_bits_to_f64(scale_bits);
      double inv = scale > 0 ? 7.0 / scale : 0.0;
      for (int64_t j = 0; j < group; j++) {
        double r = js_math_round((double)weight[g_base + j] * inv);
        double q = isnan(r) ? 0.0 : fmax(-7.0, fmin(7.0, r));
        int32_t qi = (int32_t)q;
        int64_t k_idx = g * group + j;
        packed[row * words_per_row + (k_idx >> 3)] |= ((uint32_t)qi & 0xfu) << ((k_idx & 7) * 4);
      }
    }
  }
  return 0;
}

static inline int32_t unpack_nibble(uint32_t word, int j) {
  int32_t qi = (int32_t)((word >> (j * 4)) & 0xfu);
  if (qi >= 8) qi -= 16;
  return qi;
}

/* signed nibbles as int8 [n,k] */
ORC_API void orc_unpack_int4(const uint32_t* packed, int64_t n, int64_t k, int8_t* out) {
  for (int64_t i = 0; i < n * k; i++) out[i] = (int8_t)unpack_nibble(packed[i >> 3], (int)(i & 7));
}

/* out[n,k] = (q / 7) * f16(scale[n, k / G]) in f64, one rounding to f32 (the int8 dequantizer's form) */
ORC_API void orc_dequantize_int4_to_f32(const uint32_t* packed, const uint16_t* scales, int64_t n, int64_t k,
                                        int64_t group, float* out) {
  int64_t groups_per_row = k / group;
  for (int64_t row = 0; row < n; row++)
    for (int64_t c = 0; c < k; c++) {
      int64_t e = row * k + c;
      double scale = orc_f16_bits_to_f64(scales[row * groups_per_row + c / group]);
      out[e] = (float)(((double)unpack_nibble(packed[e >> 3], (int)(e & 7)) / 7.0) * scale);
    }
}

/* ------------------------------------------------------------------------- */
/* Host dequantizer: src/backend/quantize.ts:138-156                          */
/* ------------------------------------------------------------------------- */

static inline int32_t unpack_lane(uint32_t word, int byte) {
  int32_t qi = (int32_t)((word >> (byte * 8)) & 0xffu);
  if (qi >= 128) qi -= 256;
  return qi;
}

/* Signed byte lanes of the packed words, one int8 per logical [n,k] element
 * (the integer half of quantize.ts:145-149). */
ORC_API void orc_unpack_int8(const uint32_t* packed, int64_t n, int64_t k, int8_t* out) {
  int64_t words_per_row = k / 4;
  for (int64_t row = 0; row < n; row++)
    for (int64_t k_idx = 0; k_idx < k; k_idx++)
      out[row * k + k_idx] = (int8_t)unpack_lane(packed[row * words_per_row + (k_idx >> 2)], (int)(k_idx & 3));
}

/* Reference-native convention: out = f32( (qi/127) * f16(scale) ), evaluated
 * in f64 with one rounding to f32 at the store (quantize.ts:152).  -128 is not
 * clamped. */
ORC_API void orc_dequantize_to_f32(const uint32_t* packed, const uint16_t* scales, int64_t n,
                                   int64_t k, int64_t group, float* out) {
  int64_t groups_per_row = k / group;
  int64_t words_per_row = k / 4;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < n; row++) {
    for (int64_t k_idx = 0; k_idx < k; k_idx++) {
      int32_t qi = unpack_lane(packed[row * words_per_row + (k_idx >> 2)], (int)(k_idx & 3));
      int64_t g = k_idx / group;
      double scale = orc_f16_bits_to_f64(scales[row * groups_per_row + g]);
      out[row * k + k_idx] = (float)(((double)qi / 127.0) * scale);
    }
  }
}

/* "Direct" convention of the benchmark configurations (per-output-channel or
 * per-group f32 scales, w = q*s): the exact product rounded once to f32.  It
 * has no counterpart in quantize.ts; the layout and lane order are the same
 * as above. */
ORC_API void orc_dequantize_direct_f32(const uint32_t* packed, const float* scales, int64_t n,
                                       int64_t k, int64_t group, float* out) {
  int64_t groups_per_row = k / group;
  int64_t words_per_row = k / 4;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < n; row++) {
    for (int64_t k_idx = 0; k_idx < k; k_idx++) {
      int32_t qi = unpack_lane(packed[row * words_per_row + (k_idx >> 2)], (int)(k_idx & 3));
      double s = (double)scales[row * groups_per_row + k_idx / group];
      out[row * k + k_idx] = (float)((double)qi * s);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* CPU matmul: src/backend/cpu/numeric.ts:510-595                             */
/* ------------------------------------------------------------------------- */

/* out[row,col] = f32( sum_k a[row,k] * w[col,k] ), k ascending, accumulated in
 * f64 (JS number), one rounding at the Float32Array store (:573-579).  `w` is
 * the [N,K] weight; the reference multiplies by its [K,N] transposed view,
 * which reads the same elements in the same order.  `threads` > 1 parallelises
 * over output columns only; every dot product stays sequential in k, so the
 * result does not depend on the thread count. */
ORC_API void orc_matmul_nt(const float* a, const float* w, float* out, int64_t m, int64_t n,
                           int64_t k, int threads) {
#ifdef _OPENMP
  if (threads < 1) threads = omp_get_max_threads();
#pragma omp parallel for schedule(static) num_threads(threads)
#endif
  for (int64_t col = 0; col < n; col++) {
    const float* wr = w + col * k;
    for (int64_t row = 0; row < m; row++) {
      const float* ar = a + row * k;
      double acc = 0.0;
      for (int64_t inner = 0; inner < k; inner++) acc += (double)ar[inner] * (double)wr[inner];
      out[row * n + col] = (float)acc;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Elementwise bodies: src/ops/semantic/{catalog,composite,erf,interpret}.ts  */
/* ------------------------------------------------------------------------- */

/* src/ops/semantic/erf.ts:28-56 (Abramowitz-Stegun 7.1.26, same Horner order). */
static double erf_approx(double v) {
  static const double A[5] = {0.254829592, -0.284496736, 1.421413741, -1.453152027, 1.061405429};
  const double P = 0.3275911;
  double sign = v < 0 ? -1.0 : 1.0;
  double ax = fabs(v);
  double t = 1.0 / (1.0 + P * ax);
  double poly = ((((A[4] * t + A[3]) * t + A[2]) * t + A[1]) * t + A[0]) * t;
  return sign * (1.0 - poly * exp(-ax * ax));
}

enum { ORC_RELU = 1, ORC_SILU = 2, ORC_SIGMOID = 3, ORC_TANH = 4, ORC_GELU_TANH = 5, ORC_GELU_ERF = 6 };

/* f64 evaluation of the single-source terms (interpret.ts:25-98):
 *   relu      where(gt(x,0), x, 0)                         catalog.ts:103-109
 *   silu      div(x, add(1, exp(neg(x))))                  catalog.ts:87-93
 *   sigmoid   recip(add(1, exp(neg(x))))                   catalog.ts:80-86
 *   gelu      mul(mul(.5,x), add(1, tanh(mul(c, add(x, mul(c3, x*(x*x)))))))  composite.ts:40-51
 *   gelu_erf  mul(mul(.5,x), add(1, erf(mul(x, SQRT1_2)))) composite.ts:60-65 */
ORC_API double orc_unary_f64(int op, double x) {
  switch (op) {
    case ORC_RELU: return x > 0.0 ? x : 0.0;
    case ORC_SILU: return x / (1.0 + exp(-x));
    case ORC_SIGMOID: return 1.0 / (1.0 + exp(-x));
    case ORC_TANH: return tanh(x);
    case ORC_GELU_TANH:
      return (0.5 * x) * (1.0 + tanh(0.7978845608 * (x + 0.044715 * (x * (x * x)))));
    case ORC_GELU_ERF: return (0.5 * x) * (1.0 + erf_approx(x * 0.7071067811865476));
    default: return x;
  }
}

/* applyUnaryOp (numeric.ts:436-447): read f32, evaluate in f64, store f32. */
ORC_API void orc_unary(int op, const float* x, float* out, int64_t count) {
  for (int64_t i = 0; i < count; i++) out[i] = (float)orc_unary_f64(op, (double)x[i]);
}

/* applyBinaryOp add with a [n] second operand broadcast over rows
 * (numeric.ts:448-466, 494-496): f64 add, f32 store. */
ORC_API void orc_add_bias(const float* x, const float* bias, float* out, int64_t m, int64_t n) {
  for (int64_t r = 0; r < m; r++)
    for (int64_t c = 0; c < n; c++) out[r * n + c] = (float)((double)x[r * n + c] + (double)bias[c]);
}

/* ------------------------------------------------------------------------- */
/* Probe input generator: examples/qwen3/probe-quant-gemv.ts:44-50            */
/* ------------------------------------------------------------------------- */

/* s = (s*1664525 + 1013904223) mod 2^32 ; value = s/2^31 - 1, stored to f32
 * scaled by `mul` in f64 first (probe-quant-operand.ts:67-69 uses rng()*0.1).
 * Returns the advanced state so one stream can fill several arrays. */
ORC_API uint32_t orc_lcg_fill(uint32_t state, double mul, float* out, int64_t count) {
  uint32_t s = state;
  for (int64_t i = 0; i < count; i++) {
    s = (uint32_t)(((uint64_t)s * 1664525ull + 1013904223ull) & 0xffffffffull);
    out[i] = (float)(((double)s / 2147483648.0 - 1.0) * mul);
  }
  return s;
}

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
