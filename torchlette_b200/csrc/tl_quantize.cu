// Host quantizer (the library's own implementation of torchlette's
// quantizeLinearWeight) and the explicit dequantize / unpack kernels.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>

#include "tl_common.cuh"

// ---------------------------------------------------------------------------
// f32 <-> f16 bits, following src/backend/quantize.ts:22-60 including its
// subnormal branch (round half up on bit 12, sticky bits ignored).
// ---------------------------------------------------------------------------
static inline uint32_t host_f32_to_f16_bits(float value) {
  uint32_t x;
  std::memcpy(&x, &value, sizeof(x));
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t e = int32_t((x >> 23) & 0xffu) - 112;  // rebias 127 -> 15
  const uint32_t mant = x & 0x7fffffu;
  if (e <= 0) {
    if (e < -10) return sign;
    const uint32_t shifted = (mant | 0x800000u) >> (1 - e);
    return (sign | ((shifted >> 13) + ((shifted >> 12) & 1u))) & 0xffffu;
  }
  if (e >= 31) return sign | 0x7c00u;
  uint32_t h = sign | (uint32_t(e) << 10) | (mant >> 13);
  const uint32_t rest = mant & 0x1fffu;
  if (rest > 0x1000u || (rest == 0x1000u && (h & 1u))) ++h;
  return h & 0xffffu;
}

static inline double host_f16_bits_to_f64(uint32_t bits) {
  const bool neg = (bits & 0x8000u) != 0;
  const uint32_t e = (bits >> 10) & 0x1fu;
  const uint32_t frac = bits & 0x3ffu;
  double mag;
  if (e == 0) mag = std::ldexp(double(frac), -24);
  else if (e == 31) mag = frac == 0 ? INFINITY : NAN;
  else mag = std::ldexp(double(frac | 0x400u), int(e) - 25);
  return neg ? -mag : mag;
}

// JS Math.round: ties go toward +infinity.
static inline double round_half_up(double x) {
  const double f = std::floor(x);
  return (x - f >= 0.5) ? f + 1.0 : f;
}

static void quantize_rows(const float* weight, int64_t row0, int64_t row1, int64_t k, int32_t group,
                          uint32_t* packed, uint16_t* scales) {
  const int64_t groups = k / group;
  const int64_t words = k / 4;
  for (int64_t row = row0; row < row1; ++row) {
    const float* w = weight + row * k;
    uint8_t* bytes = reinterpret_cast<uint8_t*>(packed + row * words);  // little-endian lanes
    for (int64_t g = 0; g < groups; ++g) {
      const float* wg = w + g * group;
      float amax = 0.f;
      for (int32_t j = 0; j < group; ++j) amax = std::max(amax, std::fabs(wg[j]));
      const uint32_t sbits = host_f32_to_f16_bits(amax);
      scales[row * groups + g] = uint16_t(sbits);
      const double s = host_f16_bits_to_f64(sbits);
      const double inv = s > 0 ? 127.0 / s : 0.0;
      for (int32_t j = 0; j < group; ++j) {
        double q = round_half_up(double(wg[j]) * inv);
        // JS Math.min/Math.max propagate NaN and `NaN & 0xff` is 0 (quantize.ts:115-126)
        q = std::isnan(q) ? 0.0 : std::max(-127.0, std::min(127.0, q));
        bytes[g * group + j] = uint8_t(int8_t(int32_t(q)));
      }
    }
  }
}

extern "C" {

uint32_t tl_f32_to_f16_bits(float value) { return host_f32_to_f16_bits(value); }
float tl_f16_bits_to_f32(uint32_t bits) { return float(host_f16_bits_to_f64(bits)); }

int32_t tl_quantize_linear_weight(const float* weight, int64_t n, int64_t k, int32_t group_size,
                                  uint32_t* packed, uint16_t* scales) {
  if (!weight || !packed || !scales)
    return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize: null pointer");
  if (n < 0 || k < 0) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize: negative shape");
  if (k % 4 != 0) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize: K=%lld must be divisible by 4", (long long)k);
  if (group_size <= 0 || k % group_size != 0)
    return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "quantize: K=%lld must be divisible by groupSize=%d",
                        (long long)k, group_size);
  if (n == 0 || k == 0) return TL_OK;
  unsigned hw = std::thread::hardware_concurrency();
  int64_t nthreads = std::max<int64_t>(1, std::min<int64_t>(hw ? hw : 1, (n * k) / (1 << 16)));
  nthreads = std::min<int64_t>(nthreads, n);
  if (nthreads <= 1) {
    quantize_rows(weight, 0, n, k, group_size, packed, scales);
    return TL_OK;
  }
  std::vector<std::thread> pool;
  const int64_t per = (n + nthreads - 1) / nthreads;
  for (int64_t t = 0; t < nthreads; ++t) {
    const int64_t r0 = t * per, r1 = std::min(n, r0 + per);
    if (r0 >= r1) break;
    pool.emplace_back(quantize_rows, weight, r0, r1, k, group_size, packed, scales);
  }
  for (auto& th : pool) th.join();
  return TL_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Explicit dequantize: one thread per packed word (4 outputs), f64 arithmetic so
// the f32 result carries exactly one rounding, as the host dequantizer's does
// (src/backend/quantize.ts:152).
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void __launch_bounds__(256)
dequant_int8_kernel(const uint32_t* __restrict__ packed, const void* __restrict__ scales, OutT* __restrict__ out,
                    int64_t n_words, int32_t words_per_row, int32_t group, int32_t groups_per_row,
                    int32_t scales_dtype, int32_t convention) {
  __shared__ double lut[256];  // q/127 (snorm) or q (direct), indexed by the raw byte
  {
    const int b = threadIdx.x;
    const int q = b >= 128 ? b - 256 : b;
    lut[b] = convention == TL_SCALE_SNORM127 ? double(q) / 127.0 : double(q);
  }
  __syncthreads();
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t wi = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; wi < n_words; wi += stride) {
    const int64_t row = wi / words_per_row;
    const int32_t wcol = int32_t(wi - row * words_per_row);
    const uint32_t word = __ldg(packed + wi);
    const int32_t k0 = wcol * 4;
    float r[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      // a group may end inside a word only when group is not a multiple of 4
      const int64_t sidx = row * groups_per_row + (k0 + b) / group;
      const double s = double(tl_load_scale(scales, scales_dtype, sidx));
      r[b] = float(lut[(word >> (8 * b)) & 0xffu] * s);
    }
    OutT* o = out + wi * 4;
#pragma unroll
    for (int b = 0; b < 4; ++b) o[b] = DT<OutT>::from_f32(r[b]);
  }
}

__global__ void __launch_bounds__(256)
unpack_int8_kernel(const uint32_t* __restrict__ packed, uint32_t* __restrict__ out, int64_t n_words) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t wi = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; wi < n_words; wi += stride)
    out[wi] = __ldg(packed + wi);  // lane b of the word IS the int8 at k = 4*w + b (little-endian)
}

extern "C" {

int32_t tl_dequant_int8(tl_ctx* ctx, const void* packed, const void* scales, void* out, int32_t out_dtype,
                        int64_t n, int64_t k, const tl_quant_desc* qdesc) {
  TL_CHECK_CTX(ctx);
  int32_t rc = tl_check_qargs(ctx, "tl_dequant_int8", (const void*)16, TL_F32, packed, scales, out, out_dtype,
                              1, n, k, qdesc);
  if (rc != TL_OK) return rc;
  ctx->counters[TL_COUNTER_DEQUANT]++;
  const int64_t n_words = n * (k / 4);
  if (n_words == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  const int block = 256;
  const int64_t want = (n_words + block - 1) / block;
  const int grid = int(std::min<int64_t>(want, int64_t(ctx->sm_count) * 16));
  const int32_t wpr = int32_t(k / 4), gpr = int32_t(k / qdesc->group_size);
  const uint32_t* pk = reinterpret_cast<const uint32_t*>(packed);
  if (out_dtype == TL_F32)
    dequant_int8_kernel<float><<<grid, block, 0, ctx->stream>>>(pk, scales, (float*)out, n_words, wpr,
        qdesc->group_size, gpr, qdesc->scales_dtype, qdesc->scale_convention);
  else if (out_dtype == TL_F16)
    dequant_int8_kernel<__half><<<grid, block, 0, ctx->stream>>>(pk, scales, (__half*)out, n_words, wpr,
        qdesc->group_size, gpr, qdesc->scales_dtype, qdesc->scale_convention);
  else
    dequant_int8_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(pk, scales, (__nv_bfloat16*)out,
        n_words, wpr, qdesc->group_size, gpr, qdesc->scales_dtype, qdesc->scale_convention);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_unpack_int8(tl_ctx* ctx, const void* packed, void* out_i8, int64_t n, int64_t k) {
  TL_CHECK_CTX(ctx);
  if (!packed || !out_i8) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_unpack_int8: null pointer");
  if (n < 0 || k < 0 || k % 4 != 0)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_unpack_int8: K=%lld must be divisible by 4", (long long)k);
  if ((reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(out_i8) & 3))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_unpack_int8: pointers must be 4-byte aligned");
  const int64_t n_words = n * (k / 4);
  if (n_words == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  const int block = 256;
  const int grid = int(std::min<int64_t>((n_words + block - 1) / block, int64_t(ctx->sm_count) * 16));
  unpack_int8_kernel<<<grid, block, 0, ctx->stream>>>((const uint32_t*)packed, (uint32_t*)out_i8, n_words);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Device-side quantizeLinearWeight (src/backend/quantize.ts:77-131): the weight
// stays on the GPU, one warp per (row, group).  Same arithmetic as the host
// quantizer, step by step: group abs-max in f32 with NaN skipped (`a > absMax`),
// the f16 scale bits through the reference's converter (half-up subnormal
// branch included), 127 / scale and weight * inv in f64, Math.round as
// floor-and-compare, clamp with NaN -> 0, two's-complement byte lanes.  The
// packed words and scale bits are bit-identical to the host's.
// ---------------------------------------------------------------------------
namespace {
__device__ __forceinline__ uint32_t dev_f32_to_f16_bits(float value) {
  const uint32_t x = __float_as_uint(value);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t e = int32_t((x >> 23) & 0xffu) - 112;
  const uint32_t mant = x & 0x7fffffu;
  if (e <= 0) {
    if (e < -10) return sign;
    const uint32_t shifted = (mant | 0x800000u) >> (1 - e);
    return (sign | ((shifted >> 13) + ((shifted >> 12) & 1u))) & 0xffffu;
  }
  if (e >= 31) return sign | 0x7c00u;
  uint32_t h = sign | (uint32_t(e) << 10) | (mant >> 13);
  const uint32_t rest = mant & 0x1fffu;
  if (rest > 0x1000u || (rest == 0x1000u && (h & 1u))) ++h;
  return h & 0xffffu;
}
__device__ __forceinline__ double dev_f16_bits_to_f64(uint32_t bits) {
  const uint32_t e = (bits >> 10) & 0x1fu, frac = bits & 0x3ffu;
  double mag;
  if (e == 0) mag = ldexp(double(frac), -24);
  else if (e == 31) mag = frac == 0 ? double(INFINITY) : double(NAN);
  else mag = ldexp(double(frac | 0x400u), int(e) - 25);
  return (bits & 0x8000u) ? -mag : mag;
}

__global__ void __launch_bounds__(256) quantize_kernel(const float* __restrict__ weight, int64_t n_groups, int32_t group,
                                                       uint32_t* __restrict__ packed, uint16_t* __restrict__ scales) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
  const int words = group >> 2;  // group % 4 == 0: a packed word never straddles two groups
  for (int64_t g = warp0; g < n_groups; g += nwarps) {
    const float4* src = reinterpret_cast<const float4*>(weight + g * group);  // rows are k floats, groups contiguous in k
    float amax = 0.f;
    for (int w = lane; w < words; w += 32) {
      const float4 v = __ldg(src + w);
      const float a0 = fabsf(v.x), a1 = fabsf(v.y), a2 = fabsf(v.z), a3 = fabsf(v.w);
      if (a0 > amax) amax = a0;  // a NaN never compares greater: skipped, as in the reference
      if (a1 > amax) amax = a1;
      if (a2 > amax) amax = a2;
      if (a3 > amax) amax = a3;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, amax, o);
      if (other > amax) amax = other;
    }
    const uint32_t sbits = dev_f32_to_f16_bits(amax);
    if (lane == 0) scales[g] = uint16_t(sbits);
    const double sc = dev_f16_bits_to_f64(sbits);
    const double inv = sc > 0 ? 127.0 / sc : 0.0;
    uint32_t* dst = packed + g * words;
    for (int w = lane; w < words; w += 32) {
      const float4 v = __ldg(src + w);
      const float f[4] = {v.x, v.y, v.z, v.w};
      uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const double x = double(f[b]) * inv;
        const double fl = floor(x);
        double q = (x - fl >= 0.5) ? fl + 1.0 : fl;  // Math.round: ties toward +infinity
        q = (q != q) ? 0.0 : fmax(-127.0, fmin(127.0, q));  // NaN packs 0 (`NaN & 0xff`)
        word |= (uint32_t(int32_t(q)) & 0xffu) << (8 * b);
      }
      dst[w] = word;
    }
  }
}
}  // namespace

extern "C" int32_t tl_quantize_linear_weight_device(tl_ctx* ctx, const float* weight, int64_t n, int64_t k, int32_t group_size,
                                                    uint32_t* packed, uint16_t* scales) {
  TL_CHECK_CTX(ctx);
  if (!weight || !packed || !scales) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "quantize (device): null pointer");
  if (n < 0 || k < 0) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "quantize (device): negative shape");
  if (k % 4 != 0) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "quantize: K=%lld must be divisible by 4", (long long)k);
  if (group_size <= 0 || k % group_size != 0)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "quantize: K=%lld must be divisible by groupSize=%d", (long long)k, group_size);
  if (group_size % 4 != 0)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "quantize (device): groupSize=%d must be a multiple of 4 (use the host quantizer)", group_size);
  if ((reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(scales) & 1))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "quantize (device): weight must be 16-byte aligned, packed 4, scales 2");
  if (n == 0 || k == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  const int64_t n_groups = n * (k / group_size);
  const int block = 256;
  const int64_t want = (n_groups + 7) / 8;  // 8 warps per CTA, one group per warp and pass
  const int grid = int(std::min<int64_t>(want, int64_t(ctx->sm_count) * 32));
  quantize_kernel<<<grid, block, 0, ctx->stream>>>(weight, n_groups, group_size, packed, scales);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}
