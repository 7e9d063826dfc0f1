// The ops either side of the projections in one Qwen3 decode step, so that a step can run on this
// backend end to end (packages/qwen3-browser/src/model.ts:220-420): RMSNorm (hidden-wide and the
// per-head q / k norm), rotary embedding, and single-token attention over a KV cache with grouped
// query heads.  (The residual adds, silu(gate) * up and the cache append are tl_binary_op, the
// multiply epilogue and tl_copy2d.)  All HBM-bound and small next to the projections: one pass each,
// f32 arithmetic, any of f32 / f16 / bf16 storage.
//
//   rmsnorm    y = x * rsqrt(mean(x^2) + eps) * w            src/ops/semantic/composite.ts:156-170
//   rope       half-split (GPT-NeoX / Llama) rotation         src/backend/webgpu/rope-kernel.ts:1-93
//   attention  softmax(q k^T * scale + mask) v over a KV cache   model.ts:284-318 (decode, S = 1; and the causal
//              form for several query positions, prefill or multi-token with a cache)
#include <algorithm>
#include <cfloat>

#include "tl_common.cuh"

namespace {

__device__ __forceinline__ float ld_f32(const void* p, int dtype, int64_t i) {
  if (dtype == TL_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == TL_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// one CTA per row (cols up to any size), 128 threads
__global__ void __launch_bounds__(128) rmsnorm_kernel(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                                                      int64_t rows, int cols, float eps) {
  __shared__ float part[4];
  const int64_t row = blockIdx.x;
  if (row >= rows) return;
  const int64_t base = row * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 128) {
    const float v = ld_f32(x, x_dtype, base + c);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float total = part[0] + part[1] + part[2] + part[3];
  const float inv = rsqrtf(total / float(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += 128) {
    const float v = ld_f32(x, x_dtype, base + c);
    tl_store_out(out, out_dtype, base + c, v * inv * ld_f32(w, w_dtype, c));
  }
}

// one thread per output element of qk [outer, S, D]
__global__ void __launch_bounds__(256) rope_kernel(const void* qk, int dtype, const float* cos_t, const float* sin_t, void* out,
                                                   int64_t total, int seq_len, int head_dim, float sin_scale, int64_t cos_offset,
                                                   int64_t sin_offset) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int half = head_dim >> 1;
  for (int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int d = int(idx % head_dim);
    const int s = int((idx / head_dim) % seq_len);
    const bool second = d >= half;
    const int dh = second ? d - half : d;
    const float qi = ld_f32(qk, dtype, idx), qp = ld_f32(qk, dtype, second ? idx - half : idx + half);
    const float c = cos_t[cos_offset + int64_t(s) * half + dh];
    const float sn = sin_t[sin_offset + int64_t(s) * half + dh] * sin_scale;
    tl_store_out(out, dtype, idx, qi * c + (second ? 1.f : -1.f) * qp * sn);
  }
}

// one CTA per (batch, query head, query position); 4 warps; scores for the visible positions live in
// shared memory.  q is [B, H, S, D]; the output is written as [B, S, H, D] (the permute that o_proj's
// input needs, model.ts:314-318, folded into the store).  With `causal`, query s sees the keys up to
// position kv_len - q_len + s (the mask the reference builds with triu, model.ts:300-307).
__global__ void __launch_bounds__(128) attention_kernel(const void* q, const void* kc, const void* vc, void* out, int dtype,
                                                        int n_heads, int n_kv_heads, int q_len, int head_dim, int kv_len_total,
                                                        int64_t kv_capacity, float scale, const float* mask, int causal) {
  extern __shared__ float scores[];  // [kv_len]
  __shared__ float red[4];
  const int sq = blockIdx.x % q_len;
  const int bh = blockIdx.x / q_len;
  const int b = bh / n_heads, h = bh - b * n_heads;
  const int kvh = h / (n_heads / n_kv_heads);  // repeat_kv order: head h reads kv head h / n_rep
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = causal ? kv_len_total - q_len + sq + 1 : kv_len_total;
  const int64_t q_base = ((int64_t(b) * n_heads + h) * q_len + sq) * head_dim;
  const int64_t o_base = ((int64_t(b) * q_len + sq) * n_heads + h) * head_dim;
  const int64_t kv_base = (int64_t(b) * n_kv_heads + kvh) * kv_capacity * head_dim;
  // scores: a warp per key position, lanes over the head dimension
  float wmax = -FLT_MAX;
  for (int j = warp; j < kv_len; j += 4) {
    float dot = 0.f;
    for (int d = lane; d < head_dim; d += 32) dot = fmaf(ld_f32(q, dtype, q_base + d), ld_f32(kc, dtype, kv_base + int64_t(j) * head_dim + d), dot);
    dot = warp_sum(dot) * scale + (mask ? mask[int64_t(sq) * kv_len_total + j] : 0.f);
    if (lane == 0) scores[j] = dot;
    wmax = fmaxf(wmax, dot);
  }
  if (lane == 0) red[warp] = wmax;
  __syncthreads();
  const float mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float sum = 0.f;
  for (int j = threadIdx.x; j < kv_len; j += 128) {
    const float e = expf(scores[j] - mx);
    scores[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  const float inv = 1.f / (red[0] + red[1] + red[2] + red[3]);
  // output: thread d accumulates over all positions (coalesced over d for every position)
  for (int d = threadIdx.x; d < head_dim; d += 128) {
    float acc = 0.f;
    for (int j = 0; j < kv_len; ++j) acc = fmaf(scores[j], ld_f32(vc, dtype, kv_base + int64_t(j) * head_dim + d), acc);
    tl_store_out(out, dtype, o_base + d, acc * inv);
  }
}

}  // namespace

extern "C" {

int32_t tl_rmsnorm(tl_ctx* ctx, const void* x, int32_t x_dtype, const void* weight, int32_t weight_dtype, void* out, int32_t out_dtype,
                   int64_t rows, int64_t cols, float eps) {
  TL_CHECK_CTX(ctx);
  if (rows < 0 || cols < 1 || cols > INT32_MAX || (rows > 0 && (!x || !weight || !out)))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_rmsnorm: null pointer or bad shape");
  if (!tl_dtype_valid(x_dtype) || !tl_dtype_valid(weight_dtype) || !tl_dtype_valid(out_dtype))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_rmsnorm: unknown dtype");
  if (rows == 0) return TL_OK;
  if (rows > INT32_MAX) return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_rmsnorm: too many rows for one launch");
  DeviceGuard guard(ctx->device);
  rmsnorm_kernel<<<unsigned(rows), 128, 0, ctx->stream>>>(x, x_dtype, weight, weight_dtype, out, out_dtype, rows, int(cols), eps);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_rope(tl_ctx* ctx, const void* qk, int32_t dtype, const float* cos_table, const float* sin_table, void* out, int64_t outer,
                int64_t seq_len, int64_t head_dim, float sin_scale, int64_t cos_offset, int64_t sin_offset) {
  TL_CHECK_CTX(ctx);
  if (outer < 0 || seq_len < 1 || head_dim < 2 || seq_len > INT32_MAX || head_dim > INT32_MAX || cos_offset < 0 || sin_offset < 0)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_rope: bad shape");
  if (head_dim % 2 != 0) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "applyRoPE: headDim must be even, got %lld", (long long)head_dim);
  if (!tl_dtype_valid(dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_rope: unknown dtype");
  const int64_t total = outer * seq_len * head_dim;
  if (total == 0) return TL_OK;
  if (!qk || !cos_table || !sin_table || !out || qk == out)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_rope: null or aliased pointers (an element reads its partner: not in place)");
  DeviceGuard guard(ctx->device);
  const int grid = int(std::min<int64_t>((total + 255) / 256, int64_t(ctx->sm_count) * 8));
  rope_kernel<<<grid, 256, 0, ctx->stream>>>(qk, dtype, cos_table, sin_table, out, total, int(seq_len), int(head_dim), sin_scale, cos_offset,
                                             sin_offset);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_attention(tl_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, void* out, int32_t dtype, int64_t batch,
                     int64_t n_heads, int64_t n_kv_heads, int64_t q_len, int64_t head_dim, int64_t kv_len, int64_t kv_capacity, float scale,
                     const float* mask, int32_t causal) {
  TL_CHECK_CTX(ctx);
  if (batch < 0 || n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || head_dim < 1 || q_len < 1 || kv_len < q_len ||
      kv_capacity < kv_len)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG,
                        "tl_attention: bad shape (heads %lld, kv heads %lld, q_len %lld, kv_len %lld, capacity %lld)", (long long)n_heads,
                        (long long)n_kv_heads, (long long)q_len, (long long)kv_len, (long long)kv_capacity);
  if (!tl_dtype_valid(dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_attention: unknown dtype");
  if (batch == 0) return TL_OK;
  if (!q || !k_cache || !v_cache || !out) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_attention: null pointer");
  const size_t smem = size_t(kv_len) * sizeof(float);
  if (smem > 200 * 1024 || batch * n_heads * q_len > INT32_MAX || head_dim > 1024)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_attention: kv_len %lld exceeds the %d positions one launch keeps in shared memory",
                        (long long)kv_len, 200 * 1024 / 4);
  DeviceGuard guard(ctx->device);
  if (smem > 48 * 1024) cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  attention_kernel<<<unsigned(batch * n_heads * q_len), 128, smem, ctx->stream>>>(q, k_cache, v_cache, out, dtype, int(n_heads), int(n_kv_heads),
                                                                                  int(q_len), int(head_dim), int(kv_len), kv_capacity, scale, mask,
                                                                                  causal ? 1 : 0);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_decode_attention(tl_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, void* out, int32_t dtype, int64_t batch,
                            int64_t n_heads, int64_t n_kv_heads, int64_t head_dim, int64_t kv_len, int64_t kv_capacity, float scale,
                            const float* mask) {
  return tl_attention(ctx, q, k_cache, v_cache, out, dtype, batch, n_heads, n_kv_heads, 1, head_dim, kv_len, kv_capacity, scale, mask, 0);
}

}  // extern "C"
