// The companion ops either side of the matmul seam: the UNFUSED forms of what the epilogue
// fuses (bias / residual add, activations, cast) and the materialization of a transposed
// view.  They are the "control" side of the reference's fused-vs-unfused comparisons
// (test/webgpu/matmul-epilogue.spec.ts:77-100, examples/qwen3/probe-gemv.ts:170-235) and the
// ops matmulQuantizedB composes on its explicit-dequant path
// (src/backend/webgpu/ops/matmul-ops.ts:163-181: dequant -> contiguous -> matmul -> cast).
// HBM-bound, one pass: grid-stride loops, 16-byte accesses where the types and alignment allow.
#include "tl_common.cuh"

namespace {

__device__ __forceinline__ float ld_as_f32(const void* p, int dtype, int64_t i) {
  if (dtype == TL_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == TL_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// out[i] = op(in[i]) with a cast on either side; op 0 is the plain cast / copy
__global__ void __launch_bounds__(256) unary_kernel(const void* in, int in_dtype, void* out, int out_dtype, int op, int64_t count, int vec) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec) {  // f32 -> f32, both pointers 16-byte aligned
    const int64_t n4 = count >> 2;
    const float4* in4 = reinterpret_cast<const float4*>(in);
    float4* out4 = reinterpret_cast<float4*>(out);
    for (int64_t i = tid; i < n4; i += stride) {
      float4 v = in4[i];
      v.x = tl_unary(op, v.x); v.y = tl_unary(op, v.y); v.z = tl_unary(op, v.z); v.w = tl_unary(op, v.w);
      out4[i] = v;
    }
    for (int64_t i = (n4 << 2) + tid; i < count; i += stride)
      reinterpret_cast<float*>(out)[i] = tl_unary(op, reinterpret_cast<const float*>(in)[i]);
    return;
  }
  for (int64_t i = tid; i < count; i += stride) tl_store_out(out, out_dtype, i, tl_unary(op, ld_as_f32(in, in_dtype, i)));
}

// out[r, c] = a[r, c] (op) b[b_rows == 1 ? 0 : r, c]
__global__ void __launch_bounds__(256) binary_kernel(const void* a, int a_dtype, const void* b, int b_dtype, void* out, int out_dtype,
                                                     int op, int64_t rows, int64_t cols, int b_broadcast) {
  const int64_t count = rows * cols, stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    const float x = ld_as_f32(a, a_dtype, i);
    const float y = ld_as_f32(b, b_dtype, b_broadcast ? i % cols : i);
    tl_store_out(out, out_dtype, i, op == TL_BINARY_ADD ? x + y : op == TL_BINARY_SUB ? x - y : x * y);
  }
}

// out[b, c, r] = in[b, r, c] through a 32 x 33 shared tile (both sides coalesced)
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* in, T* out, int64_t rows, int64_t cols) {
  __shared__ T tile[32][33];
  const int64_t base = int64_t(blockIdx.z) * rows * cols;
  const int64_t c0 = int64_t(blockIdx.x) * 32, r0 = int64_t(blockIdx.y) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8)
    if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = in[base + (r0 + j) * cols + c0 + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (c0 + j < cols && r0 + tx < rows) out[base + (c0 + j) * rows + r0 + tx] = tile[tx][j];
}

int grid_for(tl_ctx* ctx, int64_t work_items) {
  const int64_t blocks = (work_items + 255) / 256;
  return int(std::max<int64_t>(1, std::min<int64_t>(blocks, int64_t(ctx->sm_count) * 8)));
}

}  // namespace

extern "C" {

int32_t tl_unary_op(tl_ctx* ctx, int32_t op, const void* in, int32_t in_dtype, void* out, int32_t out_dtype, int64_t count) {
  TL_CHECK_CTX(ctx);
  if (count < 0 || (count > 0 && (!in || !out))) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_unary_op: null pointer or negative count");
  if (!tl_dtype_valid(in_dtype) || !tl_dtype_valid(out_dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_unary_op: unknown dtype");
  if (op < 0 || op > TL_UNARY_GELU_ERF) return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_unary_op: unknown op %d", op);
  if (count == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  const bool vec = in_dtype == TL_F32 && out_dtype == TL_F32 && !((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15);
  unary_kernel<<<grid_for(ctx, vec ? count / 4 + 1 : count), 256, 0, ctx->stream>>>(in, in_dtype, out, out_dtype, op, count, vec ? 1 : 0);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_binary_op(tl_ctx* ctx, int32_t op, const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, void* out, int32_t out_dtype,
                     int64_t rows, int64_t cols, int32_t b_is_row) {
  TL_CHECK_CTX(ctx);
  if (rows < 0 || cols < 0 || (rows * cols > 0 && (!a || !b || !out))) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_binary_op: null pointer or negative shape");
  if (!tl_dtype_valid(a_dtype) || !tl_dtype_valid(b_dtype) || !tl_dtype_valid(out_dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_binary_op: unknown dtype");
  if (op != TL_BINARY_ADD && op != TL_BINARY_SUB && op != TL_BINARY_MUL) return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_binary_op: unknown op %d", op);
  if (rows * cols == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  binary_kernel<<<grid_for(ctx, rows * cols), 256, 0, ctx->stream>>>(a, a_dtype, b, b_dtype, out, out_dtype, op, rows, cols, b_is_row ? 1 : 0);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_transpose2d(tl_ctx* ctx, const void* in, void* out, int64_t batch, int64_t rows, int64_t cols, int32_t elem_bytes) {
  TL_CHECK_CTX(ctx);
  if (batch < 0 || rows < 0 || cols < 0 || (batch * rows * cols > 0 && (!in || !out)) || in == out)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_transpose2d: null or aliased pointers, or a negative shape");
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_transpose2d: elements of 1, 2 or 4 bytes");
  if (batch > 65535 || (rows + 31) / 32 > 65535) return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_transpose2d: shape too large for one launch");
  if (batch * rows * cols == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  dim3 grid(unsigned((cols + 31) / 32), unsigned((rows + 31) / 32), unsigned(batch));
  if (elem_bytes == 4) transpose_kernel<uint32_t><<<grid, 256, 0, ctx->stream>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), rows, cols);
  else if (elem_bytes == 2) transpose_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), rows, cols);
  else transpose_kernel<uint8_t><<<grid, 256, 0, ctx->stream>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), rows, cols);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

}  // extern "C"
