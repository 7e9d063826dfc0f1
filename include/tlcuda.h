/*
 * tlcuda.h — C ABI of the sm_100a quantized-weight matmul library
 * (libtlcuda.so).  This is the boundary a torchlette `cuda` backend binds:
 * plain pointers and sizes, no C++ or framework types.
 *
 * Conventions
 *   - One opaque context per GPU.  A context owns one CUDA stream, its scratch
 *     memory, the variant/tuning tables and the route counters.
 *   - Every call returns an int32 status (0 = TL_OK, negative = error) and
 *     stores a message readable with tl_last_error().  No call throws, aborts
 *     or frees caller memory.  Argument errors are detected before anything is
 *     launched.
 *   - Compute entry points take raw device pointers (memory from tl_alloc or
 *     from any other allocator on the same device) and only ENQUEUE work on
 *     the context's stream; tl_sync() waits for it.
 *   - A context is single-caller (thread-compatible, not thread-safe).
 *   - Packed weight layout is fixed by the reference quantizer
 *     (src/backend/quantize.ts:62-131): u32 [N, K/4], four signed int8 per
 *     word, byte lane = k & 3, lowest k in bits 0-7; scales [N, K/G] row-major.
 *
 * Each declaration names the torchlette interface it replaces (paths relative
 * to the torchlette repository root).
 */
#ifndef TLCUDA_H_
#define TLCUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define TL_API
#else
#define TL_API __attribute__((visibility("default")))
#endif

typedef struct tl_ctx tl_ctx;

/* ---- status codes ------------------------------------------------------ */
enum {
  TL_OK = 0,
  TL_ERR_INVALID_ARG = -1,   /* the reference throws a JS Error for these */
  TL_ERR_UNSUPPORTED = -2,
  TL_ERR_CUDA = -3,
  TL_ERR_NCCL = -4,
  TL_ERR_TIMEOUT = -5,       /* a bounded device-side wait ran out */
  TL_ERR_OOM = -6,
  TL_ERR_UNIMPLEMENTED = -7
};

/* ---- element types (src/backend/types.ts:133 DType, plus bf16) --------- */
enum { TL_F32 = 0, TL_F16 = 1, TL_BF16 = 2 };

/* ---- operand storage format -------------------------------------------- */
/* Mirrors StorageFormat.packing / QuantPacking (src/backend/types.ts:38-67),
 * widened with the per-channel f32 "direct" convention:
 *   scale_convention TL_SCALE_SNORM127: w = (q/127) * s   (quantize.ts:138-156)
 *   scale_convention TL_SCALE_DIRECT  : w = q * s
 * group_size divides K; group_size == K is per-output-channel. */
enum { TL_SCHEME_INT8_GROUPED = 1, TL_SCHEME_INT4_GROUPED = 2 };
enum { TL_SCALE_SNORM127 = 0, TL_SCALE_DIRECT = 1 };
typedef struct tl_quant_desc {
  int32_t scheme;
  int32_t group_size;
  int32_t scales_dtype; /* TL_F16 or TL_F32 */
  int32_t scale_convention;
} tl_quant_desc;

/* ---- fused epilogue ------------------------------------------------------ */
/* Mirrors EpilogueConfig + epilogueInputs (src/backend/webgpu/matmul/types.ts:
 * 13-24; GEMV seam src/backend/webgpu/matmul/gemv.ts:135-192; tiled seam
 * src/schedule/matmul-skeleton.ts:916-966).  The chain is evaluated in f32 in
 * listed order on acc*alpha; the result is cast to out_dtype at the store.
 *   bias   : v += inputs[input_index][col]            (f32 [N])
 *   unary  : v = op(v)
 *   binary : v = v (op) inputs[input_index][row*N+col] (f32 [M,N])
 *   cast   : v = round-trip through to_dtype */
enum { TL_EPI_NONE = 0, TL_EPI_BIAS = 1, TL_EPI_UNARY = 2, TL_EPI_BINARY = 3, TL_EPI_CAST = 4 };
enum {
  TL_UNARY_RELU = 1, TL_UNARY_SILU = 2, TL_UNARY_SIGMOID = 3, TL_UNARY_TANH = 4,
  TL_UNARY_GELU_TANH = 5, /* the reference's op name "gelu" */
  TL_UNARY_GELU_ERF = 6
};
enum { TL_BINARY_ADD = 1, TL_BINARY_SUB = 2, TL_BINARY_MUL = 3 };
#define TL_EPI_MAX_OPS 8
#define TL_EPI_MAX_INPUTS 4
typedef struct tl_epilogue_op {
  int32_t kind;
  int32_t op;
  int32_t input_index;
  int32_t to_dtype;
} tl_epilogue_op;
typedef struct tl_epilogue {
  int32_t n_ops;
  tl_epilogue_op ops[TL_EPI_MAX_OPS];
  int32_t n_inputs;
  const void* inputs[TL_EPI_MAX_INPUTS];
} tl_epilogue;

/* ---- context -------------------------------------------------------------- */
/* initWebGPU / destroyWebGPU / syncWebGPU / getWebGPUInitError /
 * getGpuUncapturedErrorCount (src/backend/webgpu/index.ts:39-70,
 * src/backend/webgpu/gpu-context.ts:386-405). */
/* Read from the environment at tl_ctx_create (the reference's ENV, src/core/env.ts:14-26):
 *   TORCHLETTE_CUDA_VARIANT=family,kernel[,p0,p1,p2,p3]  start with that variant forced (tl_force_variant)
 *   TORCHLETTE_CUDA_PROFILE=1   CUDA events around every tl_qgemv_nt / tl_qgemm_nt / tl_qmatmul_nt / tl_matmul
 *                               call, one "[tl profile] label m n k: us" line per call on stderr (the
 *                               analogue of TORCHLETTE_PROFILE=1, src/backend/webgpu/profiler.ts); it
 *                               synchronises after each call and is silent during graph capture
 * and, where they are used: TORCHLETTE_GEMV=0, TORCHLETTE_AUTOTUNE=1, TORCHLETTE_DEBUG_AUTOTUNE=1, TL_NCCL_LIB. */
TL_API int32_t tl_ctx_create(int32_t device_ordinal, tl_ctx** out_ctx);
TL_API int32_t tl_ctx_destroy(tl_ctx* ctx);
TL_API int32_t tl_sync(tl_ctx* ctx);
TL_API int64_t tl_async_error_count(tl_ctx* ctx);
/* Message of the last failing call on ctx (or of the last failing call without
 * a context when ctx is NULL).  Valid until the next call on the same thread. */
TL_API const char* tl_last_error(tl_ctx* ctx);
/* The CUDA stream every enqueue goes to (a cudaStream_t), so a host framework
 * can order its own work or record its own events on it. */
TL_API int32_t tl_ctx_stream(tl_ctx* ctx, void** out_stream);
TL_API int32_t tl_device_sm_count(tl_ctx* ctx, int32_t* out_sms);
/* Per-context settings by name, the analogue of the reference's single ENV accessor
 * (src/core/env.ts:14-26).  Unknown names return TL_ERR_INVALID_ARG.
 *   "wait_limit_polls"       upper bound of the polls of one bounded device-side wait of the
 *                            peer collectives (default 2^26; the fused GEMV + all-reduce caps it
 *                            at 2^22).
 *   "push_poll_ranks"        reduce-on-read (tl_qgemv_nt_push's consumer): how many ranks' words a
 *                            summing thread requests together before it checks them, 1..4
 *                            (default 4; 1 polls the ranks one after the other). */
TL_API int32_t tl_set_option(tl_ctx* ctx, const char* name, int64_t value);
TL_API int32_t tl_get_option(tl_ctx* ctx, const char* name, int64_t* out_value);

/* ---- memory: tensorFromArray / read / destroy (src/backend/types.ts:341-345,
 * :666) ---------------------------------------------------------------------- */
TL_API int32_t tl_alloc(tl_ctx* ctx, size_t bytes, void** out_dptr);
TL_API int32_t tl_free(tl_ctx* ctx, void* dptr);
TL_API int32_t tl_upload(tl_ctx* ctx, void* dst_dptr, const void* src_host, size_t bytes);
TL_API int32_t tl_download(tl_ctx* ctx, void* dst_host, const void* src_dptr, size_t bytes);
TL_API int32_t tl_host_alloc_pinned(tl_ctx* ctx, size_t bytes, void** out_hptr);
TL_API int32_t tl_host_free_pinned(tl_ctx* ctx, void* hptr);
TL_API int32_t tl_memset(tl_ctx* ctx, void* dptr, int32_t byte_value, size_t bytes);
/* Strided device-to-device copy on the context's stream (height rows of
 * width_bytes, pitches in bytes): the `contiguous` of a column slice. */
TL_API int32_t tl_copy2d(tl_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                         size_t width_bytes, size_t height);

/* ---- device quantizer: the same function with the weight already on the GPU ----
 * (src/backend/quantize.ts:77-131; the loader quantizes at load time,
 * examples/qwen3/loader.ts:228-253).  weight f32 [n,k], packed u32 [n,k/4] and scales
 * u16 [n,k/group] are DEVICE buffers; enqueued on the context's stream.  Bit-identical to
 * tl_quantize_linear_weight.  group_size must be a multiple of 4. */
TL_API int32_t tl_quantize_linear_weight_device(tl_ctx* ctx, const float* weight, int64_t n, int64_t k,
                                                int32_t group_size, uint32_t* packed, uint16_t* scales);

/* ---- host quantizer: quantizeLinearWeight (src/backend/quantize.ts:77-131) --
 * weight f32 [n,k] (host) -> packed u32 [n,k/4] + scales u16 [n,k/group] (f16
 * bits of the group abs-max), both host buffers.  Multi-threaded over rows. */
TL_API int32_t tl_quantize_linear_weight(const float* weight, int64_t n, int64_t k,
                                         int32_t group_size, uint32_t* packed, uint16_t* scales);
/* f32ToF16Bits / f16BitsToF32 (src/backend/quantize.ts:22-60). */
TL_API uint32_t tl_f32_to_f16_bits(float value);
TL_API float tl_f16_bits_to_f32(uint32_t bits);

/* ---- the hot path ---------------------------------------------------------- */
/* dispatchQuantizedGemvNT (src/backend/webgpu/matmul/dispatch.ts:875-931),
 * widened to m in [1,16], f16/bf16/f32 activations and outputs, and the GEMV
 * epilogue seam (gemv.ts:168-192):
 *   out[r, c] = epilogue(alpha * sum_k a[r,k] * dequant(packed, scales)[c,k])
 * a: [m,k] a_dtype row-major; out: [m,n] out_dtype row-major; f32 accumulate.
 * Bumps the quant-GEMV counter.  epilogue may be NULL. */
TL_API int32_t tl_qgemv_nt(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed,
                           const void* scales, void* out, int32_t out_dtype, int32_t m, int64_t n,
                           int64_t k, const tl_quant_desc* qdesc, float alpha,
                           const tl_epilogue* epilogue);

/* Horizontal fusion (no counterpart in the reference, which dispatches one GEMV per linear):
 * up to 4 projections that read the SAME activations a[m,k] -- q/k/v, gate/up -- in ONE
 * launch.  Each item has its own weight, scales, output [m, n_i], alpha and epilogue; m, k,
 * dtypes and the packing descriptor are shared.  Results are identical to n_items
 * tl_qgemv_nt calls (shapes the fused kernel does not take are run that way); the
 * quant-GEMV counter moves by n_items. */
typedef struct tl_qgemv_item {
  const void* packed;
  const void* scales;
  void* out;
  int64_t n;
  float alpha;
  const tl_epilogue* epilogue; /* may be NULL */
} tl_qgemv_item;
TL_API int32_t tl_qgemv_nt_batched(tl_ctx* ctx, const void* a, int32_t a_dtype, const tl_qgemv_item* items,
                                   int32_t n_items, int32_t out_dtype, int32_t m, int64_t k,
                                   const tl_quant_desc* qdesc);

/* Vertical fusion (no counterpart in the reference, whose executor replays one dispatch per
 * node of a compiled plan, src/executor/lazy-executor.ts): a whole SEQUENCE of dependent
 * small-batch products -- the matmuls of a decode step -- in one persistent cooperative
 * launch.  A phase is 1..4 projections that read the same activations a[m, k] (the items of
 * tl_qgemv_nt_batched); phases run in order, and the activations of a phase may be outputs of
 * any earlier phase.  The weight stream runs ahead across phase boundaries.  Experimental:
 * results are exact, but on the decode stack it measured slower than a replayed graph of
 * tl_qgemv_nt launches, which stays the recommended path.  Results equal those of tl_qgemv_nt on the
 * same operands (same summation order as its "ring" kernel with 8 warps).
 * Limits: m in [1,16]; f16/bf16 activations, 16-byte aligned; every K % 64 == 0; group_size
 * % 64 == 0 and dividing K (group_size == k: one scale per output channel); an item's out
 * must not alias its phase's activations.  Pointers (weights, scales, outputs, activations,
 * epilogue inputs) are captured at creation and must stay valid until the chain is destroyed.
 * tl_qgemv_chain_launch enqueues a 4-byte-per-phase memset and the kernel on the context's
 * stream; it moves the quant-GEMV counter by the number of items and the launch counter by 1. */
typedef struct tl_chain tl_chain;
typedef struct tl_chain_phase {
  const void* a;      /* activations [m, k] */
  int64_t k;
  int32_t group_size; /* as tl_quant_desc.group_size, for this phase's K */
  int32_t out_dtype;  /* of this phase's outputs [m, n_i] */
  int32_t n_items;
  int32_t reserved;
  tl_qgemv_item items[4];
} tl_chain_phase;
TL_API int32_t tl_qgemv_chain_create(tl_ctx* ctx, const tl_chain_phase* phases, int32_t n_phases, int32_t a_dtype,
                                     int32_t m, int32_t scales_dtype, int32_t scale_convention, tl_chain** out);
TL_API int32_t tl_qgemv_chain_launch(tl_ctx* ctx, tl_chain* chain);
TL_API int32_t tl_qgemv_chain_destroy(tl_ctx* ctx, tl_chain* chain);

/* No counterpart in the reference.  Same operation and arguments as tl_qgemv_nt for
 * hosts that must not allocate device memory at call time (all device memory belongs
 * to the host's own pool, so a library's cudaMalloc can only fail; or cudaMalloc's
 * device-wide synchronisation cannot be tolerated): the kernel's partial-sum scratch is a fixed
 * 4 MiB array inside the library image instead of a buffer grown with cudaMalloc, so
 * the call makes no allocation.  Limits: f16/bf16 activations, K % 128 == 0,
 * group_size % 64 == 0, and m*n*4 + ceil(n/256)*64 <= 4 MiB (else TL_ERR_UNSUPPORTED).
 * All calls on a device share the array: calls ordered on one stream are safe, calls
 * that overlap on the GPU race.  The first call on a device also looks up the array's
 * address (a one-time set-up step); make that call before any stream capture starts. */
TL_API int32_t tl_qgemv_nt_static_scratch(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed,
                                          const void* scales, void* out, int32_t out_dtype, int32_t m,
                                          int64_t n, int64_t k, const tl_quant_desc* qdesc, float alpha,
                                          const tl_epilogue* epilogue);

/* Prefill GEMM with dequantization fused into the tile loads (tcgen05 / TMEM).
 * Replaces the reference's dispatchDequantizeInt8Grouped + dispatchMatmul pair
 * for m > 1 (src/backend/webgpu/ops/matmul-ops.ts:163-181).  a is f16 or bf16;
 * the dequantized weight is rounded to a_dtype before the tensor-core product.
 * Bumps the quant-GEMM counter. */
TL_API int32_t tl_qgemm_nt(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed,
                           const void* scales, void* out, int32_t out_dtype, int64_t m, int64_t n,
                           int64_t k, const tl_quant_desc* qdesc, float alpha,
                           const tl_epilogue* epilogue);

/* The backend matmul seam for a packed B operand: matmulQuantizedB
 * (src/backend/webgpu/ops/matmul-ops.ts:113-182).  Routes m <= 16 to
 * tl_qgemv_nt and larger m to tl_qgemm_nt. */
TL_API int32_t tl_qmatmul_nt(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed,
                             const void* scales, void* out, int32_t out_dtype, int64_t m,
                             int64_t n, int64_t k, const tl_quant_desc* qdesc, float alpha,
                             const tl_epilogue* epilogue);

/* dispatchDequantizeInt8Grouped (src/backend/webgpu/matmul/dispatch.ts:949-1037):
 * out[n,k] = dequant(packed, scales).  With out_dtype TL_F32 the result is
 * bit-identical to dequantizeToF32 (quantize.ts:138-156).  Bumps the dequant
 * counter. */
TL_API int32_t tl_dequant_int8(tl_ctx* ctx, const void* packed, const void* scales, void* out,
                               int32_t out_dtype, int64_t n, int64_t k,
                               const tl_quant_desc* qdesc);
/* Debug op: the signed byte lanes as int8 [n,k] (integer half of the dequant). */
TL_API int32_t tl_unpack_int8(tl_ctx* ctx, const void* packed, void* out_i8, int64_t n, int64_t k);

/* ---- companion ops: the unfused forms of what the epilogue fuses, and the materialization of
 * a transposed view (BackendOps add / sub / mul / relu / silu / gelu / cast / contiguous,
 * src/backend/types.ts:340-680; composed by matmulQuantizedB's explicit-dequant path,
 * src/backend/webgpu/ops/matmul-ops.ts:163-181).  One HBM pass each.
 * tl_unary_op: out[i] = op(in[i]); op is TL_UNARY_* or 0 for a plain cast / copy; dtypes independent.
 * tl_binary_op: out[r,c] = a[r,c] (op) b[r,c], or b[c] when b_is_row (a bias row); op is TL_BINARY_*.
 * tl_transpose2d: out[b,c,r] = in[b,r,c] for elements of 1, 2 or 4 bytes (in != out). */
TL_API int32_t tl_unary_op(tl_ctx* ctx, int32_t op, const void* in, int32_t in_dtype, void* out,
                           int32_t out_dtype, int64_t count);
TL_API int32_t tl_binary_op(tl_ctx* ctx, int32_t op, const void* a, int32_t a_dtype, const void* b,
                            int32_t b_dtype, void* out, int32_t out_dtype, int64_t rows, int64_t cols,
                            int32_t b_is_row);
TL_API int32_t tl_transpose2d(tl_ctx* ctx, const void* in, void* out, int64_t batch, int64_t rows,
                              int64_t cols, int32_t elem_bytes);

/* ---- the other ops of one decode step (packages/qwen3-browser/src/model.ts:220-420), so that a step
 * runs on this backend end to end.  f32 arithmetic; storage f32 / f16 / bf16.
 * tl_rmsnorm: out[r,c] = x[r,c] * rsqrt(mean_c(x[r,:]^2) + eps) * weight[c]
 *   (src/ops/semantic/composite.ts:156-170; rows x cols, also the per-head q / k norm with cols = headDim).
 * tl_rope: the half-split rotation of fusedRoPE (src/backend/webgpu/rope-kernel.ts:1-93,
 *   src/backend/types.ts:593-598): qk is [outer, seq_len, head_dim], cos / sin are f32 [.., head_dim/2]
 *   tables read at row s from the given element offsets (a narrow() view of a persistent table);
 *   first half  out[d] = qk[d] cos - qk[d + D/2] sin, second half out[d] = qk[d] cos + qk[d - D/2] sin;
 *   sin_scale -1 is the inverse rotation.  Not in place.
 * tl_decode_attention: one query token per sequence against a KV cache (model.ts:292-312): q is
 *   [batch, n_heads, head_dim], the caches are [batch, n_kv_heads, kv_capacity, head_dim] of which the
 *   first kv_len positions are read; query head h reads kv head h / (n_heads / n_kv_heads) (the order of
 *   expandKV, model.ts:171-180); out[b,h,:] = softmax_j(q . k_j * scale + mask[j]) . v; mask is f32
 *   [kv_len] or NULL.  kv_len <= 51200 per launch.  (Appending this step's k / v at a position is
 *   tl_copy2d; the residual adds are tl_binary_op; silu(gate) * up rides in an epilogue.) */
TL_API int32_t tl_rmsnorm(tl_ctx* ctx, const void* x, int32_t x_dtype, const void* weight, int32_t weight_dtype,
                          void* out, int32_t out_dtype, int64_t rows, int64_t cols, float eps);
TL_API int32_t tl_rope(tl_ctx* ctx, const void* qk, int32_t dtype, const float* cos_table, const float* sin_table,
                       void* out, int64_t outer, int64_t seq_len, int64_t head_dim, float sin_scale,
                       int64_t cos_offset, int64_t sin_offset);
/* tl_attention: the same for q_len query positions per sequence: q [batch, n_heads, q_len, head_dim],
 * out [batch, q_len, n_heads, head_dim] (the permute in front of o_proj, model.ts:314-318, is folded
 * into the store).  causal != 0: query s sees the keys up to position kv_len - q_len + s (the triu mask
 * of model.ts:300-307; prefill is kv_len == q_len).  mask, if given, is f32 [q_len, kv_len], added to
 * the scores.  tl_decode_attention is q_len = 1. */
TL_API int32_t tl_attention(tl_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, void* out,
                            int32_t dtype, int64_t batch, int64_t n_heads, int64_t n_kv_heads, int64_t q_len,
                            int64_t head_dim, int64_t kv_len, int64_t kv_capacity, float scale,
                            const float* mask, int32_t causal);
TL_API int32_t tl_decode_attention(tl_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, void* out,
                                   int32_t dtype, int64_t batch, int64_t n_heads, int64_t n_kv_heads,
                                   int64_t head_dim, int64_t kv_len, int64_t kv_capacity, float scale,
                                   const float* mask);

/* ---- selection: planTiledMatmul / selectMatmulChoice / SelectionReceipt
 * (src/backend/webgpu/matmul/dispatch.ts:171-192, 1130-1329;
 *  src/backend/webgpu/matmul/variants.ts:54-260) ------------------------------ */
/* Kernel ids and parameters by family (tl_variant_name prints them):
 *   TL_FAMILY_QGEMV  (m <= 16): 0 scalar, 1 simt, 2 mma, 3 sk, 4 ring (default; p0 warps, p1 k blocks in flight,
 *                    p2 = 2: 32-row tiles), 5 tma, 6 bulk, 7 chain, 8 stream, 9 int4
 *   TL_FAMILY_QGEMM  (m > 16): 0 tcgen05 with the int8 -> 16-bit conversion on the operand path (p0 token tile,
 *                    p1 k per stage, p2 stages, p3 converter warps); 1 sliced (sixteen-row slices through the
 *                    small-batch kernels: f32 activations, odd K); 2 dequant+dense (the weight written once as a
 *                    16-bit matrix into scratch, then the dense tcgen05 kernel; receipt: p0 BN, p1 stages, p2 MH)
 *   TL_FAMILY_MATMUL (dense): 0 tiled (CUDA cores, always applicable), 1 gemv (m <= 16 NT; p0 warps),
 *                    2 tc (tcgen05, both operands from shared memory; p0 BN columns per tile, p1 stages,
 *                    p2 MH = row halves of 128 per tile; forcing with p0 = 0 leaves the tile to the library) */
enum { TL_FAMILY_QGEMV = 1, TL_FAMILY_QGEMM = 2, TL_FAMILY_MATMUL = 3 };
typedef struct tl_variant {
  int32_t family;   /* TL_FAMILY_* */
  int32_t kernel;   /* family-specific kernel id (see tl_variant_name) */
  int32_t p0, p1, p2, p3; /* family-specific parameters */
} tl_variant;
typedef struct tl_plan_receipt {
  tl_variant choice;
  int32_t grid[3];
  int32_t block;
  int32_t split_k;
  int32_t from_tuning_cache; /* 1: the exact shape's tuned winner was used; 2: its shape class's */
  int32_t epilogue_engaged;
} tl_plan_receipt;
/* Pure function of geometry, dtypes and format: what tl_qmatmul_nt would run. */
TL_API int32_t tl_plan_qmatmul(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                               int32_t out_dtype, const tl_quant_desc* qdesc,
                               const tl_epilogue* epilogue, tl_plan_receipt* out_receipt);
/* ---- int4-grouped: the scheme the reference plans as "a new value on the format axis"
 * (docs/quantization-design.md:69-75, 386-396; no code there).  Packed u32 [N, K/8], eight int4 per
 * word, nibble j = k & 7 in bits 4j..4j+3, two's complement in [-7, 7]; scales [N, K/G] as for int8
 * (f16 abs-max with w = (q/7)*scale when the convention is TL_SCALE_SNORM127, or f32 direct scales).
 * K % 8 == 0, G % 8 == 0.  tl_qmatmul_nt / tl_qgemv_nt / tl_qgemm_nt / tl_plan_qmatmul accept a
 * descriptor with scheme TL_SCHEME_INT4_GROUPED: m <= 16 runs the fused-dequant int4 GEMV, larger m
 * dequantizes into library scratch and runs tl_matmul (the reference's explicit-dequant fallback).
 * The batched / chain / push / static-scratch entry points are int8 only. */
TL_API int32_t tl_quantize_linear_weight_int4(const float* weight, int64_t n, int64_t k, int32_t group_size,
                                              uint32_t* packed, uint16_t* scales);
TL_API int32_t tl_dequant_int4(tl_ctx* ctx, const void* packed, const void* scales, void* out,
                               int32_t out_dtype, int64_t n, int64_t k, const tl_quant_desc* qdesc);
/* Debug op: the signed nibbles as int8 [n,k]. */
TL_API int32_t tl_unpack_int4(tl_ctx* ctx, const void* packed, void* out_i8, int64_t n, int64_t k);

/* ---- dense matmul: dispatchTiledMatmul / dispatchMatmul for an unquantized B
 * (src/backend/webgpu/matmul/dispatch.ts:1331-1700; dense GEMV builders
 *  src/backend/webgpu/matmul/gemv.ts:430-532; tiled body
 *  src/schedule/matmul-skeleton.ts:738-908).
 * out[b] = epilogue(alpha * op(A[b]) . op(B[b])), f32 accumulation.
 *   A is [m,k] row-major, or [k,m] when trans_a; B is [k,n], or [n,k] when trans_b; out [m,n].
 *   stride_a / stride_b / stride_c: elements between consecutive batches; 0 broadcasts an
 *   operand over the batch (dispatch.ts:1411-1510); stride_c >= m*n when batch > 1.
 *   dtype_a, dtype_b, out_dtype: any of TL_F32 / TL_F16 / TL_BF16, independently.
 *   cast_a, cast_b: -1, or TL_F16 / TL_BF16 to round the operand through that type as it is
 *   loaded (the read-wider-cast-on-load prologue, variants.ts:170-175).
 *   A binary epilogue input is [m,n] and needs batch == 1.
 * Selection: m <= 16, batch 1, trans_b, no trans_a, both operands the same 2-byte type, k % 32 == 0
 * and 16-byte aligned pointers run the tensor-core GEMV (counter TL_COUNTER_GEMV) unless the
 * environment has TORCHLETTE_GEMV=0 or tl_force_variant names {TL_FAMILY_MATMUL, 0}; all else
 * runs the tiled kernel (TL_COUNTER_MATMUL).  With receipt_only non-NULL nothing is launched
 * and the operand pointers may be NULL: the choice is written there (planTiledMatmul). */
TL_API int32_t tl_matmul(tl_ctx* ctx, const void* a, const void* b, void* out, int64_t m, int64_t n,
                         int64_t k, int64_t batch, int64_t stride_a, int64_t stride_b,
                         int64_t stride_c, int32_t trans_a, int32_t trans_b, float alpha,
                         int32_t dtype_a, int32_t dtype_b, int32_t out_dtype, int32_t cast_a,
                         int32_t cast_b, const tl_epilogue* epilogue, tl_plan_receipt* receipt_only);
TL_API const char* tl_variant_name(const tl_variant* v);
/* Force one variant for every following call (NULL clears).  A/B testing hook,
 * the analogue of an explicit MatmulKernelConfig (variants.ts:214-236). */
TL_API int32_t tl_force_variant(tl_ctx* ctx, const tl_variant* v);

/* ---- route counters (src/backend/webgpu/matmul/dispatch.ts:833-864, 943-947) */
enum {
  TL_COUNTER_QGEMV = 0,         /* getQuantGemvDispatchCount */
  TL_COUNTER_DEQUANT = 1,       /* getDequantI8DispatchCount */
  TL_COUNTER_QGEMV_EPILOGUE = 2,/* getGemvEpilogueDispatchCount */
  TL_COUNTER_QGEMM = 3,
  TL_COUNTER_KERNEL_LAUNCHES = 4, /* every kernel this library launched */
  TL_COUNTER_GEMV = 5,          /* getGemvDispatchCount: dense small-batch GEMV */
  TL_COUNTER_MATMUL = 6,        /* dense tiled matmul */
  TL_COUNTER_COUNT = 7
};
TL_API int64_t tl_counter_get(tl_ctx* ctx, int32_t which);
TL_API int32_t tl_counters_reset(tl_ctx* ctx);

/* ---- autotune (src/backend/webgpu/matmul/autotune.ts:97-329;
 * src/backend/webgpu/matmul/dispatch.ts:79-141, 405-578) ---------------------- */
typedef struct tl_shape { int64_t m, n, k; } tl_shape;
/* classifyShape (src/backend/webgpu/matmul/types.ts:77-200): the class a geometry falls in.  A shape
 * tuned by tl_pretune (or imported) also becomes its class's winner; selection order is
 * forced variant -> exact-shape winner -> class winner -> default, each re-gated on
 * applicability.  tl_plan_receipt.from_tuning_cache: 0 none, 1 exact shape, 2 shape class. */
enum {
  TL_SHAPE_SQUARE_SMALL = 0, TL_SHAPE_SQUARE_MEDIUM = 1, TL_SHAPE_SQUARE_LARGE = 2, TL_SHAPE_TALL_SKINNY = 3,
  TL_SHAPE_SHORT_WIDE = 4, TL_SHAPE_LARGE_K = 5, TL_SHAPE_SMALL_K = 6, TL_SHAPE_GEMV = 7, TL_SHAPE_GEMV_ROW = 8,
  TL_SHAPE_BATCHED_SMALL = 9
};
TL_API int32_t tl_classify_shape(int64_t m, int64_t n, int64_t k, int64_t batch);
TL_API const char* tl_shape_class_name(int32_t shape_class);
TL_API int32_t tl_autotune_set_enabled(tl_ctx* ctx, int32_t enabled);
TL_API int32_t tl_autotune_is_enabled(tl_ctx* ctx);
/* pretuneMatmulShapes: time every applicable candidate for each shape on
 * rotated buffers and cache the winner per exact (m,n,k,dtype,format). */
TL_API int32_t tl_pretune(tl_ctx* ctx, const tl_shape* shapes, int32_t n_shapes, int32_t a_dtype,
                          int32_t out_dtype, const tl_quant_desc* qdesc);
TL_API int32_t tl_tune_seed(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                            const tl_quant_desc* qdesc, const tl_variant* choice);
TL_API int32_t tl_tune_get(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                           const tl_quant_desc* qdesc, tl_variant* out_choice); /* 1 = found */
TL_API int32_t tl_tune_clear(tl_ctx* ctx);
TL_API int64_t tl_tune_run_count(tl_ctx* ctx);
/* exportTuningCache / importTuningCache: JSON text.  Export writes at most cap
 * bytes (NUL-terminated) and returns the full length needed in *out_len. */
TL_API int32_t tl_tune_export_json(tl_ctx* ctx, char* buf, size_t cap, size_t* out_len);
TL_API int32_t tl_tune_import_json(tl_ctx* ctx, const char* json);

/* ---- replay: the analogue of the reference's CompiledPlan replay
 * (src/executor/executor.ts:1249) is a captured CUDA graph of enqueued calls. */
/* A captured graph keeps the addresses of the library's scratch buffers of its capture time.  A
 * later call that needs more scratch allocates a new buffer; the old one stays allocated for as
 * long as any graph of the context is alive, so earlier graphs remain valid to replay.  Growing
 * the scratch DURING a capture is refused (run the call once before capturing). */
typedef struct tl_graph tl_graph;
TL_API int32_t tl_graph_begin(tl_ctx* ctx);
TL_API int32_t tl_graph_end(tl_ctx* ctx, tl_graph** out_graph);
TL_API int32_t tl_graph_launch(tl_ctx* ctx, tl_graph* graph);
TL_API int32_t tl_graph_destroy(tl_ctx* ctx, tl_graph* graph);

/* ---- timing on the context's stream (CUDA events) -------------------------- */
typedef struct tl_event tl_event;
TL_API int32_t tl_event_create(tl_ctx* ctx, tl_event** out_event);
TL_API int32_t tl_event_record(tl_ctx* ctx, tl_event* ev);
TL_API int32_t tl_event_elapsed_ms(tl_ctx* ctx, tl_event* start, tl_event* stop, float* out_ms);
/* Blocks the calling host thread until the event has happened.  The one call that another host
 * thread may make while the context's own thread keeps enqueueing: it neither reads nor writes
 * the context's error state (so it returns a bare status, no tl_last_error text).  The N-API
 * shim's Promise-returning download waits with it on a worker thread. */
TL_API int32_t tl_event_synchronize(tl_ctx* ctx, tl_event* ev);
TL_API int32_t tl_event_destroy(tl_ctx* ctx, tl_event* ev);

/* ---- multi-GPU (no counterpart in the reference, whose only parallelism is
 * DiLoCo over WebSocket, src/distributed/) ------------------------------------
 * One context per process/GPU.  tl_comm_unique_id fills a 128-byte NCCL id on
 * rank 0; the host distributes it and every rank calls tl_comm_init. */
#define TL_COMM_ID_BYTES 128
TL_API int32_t tl_comm_unique_id(void* out_id128);
TL_API int32_t tl_comm_init(tl_ctx* ctx, int32_t rank, int32_t world, const void* id128);
TL_API int32_t tl_comm_destroy(tl_ctx* ctx);
/* Column-parallel gather: every rank contributes local [m, n_local]; out is
 * [m, world*n_local] with rank r's columns at offset r*n_local. */
TL_API int32_t tl_allgather_cols(tl_ctx* ctx, const void* local, void* out, int64_t m,
                                 int64_t n_local, int32_t dtype);
/* Row-parallel reduction: in-place sum over ranks of buf[count]. */
TL_API int32_t tl_allreduce_sum(tl_ctx* ctx, void* buf, int64_t count, int32_t dtype);


/* One-shot all-reduce over peer memory (NVLink/NVSwitch P2P loads and stores, no NCCL on
 * the data path) for the small, latency-bound sums of a row-parallel decode step
 * ([m, hidden] partial outputs: tens of KB).  Every rank stages its partial in a buffer
 * that its peers have mapped, raises a flag in every peer's memory, waits (bounded) for
 * the peers' flags and sums all partials in rank order, so every rank computes
 * bit-identical results.  No counterpart in the reference.
 *   tl_p2p_create  allocates this rank's exchange buffer (max_bytes per message) and returns
 *                  a 64-byte inter-process handle to hand to the other ranks;
 *   tl_p2p_attach  maps the peers' buffers from the world*64 handle bytes (rank order);
 *   tl_allreduce_sum_p2p  dst[count] = sum over ranks of src[count]; src may be dst.
 * A wait that runs out sets the context's status word (TL_ERR_TIMEOUT at tl_sync). */
#define TL_P2P_HANDLE_BYTES 64
TL_API int32_t tl_p2p_create(tl_ctx* ctx, size_t max_bytes, void* out_handle64);
TL_API int32_t tl_p2p_attach(tl_ctx* ctx, const void* handles_world_x64);
TL_API int32_t tl_allreduce_sum_p2p(tl_ctx* ctx, const void* src, void* dst, int64_t count, int32_t dtype);
/* After a wait of a peer collective ran out (tl_sync returned TL_ERR_TIMEOUT) the ranks disagree
 * on call counts and the exchange is unusable: every rank must call tl_p2p_reset (it waits for the
 * context's stream, then clears flags, call counters and the status word of ITS buffer), and the
 * host must put a barrier between the resets and the next peer collective.  No counterpart in the
 * reference. */
/* The same exchange for f32 partial sums whose total is stored as dst_dtype (f32, f16 or bf16): the
 * sum is rounded once, so a row-parallel product is as accurate sharded as unsharded.  (With 16-bit
 * partials every rank's rounding error, up to half an ulp of a partial that may be much larger than
 * the total, adds up: measured 1.0e-2 on the metric |x - ref| / max(1, |ref|) at 8 ranks.)
 * dst may alias src only when dst_dtype is f32.  count * 4 bytes must fit the exchange buffer. */
TL_API int32_t tl_allreduce_sum_p2p_f32_to(tl_ctx* ctx, const float* src, void* dst, int32_t dst_dtype,
                                           int64_t count);
TL_API int32_t tl_p2p_reset(tl_ctx* ctx);
/* Diagnostic hook: maps this rank's OWN exchange buffer in place of every peer of a `world`-rank
 * group (rank 0), so that a single process can run the peer kernels on local memory only.  The
 * other ranks' flags are then never raised: a peer collective waits until the context's
 * "wait_limit_polls" is used up and gives up, which is how the time-out path is tested without
 * a second GPU and without a rank that has to be killed.  With world = 1 the group is complete, and
 * tl_qgemv_nt_push followed by its consumer runs the whole push / reduce-on-read path on one GPU
 * (the sum has a single term).  Needs tl_p2p_create; not for contexts that called tl_comm_init. */
TL_API int32_t tl_p2p_attach_loopback(tl_ctx* ctx, int32_t world);

/* Row-parallel projection fused with its all-reduce (tensor parallelism; no counterpart in
 * the reference): out[m, n] = sum over ranks of alpha * a_r[m, k_r] . W_r[n, k_r]^T in ONE
 * kernel.  Every CTA computes a 16-row tile of the local partial product, stores it --
 * rounded to out_dtype, exactly what tl_qgemv_nt would have written -- into all ranks'
 * exchange buffers over NVLink, waits (bounded) for the other ranks' versions of the same
 * tile and writes their sum in rank order, so the result has the bits of tl_qgemv_nt
 * followed by tl_allreduce_sum_p2p.  Needs tl_p2p_create / tl_p2p_attach with max_bytes >=
 * m*n*sizeof(out element); m in [1,16]; f16/bf16 activations; K % 64 == 0; n <= 16384 and
 * the same n for every fused call on a context; no epilogue ops (alpha only: anything
 * non-linear would have to follow the sum).  Collective: every rank must call it in the same
 * order.  With one rank it is tl_qgemv_nt. */
TL_API int32_t tl_qgemv_nt_allreduce(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed,
                                     const void* scales, void* out, int32_t out_dtype, int32_t m, int64_t n,
                                     int64_t k, const tl_quant_desc* qdesc, float alpha);

/* Row-parallel sum WITHOUT a collective launch (tensor parallelism; no counterpart in the
 * reference).  tl_qgemv_nt_push computes this rank's partial product alpha * a_r . W_r^T exactly as
 * tl_qgemv_nt would and, instead of storing it, pushes it -- as 24-bit floats (15 mantissa bits; 16-bit
 * partials measured 1e-2 off at 8 ranks), two of them and an arrival tag per 8-byte word -- into every
 * rank's exchange buffer over NVLink; it waits for nobody.  `out` names the local [m, n] buffer
 * that is to hold the sum over ranks.  The NEXT small-batch launch on the context (tl_qgemv_nt,
 * tl_qgemv_nt_batched or tl_qmatmul_nt with m <= 16) must be the one that reads `out` as its
 * activations: after its weight prefetch it waits (bounded, TL_ERR_TIMEOUT at tl_sync) for all
 * ranks' partials, sums them in rank order into `out` (identical bits on every rank) and then runs
 * its own product.  Any other consumer calls tl_reduce_pending first, which does the same sum in a
 * small launch of its own.  Needs tl_p2p_create / tl_p2p_attach with max_bytes >= m*n*4; m in
 * [1,16]; f16/bf16 activations and outputs; K % 64 == 0; N % 16 == 0; no epilogue ops (alpha only:
 * anything non-linear would have to follow the sum).  Collective: every rank makes the same calls
 * in the same order.  With one rank (and no loopback exchange attached) it is tl_qgemv_nt. */
TL_API int32_t tl_qgemv_nt_push(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed,
                                const void* scales, void* out, int32_t out_dtype, int32_t m, int64_t n,
                                int64_t k, const tl_quant_desc* qdesc, float alpha);
TL_API int32_t tl_reduce_pending(tl_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* TLCUDA_H_ */
