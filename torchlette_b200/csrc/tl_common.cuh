// Shared internals of libtlcuda: the context object, error plumbing, dtype
// helpers and the fused-epilogue evaluator used by every kernel family.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "../../include/tlcuda.h"

// ---------------------------------------------------------------------------
// Context
// ---------------------------------------------------------------------------
struct TuneKey {
  int64_t m, n, k;
  int32_t a_dtype, group, scales_dtype, convention;
  bool operator<(const TuneKey& o) const {
    if (m != o.m) return m < o.m;
    if (n != o.n) return n < o.n;
    if (k != o.k) return k < o.k;
    if (a_dtype != o.a_dtype) return a_dtype < o.a_dtype;
    if (group != o.group) return group < o.group;
    if (scales_dtype != o.scales_dtype) return scales_dtype < o.scales_dtype;
    return convention < o.convention;
  }
};

struct tl_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  int sm_count = 0;
  int l2_bytes = 0;
  int64_t counters[TL_COUNTER_COUNT] = {};
  int64_t async_errors = 0;
  std::string last_error;
  // library-owned scratch (split-K partials, GEMM staging), grown on demand and
  // kept until teardown (the reference caches its K-split scratch the same way:
  // src/backend/webgpu/matmul/dispatch.ts:695-718)
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // second scratch that is all zero between launches: kernels that use it restore
  // the zeros themselves (partial-sum meeting point of the balanced GEMV)
  void* zscratch = nullptr;
  size_t zscratch_bytes = 0;
  // Captured graphs have the scratch pointers of their capture time baked in.  While any tl_graph
  // of this context is alive, a scratch buffer that has to grow is not freed but retired: it stays
  // allocated (the old graphs keep replaying on it) until the last graph is destroyed or the
  // context goes away.
  int live_graphs = 0;
  std::vector<std::pair<void*, size_t>> retired_scratch;
  int* dev_status = nullptr;  // written by kernels whose bounded waits ran out; read back by tl_sync
  // drain-timed ring fill of the streaming GEMV (tl_qgemv_stream.cu): flag words on the device
  // and the slot the next launch takes; stream_scratch holds the partial sums and arrival
  // counters of row tiles that two CTAs share (fixed size, allocated once)
  uint32_t* pf_flags = nullptr;
  int pf_next = 0;
  int pf_last_grid = 0;
  void* stream_scratch = nullptr;
  int wait_limit_polls = 1 << 26;  // bound of one device-side wait of the peer collectives
  int push_poll_ranks = 4;         // reduce-on-read: ranks polled together (1 = one after the other)
  // selection
  bool has_forced = false;
  tl_variant forced{};
  bool autotune_enabled = false;
  int64_t tune_runs = 0;
  std::map<TuneKey, tl_variant> tuned;
  // shape-class winners: the TuneKey's m carries the class id, n the kernel family, k is 0, and a
  // per-channel format (group == K) is recorded as group 0 so that shapes of different K share it
  std::map<TuneKey, tl_variant> class_tuned;
  std::map<int, int> ring_occupancy;  // resident CTAs per SM of each ring kernel shape (queried once)
  bool capturing = false;
  // TORCHLETTE_CUDA_PROFILE=1: CUDA events around every product call, one line per call on stderr
  bool profile = false;
  cudaEvent_t prof_e0 = nullptr, prof_e1 = nullptr;
  // multi-GPU
  void* nccl_comm = nullptr;
  int rank = 0, world = 1;
  // one-shot peer all-reduce: this rank's exchange buffer and the peers' mappings
  static constexpr int kMaxPeers = 8;
  void* p2p_local = nullptr;
  void* p2p_peer[kMaxPeers] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  size_t p2p_max_bytes = 0;
  bool p2p_attached = false;
  int64_t fused_tiles = 0;  // tiles of the fused GEMV + all-reduce calls made on this context (0: none yet)
  // a tl_qgemv_nt_push whose partial sums wait to be reduced by the next small-batch launch
  bool push_pending = false;
  void* push_dst = nullptr;
  int32_t push_m = 0, push_dtype = 0;
  int64_t push_n = 0, push_tiles = 0;
};

int32_t tl_set_error(tl_ctx* ctx, int32_t code, const char* fmt, ...);
int32_t tl_ensure_scratch(tl_ctx* ctx, size_t bytes, void** out);
int32_t tl_ensure_zeroed_scratch(tl_ctx* ctx, size_t bytes, void** out);

#define TL_CHECK_CTX(ctx)                                                       \
  do {                                                                          \
    if ((ctx) == nullptr) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "%s: null context", __func__); \
  } while (0)

#define TL_CUDA(ctx, expr)                                                      \
  do {                                                                          \
    cudaError_t _e = (expr);                                                    \
    if (_e != cudaSuccess) {                                                    \
      if (ctx) (ctx)->async_errors++;                                           \
      return tl_set_error((ctx), TL_ERR_CUDA, "%s: %s failed: %s", __func__, #expr, cudaGetErrorString(_e)); \
    }                                                                           \
  } while (0)

// Sets the calling thread's current device to the context's for one scope.
// Per-call timing behind TORCHLETTE_CUDA_PROFILE=1 (the reference's TORCHLETTE_PROFILE=1 timestamp pairs per
// compute pass, src/backend/webgpu/profiler.ts, webgpu/dispatch.ts:80-84): two events around the call's
// launches on the context's stream, a synchronize, and one line "[tl profile] <label> m n k: us" on stderr.
// It serialises the stream, so it is for reading kernel times, not for running a benchmark; it does nothing
// while a graph is being captured.
struct TlProfileScope {
  tl_ctx* ctx;
  const char* label;
  int64_t m, n, k;
  bool on;
  TlProfileScope(tl_ctx* c, const char* l, int64_t m_, int64_t n_, int64_t k_);
  ~TlProfileScope();
};

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

static inline size_t tl_dtype_size(int32_t dt) { return dt == TL_F32 ? 4 : 2; }
static inline bool tl_dtype_valid(int32_t dt) { return dt == TL_F32 || dt == TL_F16 || dt == TL_BF16; }
static inline const char* tl_dtype_name(int32_t dt) {
  return dt == TL_F32 ? "f32" : dt == TL_F16 ? "f16" : dt == TL_BF16 ? "bf16" : "?";
}

// ---------------------------------------------------------------------------
// Epilogue parameters as passed (by value) to kernels
// ---------------------------------------------------------------------------
struct EpiParams {
  int32_t n_ops;
  int32_t kind[TL_EPI_MAX_OPS];
  int32_t op[TL_EPI_MAX_OPS];
  int32_t idx[TL_EPI_MAX_OPS];  // input index (bias/binary) or to_dtype (cast)
  const float* inputs[TL_EPI_MAX_INPUTS];
  float alpha;
  // Pre-decoded form of the common chain [bias] [unary] [cast to the output type]: kernels
  // with many outputs per thread evaluate it without walking the op list.
  int32_t fast;           // 1 when the chain has that form (an empty chain included)
  int32_t fast_unary;     // TL_UNARY_* or 0
  const float* fast_bias; // [N] or null
};

// Validates an epilogue description and flattens it; returns TL_OK or an error
// (with the message set on ctx).
int32_t tl_make_epi(tl_ctx* ctx, const tl_epilogue* e, float alpha, EpiParams* out, bool* has_ops);

// Layout of a rank's peer-exchange buffer (tl_p2p_create): slots [2 halves][kMaxPeers][max_bytes],
// then the flags and per-CTA epochs of the stand-alone all-reduce kernel, then -- from a 256-byte
// boundary -- the words of the fused GEMV + all-reduce: tile epochs u32 [kP2PFusedMaxTiles] and
// arrival counters u32 [2 halves][kP2PFusedMaxTiles], and the fused kernel's OWN slots
// [2 halves][kMaxPeers][max_bytes] (separate from the stand-alone kernel's, so that the two may
// be mixed freely on one stream).
constexpr int kP2PFusedMaxTiles = 1024;
#ifdef __CUDACC__
__host__ __device__
#endif
inline size_t tl_p2p_fused_offset(size_t max_bytes) {
  return (2 * size_t(tl_ctx::kMaxPeers) * max_bytes + sizeof(uint32_t) * (2 * tl_ctx::kMaxPeers * 8 + 8) + 255) & ~size_t(255);
}
#ifdef __CUDACC__
__host__ __device__
#endif
inline size_t tl_p2p_fused_slots_offset(size_t max_bytes) {
  return tl_p2p_fused_offset(max_bytes) + ((sizeof(uint32_t) * 3 * kP2PFusedMaxTiles + 255) & ~size_t(255));
}
// After the fused kernel's slots: the words of the push / reduce-on-read pair (tl_qgemv_nt_push and
// the consuming launch): u32 arrive[2], done[2], epoch_p, epoch_c (256 bytes reserved), and ITS slots
// [2 halves][kMaxPeers][max_bytes].
#ifdef __CUDACC__
__host__ __device__
#endif
inline size_t tl_p2p_push_words_offset(size_t max_bytes) {
  return tl_p2p_fused_slots_offset(max_bytes) + 2 * size_t(tl_ctx::kMaxPeers) * max_bytes;
}
#ifdef __CUDACC__
__host__ __device__
#endif
inline size_t tl_p2p_push_slots_offset(size_t max_bytes) { return tl_p2p_push_words_offset(max_bytes) + 256; }
inline size_t tl_p2p_total_bytes(size_t max_bytes) {
  return tl_p2p_push_slots_offset(max_bytes) + 2 * size_t(tl_ctx::kMaxPeers) * max_bytes;
}

void tl_record_class_winner(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc& q, const tl_variant& v);
bool tl_lookup_tuned(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc& q, tl_variant* v);

// Common argument validation of the quantized entry points.
int32_t tl_check_qargs(tl_ctx* ctx, const char* who, const void* a, int32_t a_dtype,
                       const void* packed, const void* scales, const void* out, int32_t out_dtype,
                       int64_t m, int64_t n, int64_t k, const tl_quant_desc* q);

// Launchers implemented by the kernel translation units.
int32_t tl_launch_qgemv(tl_ctx* ctx, const tl_variant& v, const void* a, int32_t a_dtype,
                        const void* packed, const void* scales, void* out, int32_t out_dtype,
                        int32_t m, int64_t n, int64_t k, const tl_quant_desc& q,
                        const EpiParams& epi, tl_plan_receipt* receipt_only);
int32_t tl_launch_qgemm(tl_ctx* ctx, const tl_variant& v, const void* a, int32_t a_dtype,
                        const void* packed, const void* scales, void* out, int32_t out_dtype,
                        int64_t m, int64_t n, int64_t k, const tl_quant_desc& q,
                        const EpiParams& epi, tl_plan_receipt* receipt_only);
// int4-grouped branch of the seam (tl_int4.cu)
int32_t tl_int4_matmul(tl_ctx* ctx, const char* who, int route, const void* a, int32_t a_dtype, const void* packed, const void* scales,
                       void* out, int32_t out_dtype, int64_t m, int64_t n, int64_t k, const tl_quant_desc* q, float alpha,
                       const tl_epilogue* epilogue, tl_plan_receipt* receipt_only);
// Dense tensor-core matmul (tl_matmul_tc.cu): NT layout, both operands f16 or both bf16.
bool tl_dense_tc_applicable(const void* a, const void* b, int64_t m, int64_t n, int64_t k, int32_t dtype_a, int32_t dtype_b);
// The tile the dense tensor-core kernel would use and the modelled time of that launch: bn columns and
// mh row halves of 128 per tile, ring stages, CTAs.  forced_bn > 0 pins the tile; bn_multiple = 64 when an
// operand is multiplied MN-major.
struct TlDenseTcChoice { int bn, mh, stages, grid; double cost_us; };
TlDenseTcChoice tl_dense_tc_choose(int64_t m, int64_t n, int64_t k, int sms, int forced_bn = 0, int forced_mh = 0, int bn_multiple = 16);
int32_t tl_launch_dense_tc(tl_ctx* ctx, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int32_t dtype,
                           int32_t out_dtype, const struct EpiParams& epi, const void* colscale = nullptr,
                           int32_t colscale_dtype = 0, float colscale_mul = 1.0f, bool b_mn = false, bool a_mn = false);
bool tl_qgemv_stream_applicable(const tl_variant& v, int64_t m, int64_t k, int32_t a_dtype, const tl_quant_desc& q);
void tl_qgemv_stream_geometry(tl_ctx* ctx, const tl_variant& v, int32_t m, int64_t tiles, int64_t k, int* grid, int* block,
                              size_t* smem);
int32_t tl_launch_qgemv_stream(tl_ctx* ctx, const tl_variant& v, const void* a, int32_t a_dtype, int32_t n_items,
                               const void* const* packed, const void* const* scales, void* const* out, const int64_t* n,
                               const struct EpiParams* epi, int32_t out_dtype, int32_t m, int64_t k,
                               const tl_quant_desc& q, tl_plan_receipt* receipt_only);
int32_t tl_qgemv_default_variant(tl_ctx* ctx, int32_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q, tl_variant* out);
int32_t tl_qgemv_candidates(tl_ctx* ctx, int32_t m, int64_t n, int64_t k, int32_t a_dtype,
                            const tl_quant_desc& q, std::vector<tl_variant>* out);
int32_t tl_qgemm_default_variant(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q, tl_variant* out);
int32_t tl_qgemm_candidates(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                            const tl_quant_desc& q, std::vector<tl_variant>* out);
bool tl_variant_applicable(tl_ctx* ctx, const tl_variant& v, int64_t m, int64_t n, int64_t k,
                           int32_t a_dtype, const tl_quant_desc& q);

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------
template <typename T> struct DT;
template <> struct DT<float> {
  static constexpr int id = TL_F32;
  __device__ static float to_f32(float v) { return v; }
  __device__ static float from_f32(float v) { return v; }
};
template <> struct DT<__half> {
  static constexpr int id = TL_F16;
  __device__ static float to_f32(__half v) { return __half2float(v); }
  __device__ static __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct DT<__nv_bfloat16> {
  static constexpr int id = TL_BF16;
  __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float tl_load_scale(const void* scales, int scales_dtype, int64_t idx) {
  return scales_dtype == TL_F16 ? __half2float(reinterpret_cast<const __half*>(scales)[idx])
                                : reinterpret_cast<const float*>(scales)[idx];
}

// Activation bodies in f32: the reference's GPU path folds the same terms to
// f32 (src/backend/webgpu/fusion-tile-ir.ts:44-78); the CPU path evaluates them
// in f64 (src/ops/semantic/interpret.ts:25-98).
__device__ __forceinline__ float tl_unary(int op, float x) {
  switch (op) {
    case TL_UNARY_RELU: return x > 0.f ? x : 0.f;
    case TL_UNARY_SILU: return x / (1.f + expf(-x));
    case TL_UNARY_SIGMOID: return 1.f / (1.f + expf(-x));
    case TL_UNARY_TANH: return tanhf(x);
    case TL_UNARY_GELU_TANH:
      return (0.5f * x) * (1.f + tanhf(0.7978845608f * (x + 0.044715f * (x * (x * x)))));
    case TL_UNARY_GELU_ERF: {
      // Abramowitz-Stegun 7.1.26, the polynomial the reference uses for erf
      // (src/ops/semantic/erf.ts:28-56)
      float u = x * 0.70710678118654752f;
      float ax = fabsf(u);
      float t = 1.f / (1.f + 0.3275911f * ax);
      float poly = ((((1.061405429f * t - 1.453152027f) * t + 1.421413741f) * t - 0.284496736f) * t +
                    0.254829592f) * t;
      float er = 1.f - poly * expf(-ax * ax);
      return (0.5f * x) * (1.f + (u < 0.f ? -er : er));
    }
    default: return x;
  }
}

// Hardware-approximated bodies (tanh.approx / ex2.approx, ~2^-11 absolute on tanh): used
// only when the result is stored as f16/bf16, whose own rounding is coarser.
__device__ __forceinline__ float tl_tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tl_unary_approx(int op, float x) {
  switch (op) {
    case TL_UNARY_RELU: return x > 0.f ? x : 0.f;
    case TL_UNARY_SILU: return __fdividef(x, 1.f + __expf(-x));
    case TL_UNARY_SIGMOID: return __fdividef(1.f, 1.f + __expf(-x));
    case TL_UNARY_TANH: return tl_tanh_approx(x);
    case TL_UNARY_GELU_TANH:
      return (0.5f * x) * (1.f + tl_tanh_approx(0.7978845608f * (x + 0.044715f * (x * (x * x)))));
    default: return tl_unary(op, x);
  }
}

// v = acc (unscaled by alpha); row/col index the [M,N] output.
__device__ __forceinline__ float tl_apply_epilogue(const EpiParams& e, float v, int64_t row,
                                                   int64_t col, int64_t n) {
  v *= e.alpha;
#pragma unroll 1
  for (int i = 0; i < e.n_ops; ++i) {
    const int kind = e.kind[i];
    if (kind == TL_EPI_BIAS) {
      v += __ldg(e.inputs[e.idx[i]] + col);
    } else if (kind == TL_EPI_UNARY) {
      v = tl_unary(e.op[i], v);
    } else if (kind == TL_EPI_BINARY) {
      float o = __ldg(e.inputs[e.idx[i]] + row * n + col);
      v = e.op[i] == TL_BINARY_ADD ? v + o : e.op[i] == TL_BINARY_SUB ? v - o : v * o;
    } else if (kind == TL_EPI_CAST) {
      if (e.idx[i] == TL_F16) v = __half2float(__float2half_rn(v));
      else if (e.idx[i] == TL_BF16) v = __bfloat162float(__float2bfloat16_rn(v));
    }
  }
  return v;
}

__device__ __forceinline__ void tl_store_out(void* out, int out_dtype, int64_t idx, float v) {
  if (out_dtype == TL_F32) reinterpret_cast<float*>(out)[idx] = v;
  else if (out_dtype == TL_F16) reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}
#endif  // __CUDACC__
