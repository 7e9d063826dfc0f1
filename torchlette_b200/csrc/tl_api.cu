// Context, memory, counters, replay graphs, events, argument validation and the
// quantized-matmul seam of libtlcuda.
#include <cstdlib>
#include <cstring>

#include "tl_common.cuh"

static thread_local std::string g_last_error;  // for calls that fail without a context

int32_t tl_set_error(tl_ctx* ctx, int32_t code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) ctx->last_error = buf;
  g_last_error = buf;
  return code;
}

int32_t tl_ensure_scratch(tl_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->scratch_bytes) {
    if (ctx->capturing)
      return tl_set_error(ctx, TL_ERR_UNSUPPORTED,
                          "scratch must grow from %zu to %zu bytes during graph capture; run the "
                          "call once before capturing", ctx->scratch_bytes, bytes);
    if (ctx->scratch) {
      TL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      if (ctx->live_graphs > 0) ctx->retired_scratch.push_back({ctx->scratch, ctx->scratch_bytes});  // a captured graph may still use it
      else TL_CUDA(ctx, cudaFree(ctx->scratch));
      ctx->scratch = nullptr;
      ctx->scratch_bytes = 0;
    }
    size_t want = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
    cudaError_t e = cudaMalloc(&ctx->scratch, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return tl_set_error(ctx, TL_ERR_OOM, "scratch allocation of %zu bytes failed: %s", want,
                          cudaGetErrorString(e));
    }
    ctx->scratch_bytes = want;
  }
  *out = ctx->scratch;
  return TL_OK;
}

int32_t tl_ensure_zeroed_scratch(tl_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->zscratch_bytes) {
    if (ctx->capturing)
      return tl_set_error(ctx, TL_ERR_UNSUPPORTED,
                          "scratch must grow from %zu to %zu bytes during graph capture; run the "
                          "call once before capturing", ctx->zscratch_bytes, bytes);
    if (ctx->zscratch) {
      TL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      if (ctx->live_graphs > 0) ctx->retired_scratch.push_back({ctx->zscratch, ctx->zscratch_bytes});  // a captured graph may still use it
      else TL_CUDA(ctx, cudaFree(ctx->zscratch));
      ctx->zscratch = nullptr;
      ctx->zscratch_bytes = 0;
    }
    size_t want = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
    cudaError_t e = cudaMalloc(&ctx->zscratch, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return tl_set_error(ctx, TL_ERR_OOM, "scratch allocation of %zu bytes failed: %s", want,
                          cudaGetErrorString(e));
    }
    ctx->zscratch_bytes = want;
    TL_CUDA(ctx, cudaMemsetAsync(ctx->zscratch, 0, want, ctx->stream));
  }
  *out = ctx->zscratch;
  return TL_OK;
}

TlProfileScope::TlProfileScope(tl_ctx* c, const char* l, int64_t m_, int64_t n_, int64_t k_)
    : ctx(c), label(l), m(m_), n(n_), k(k_), on(false) {
  if (!c || !c->profile || c->capturing) return;
  DeviceGuard guard(c->device);
  if (!c->prof_e0 && (cudaEventCreate(&c->prof_e0) != cudaSuccess || cudaEventCreate(&c->prof_e1) != cudaSuccess)) return;
  on = cudaEventRecord(c->prof_e0, c->stream) == cudaSuccess;
}
TlProfileScope::~TlProfileScope() {
  if (!on) return;
  DeviceGuard guard(ctx->device);
  float ms = 0.f;
  if (cudaEventRecord(ctx->prof_e1, ctx->stream) == cudaSuccess && cudaEventSynchronize(ctx->prof_e1) == cudaSuccess &&
      cudaEventElapsedTime(&ms, ctx->prof_e0, ctx->prof_e1) == cudaSuccess)
    fprintf(stderr, "[tl profile] %s m=%lld n=%lld k=%lld: %.2f us\n", label, (long long)m, (long long)n, (long long)k, ms * 1e3);
}

extern "C" {

int32_t tl_ctx_create(int32_t device_ordinal, tl_ctx** out_ctx) {
  if (!out_ctx) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "tl_ctx_create: out_ctx is null");
  *out_ctx = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return tl_set_error(nullptr, TL_ERR_CUDA, "tl_ctx_create: no usable CUDA device: %s",
                        cudaGetErrorString(e));
  }
  if (device_ordinal < 0 || device_ordinal >= count)
    return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "tl_ctx_create: device %d out of range [0,%d)",
                        device_ordinal, count);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device_ordinal);
  if (e != cudaSuccess)
    return tl_set_error(nullptr, TL_ERR_CUDA, "tl_ctx_create: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return tl_set_error(nullptr, TL_ERR_UNSUPPORTED,
                        "tl_ctx_create: device %d is sm_%d%d; this library holds sm_100a code only",
                        device_ordinal, prop.major, prop.minor);
  tl_ctx* ctx = new tl_ctx();
  ctx->device = device_ordinal;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->l2_bytes = prop.l2CacheSize;
  DeviceGuard guard(device_ordinal);
  e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete ctx;
    return tl_set_error(nullptr, TL_ERR_CUDA, "tl_ctx_create: stream: %s", cudaGetErrorString(e));
  }
  // one small block: the status word, then (from byte 64) the eight flag words of the timed
  // weight prefetch, which start out raised ("no launch is streaming")
  const uint32_t ones[8] = {1, 1, 1, 1, 1, 1, 1, 1};
  if (cudaMalloc(&ctx->dev_status, 128) != cudaSuccess || cudaMemset(ctx->dev_status, 0, 128) != cudaSuccess ||
      cudaMemcpy(reinterpret_cast<uint8_t*>(ctx->dev_status) + 64, ones, sizeof(ones), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return tl_set_error(nullptr, TL_ERR_OOM, "tl_ctx_create: cannot allocate the device status word");
  }
  ctx->pf_flags = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(ctx->dev_status) + 64);
  // environment knobs, read once per context like the reference's ENV (src/core/env.ts:14-26):
  //   TORCHLETTE_CUDA_VARIANT=family,kernel,p0,p1,p2,p3   force one kernel variant (A/B runs without code)
  //   TORCHLETTE_CUDA_PROFILE=1                           per-call event timing on stderr
  if (const char* ev = getenv("TORCHLETTE_CUDA_VARIANT")) {
    tl_variant v{};
    if (sscanf(ev, "%d,%d,%d,%d,%d,%d", &v.family, &v.kernel, &v.p0, &v.p1, &v.p2, &v.p3) >= 2 &&
        (v.family == TL_FAMILY_QGEMV || v.family == TL_FAMILY_QGEMM || v.family == TL_FAMILY_MATMUL)) {
      ctx->forced = v;
      ctx->has_forced = true;
    } else {
      fprintf(stderr, "[tlcuda] TORCHLETTE_CUDA_VARIANT='%s' ignored: expected family,kernel[,p0,p1,p2,p3] with family 1..3\n", ev);
    }
  }
  if (const char* ev = getenv("TORCHLETTE_CUDA_PROFILE")) ctx->profile = ev[0] == '1';
  *out_ctx = ctx;
  return TL_OK;
}

int32_t tl_ctx_destroy(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  DeviceGuard guard(ctx->device);
  if (ctx->nccl_comm) tl_comm_destroy(ctx);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->zscratch) cudaFree(ctx->zscratch);
  for (auto& p : ctx->retired_scratch) cudaFree(p.first);
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  if (ctx->stream_scratch) cudaFree(ctx->stream_scratch);
  if (ctx->prof_e0) { cudaEventDestroy(ctx->prof_e0); cudaEventDestroy(ctx->prof_e1); }
  for (int r = 0; r < tl_ctx::kMaxPeers; ++r)
    if (ctx->p2p_peer[r] && ctx->p2p_peer[r] != ctx->p2p_local) cudaIpcCloseMemHandle(ctx->p2p_peer[r]);
  if (ctx->p2p_local) cudaFree(ctx->p2p_local);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return TL_OK;
}

int32_t tl_sync(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  int status = 0;
  TL_CUDA(ctx, cudaMemcpy(&status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (status != 0) {
    // a bounded device-side wait ran out: the scratch may hold partial sums, so clear it
    cudaMemset(ctx->dev_status, 0, sizeof(int));
    if (ctx->zscratch) cudaMemset(ctx->zscratch, 0, ctx->zscratch_bytes);
    for (auto& p : ctx->retired_scratch) cudaMemset(p.first, 0, p.second);  // older graphs' meeting points too
    if (ctx->stream_scratch) cudaMemset(ctx->stream_scratch, 0, size_t(ctx->sm_count) * (2 * 2 * 128 * sizeof(float) + sizeof(unsigned)));
    ctx->async_errors++;
    return tl_set_error(ctx, TL_ERR_TIMEOUT, "tl_sync: a kernel gave up a bounded wait (device code %d)", status);
  }
  return TL_OK;
}

int64_t tl_async_error_count(tl_ctx* ctx) { return ctx ? ctx->async_errors : -1; }

const char* tl_last_error(tl_ctx* ctx) { return ctx ? ctx->last_error.c_str() : g_last_error.c_str(); }

int32_t tl_ctx_stream(tl_ctx* ctx, void** out_stream) {
  TL_CHECK_CTX(ctx);
  if (!out_stream) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_ctx_stream: null out pointer");
  *out_stream = (void*)ctx->stream;
  return TL_OK;
}

int32_t tl_device_sm_count(tl_ctx* ctx, int32_t* out_sms) {
  TL_CHECK_CTX(ctx);
  if (!out_sms) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_device_sm_count: null out pointer");
  *out_sms = ctx->sm_count;
  return TL_OK;
}

int32_t tl_set_option(tl_ctx* ctx, const char* name, int64_t value) {
  TL_CHECK_CTX(ctx);
  if (!name) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_set_option: null name");
  if (!strcmp(name, "wait_limit_polls")) {
    if (value < 1 || value > (int64_t(1) << 30))
      return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_set_option: wait_limit_polls outside [1, 2^30]");
    ctx->wait_limit_polls = int(value);
  } else if (!strcmp(name, "push_poll_ranks")) {
    if (value < 1 || value > 4) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_set_option: push_poll_ranks outside [1, 4]");
    ctx->push_poll_ranks = int(value);
  } else {
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_set_option: unknown option '%s'", name);
  }
  return TL_OK;
}

int32_t tl_get_option(tl_ctx* ctx, const char* name, int64_t* out_value) {
  TL_CHECK_CTX(ctx);
  if (!name || !out_value) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_get_option: null argument");
  if (!strcmp(name, "wait_limit_polls")) *out_value = ctx->wait_limit_polls;
  else if (!strcmp(name, "push_poll_ranks")) *out_value = ctx->push_poll_ranks;
  else if (!strcmp(name, "p2p_buffer_address")) *out_value = int64_t(reinterpret_cast<uintptr_t>(ctx->p2p_local));
  else if (!strcmp(name, "p2p_slot_bytes")) *out_value = int64_t(ctx->p2p_max_bytes);
  else return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_get_option: unknown option '%s'", name);
  return TL_OK;
}

// ---- memory ---------------------------------------------------------------
int32_t tl_alloc(tl_ctx* ctx, size_t bytes, void** out_dptr) {
  TL_CHECK_CTX(ctx);
  if (!out_dptr) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_alloc: null out pointer");
  *out_dptr = nullptr;
  DeviceGuard guard(ctx->device);
  cudaError_t e = cudaMalloc(out_dptr, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return tl_set_error(ctx, e == cudaErrorMemoryAllocation ? TL_ERR_OOM : TL_ERR_CUDA,
                        "tl_alloc(%zu): %s", bytes, cudaGetErrorString(e));
  }
  return TL_OK;
}

int32_t tl_free(tl_ctx* ctx, void* dptr) {
  TL_CHECK_CTX(ctx);
  if (!dptr) return TL_OK;
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  TL_CUDA(ctx, cudaFree(dptr));
  return TL_OK;
}

int32_t tl_upload(tl_ctx* ctx, void* dst, const void* src, size_t bytes) {
  TL_CHECK_CTX(ctx);
  if (bytes == 0) return TL_OK;
  if (!dst || !src) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_upload: null pointer");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return TL_OK;
}

int32_t tl_download(tl_ctx* ctx, void* dst, const void* src, size_t bytes) {
  TL_CHECK_CTX(ctx);
  if (bytes == 0) return TL_OK;
  if (!dst || !src) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_download: null pointer");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return TL_OK;
}

int32_t tl_host_alloc_pinned(tl_ctx* ctx, size_t bytes, void** out_hptr) {
  TL_CHECK_CTX(ctx);
  if (!out_hptr) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_host_alloc_pinned: null out pointer");
  DeviceGuard guard(ctx->device);
  cudaError_t e = cudaHostAlloc(out_hptr, bytes ? bytes : 1, cudaHostAllocDefault);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return tl_set_error(ctx, TL_ERR_OOM, "tl_host_alloc_pinned(%zu): %s", bytes, cudaGetErrorString(e));
  }
  return TL_OK;
}

int32_t tl_host_free_pinned(tl_ctx* ctx, void* hptr) {
  TL_CHECK_CTX(ctx);
  if (!hptr) return TL_OK;
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaFreeHost(hptr));
  return TL_OK;
}

int32_t tl_memset(tl_ctx* ctx, void* dptr, int32_t byte_value, size_t bytes) {
  TL_CHECK_CTX(ctx);
  if (bytes == 0) return TL_OK;
  if (!dptr) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_memset: null pointer");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaMemsetAsync(dptr, byte_value, bytes, ctx->stream));
  return TL_OK;
}

int32_t tl_copy2d(tl_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                  size_t height) {
  TL_CHECK_CTX(ctx);
  if (width_bytes == 0 || height == 0) return TL_OK;
  if (!dst || !src) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_copy2d: null pointer");
  if (dst_pitch < width_bytes || src_pitch < width_bytes)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_copy2d: pitch smaller than the row width");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, height, cudaMemcpyDeviceToDevice,
                                 ctx->stream));
  return TL_OK;
}

// ---- counters -------------------------------------------------------------
int64_t tl_counter_get(tl_ctx* ctx, int32_t which) {
  if (!ctx || which < 0 || which >= TL_COUNTER_COUNT) return -1;
  return ctx->counters[which];
}

int32_t tl_counters_reset(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  for (int i = 0; i < TL_COUNTER_COUNT; ++i) ctx->counters[i] = 0;
  return TL_OK;
}

// ---- replay graphs ----------------------------------------------------------
struct tl_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int64_t counter_delta[TL_COUNTER_COUNT] = {0, 0, 0, 0, 0};
};

static thread_local int64_t g_capture_base[TL_COUNTER_COUNT];

int32_t tl_graph_begin(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  if (ctx->capturing) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_graph_begin: already capturing");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->capturing = true;
  for (int i = 0; i < TL_COUNTER_COUNT; ++i) g_capture_base[i] = ctx->counters[i];
  return TL_OK;
}

int32_t tl_graph_end(tl_ctx* ctx, tl_graph** out_graph) {
  TL_CHECK_CTX(ctx);
  if (!ctx->capturing) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_graph_end: not capturing");
  if (!out_graph) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_graph_end: null out pointer");
  DeviceGuard guard(ctx->device);
  ctx->capturing = false;
  tl_graph* g = new tl_graph();
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
  if (e != cudaSuccess || !g->graph) {
    delete g;
    cudaGetLastError();
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_graph_end: capture failed: %s", cudaGetErrorString(e));
  }
  e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(g->graph);
    delete g;
    cudaGetLastError();
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_graph_end: instantiate failed: %s", cudaGetErrorString(e));
  }
  // Replays bump the route counters by what the captured calls bumped, so the
  // counters keep meaning "dispatches that ran" under replay.
  for (int i = 0; i < TL_COUNTER_COUNT; ++i) {
    g->counter_delta[i] = ctx->counters[i] - g_capture_base[i];
    ctx->counters[i] = g_capture_base[i];
  }
  *out_graph = g;
  ctx->live_graphs++;
  return TL_OK;
}

int32_t tl_graph_launch(tl_ctx* ctx, tl_graph* graph) {
  TL_CHECK_CTX(ctx);
  if (!graph || !graph->exec) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_graph_launch: null graph");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaGraphLaunch(graph->exec, ctx->stream));
  for (int i = 0; i < TL_COUNTER_COUNT; ++i) ctx->counters[i] += graph->counter_delta[i];
  return TL_OK;
}

int32_t tl_graph_destroy(tl_ctx* ctx, tl_graph* graph) {
  TL_CHECK_CTX(ctx);
  if (!graph) return TL_OK;
  DeviceGuard guard(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (graph->exec) cudaGraphExecDestroy(graph->exec);
  if (graph->graph) cudaGraphDestroy(graph->graph);
  delete graph;
  if (ctx->live_graphs > 0 && --ctx->live_graphs == 0) {
    for (auto& p : ctx->retired_scratch) cudaFree(p.first);  // no graph can reference them any more
    ctx->retired_scratch.clear();
  }
  return TL_OK;
}

// ---- events -----------------------------------------------------------------
struct tl_event {
  cudaEvent_t ev = nullptr;
};

int32_t tl_event_create(tl_ctx* ctx, tl_event** out_event) {
  TL_CHECK_CTX(ctx);
  if (!out_event) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_event_create: null out pointer");
  DeviceGuard guard(ctx->device);
  tl_event* e = new tl_event();
  cudaError_t err = cudaEventCreate(&e->ev);
  if (err != cudaSuccess) {
    delete e;
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_event_create: %s", cudaGetErrorString(err));
  }
  *out_event = e;
  return TL_OK;
}

int32_t tl_event_record(tl_ctx* ctx, tl_event* ev) {
  TL_CHECK_CTX(ctx);
  if (!ev) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_event_record: null event");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaEventRecord(ev->ev, ctx->stream));
  return TL_OK;
}

int32_t tl_event_elapsed_ms(tl_ctx* ctx, tl_event* start, tl_event* stop, float* out_ms) {
  TL_CHECK_CTX(ctx);
  if (!start || !stop || !out_ms) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_event_elapsed_ms: null argument");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaEventSynchronize(stop->ev));
  TL_CUDA(ctx, cudaEventElapsedTime(out_ms, start->ev, stop->ev));
  return TL_OK;
}

// Host-side wait for one recorded event.  Reads nothing of the context but its device ordinal
// and writes nothing to it (no error text), so a worker thread may call it while the thread
// that owns the context keeps enqueueing work.
int32_t tl_event_synchronize(tl_ctx* ctx, tl_event* ev) {
  if (!ctx || !ev) return TL_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  return cudaEventSynchronize(ev->ev) == cudaSuccess ? TL_OK : TL_ERR_CUDA;
}

int32_t tl_event_destroy(tl_ctx* ctx, tl_event* ev) {
  TL_CHECK_CTX(ctx);
  if (!ev) return TL_OK;
  DeviceGuard guard(ctx->device);
  cudaEventDestroy(ev->ev);
  delete ev;
  return TL_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Argument validation shared by the quantized entry points.  The messages
// follow the reference's thrown errors (src/backend/webgpu/ops/matmul-ops.ts:
// 121-126; src/backend/webgpu/matmul/dispatch.ts:890-892, 960-962;
// src/backend/quantize.ts:88-93).
// ---------------------------------------------------------------------------
int32_t tl_check_qargs(tl_ctx* ctx, const char* who, const void* a, int32_t a_dtype,
                       const void* packed, const void* scales, const void* out, int32_t out_dtype,
                       int64_t m, int64_t n, int64_t k, const tl_quant_desc* q) {
  if (!q) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: missing packing descriptor on B operand", who);
  if (q->scheme != TL_SCHEME_INT8_GROUPED)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "%s: unsupported scheme %d", who, q->scheme);
  if (!packed) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: null packed weight", who);
  if (!scales) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: missing packing/scales on B operand", who);
  if (!out) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: null output", who);
  if (m < 0 || n < 0 || k < 0)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: negative dimension m=%lld n=%lld k=%lld", who,
                        (long long)m, (long long)n, (long long)k);
  if (m > 0 && !a) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: null activation", who);
  if (k % 4 != 0) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: K=%lld must be divisible by 4", who, (long long)k);
  if (q->group_size <= 0 || (k > 0 && k % q->group_size != 0))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: K=%lld must be divisible by groupSize=%d", who,
                        (long long)k, q->group_size);
  if (q->scales_dtype != TL_F16 && q->scales_dtype != TL_F32)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: scales dtype must be f16 or f32", who);
  if (q->scale_convention != TL_SCALE_SNORM127 && q->scale_convention != TL_SCALE_DIRECT)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: unknown scale convention %d", who, q->scale_convention);
  if (!tl_dtype_valid(a_dtype) || !tl_dtype_valid(out_dtype))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: unknown dtype", who);
  if (n > 0x7fffffffLL || k > 0x7fffffffLL)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "%s: N and K must fit in 31 bits", who);
  if ((reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(scales) & (tl_dtype_size(q->scales_dtype) - 1)))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: misaligned weight or scales pointer", who);
  if ((reinterpret_cast<uintptr_t>(a) & (tl_dtype_size(a_dtype) - 1)) || (reinterpret_cast<uintptr_t>(out) & (tl_dtype_size(out_dtype) - 1)))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: misaligned activation or output pointer", who);
  return TL_OK;
}

int32_t tl_make_epi(tl_ctx* ctx, const tl_epilogue* e, float alpha, EpiParams* out, bool* has_ops) {
  memset(out, 0, sizeof(*out));
  out->alpha = alpha;
  out->fast = 1;
  *has_ops = false;
  if (!e) return TL_OK;
  if (e->n_ops < 0 || e->n_ops > TL_EPI_MAX_OPS)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "epilogue: n_ops=%d out of range [0,%d]", e->n_ops, TL_EPI_MAX_OPS);
  if (e->n_inputs < 0 || e->n_inputs > TL_EPI_MAX_INPUTS)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "epilogue: at most %d extra inputs (got %d)", TL_EPI_MAX_INPUTS, e->n_inputs);
  for (int i = 0; i < e->n_inputs; ++i) {
    if (!e->inputs[i]) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "epilogue: input %d is null", i);
    if (reinterpret_cast<uintptr_t>(e->inputs[i]) & 3)
      return tl_set_error(ctx, TL_ERR_INVALID_ARG, "epilogue: input %d is not 4-byte aligned", i);
    out->inputs[i] = reinterpret_cast<const float*>(e->inputs[i]);
  }
  int n = 0;
  for (int i = 0; i < e->n_ops; ++i) {
    const tl_epilogue_op& op = e->ops[i];
    switch (op.kind) {
      case TL_EPI_NONE: continue;
      case TL_EPI_BIAS:
      case TL_EPI_BINARY:
        if (op.input_index < 0 || op.input_index >= e->n_inputs)
          return tl_set_error(ctx, TL_ERR_INVALID_ARG, "epilogue: op %d reads input %d but only %d inputs were given", i, op.input_index, e->n_inputs);
        if (op.kind == TL_EPI_BINARY && (op.op < TL_BINARY_ADD || op.op > TL_BINARY_MUL))
          return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "epilogue: unsupported binary op %d", op.op);
        out->idx[n] = op.input_index;
        break;
      case TL_EPI_UNARY:
        if (op.op < TL_UNARY_RELU || op.op > TL_UNARY_GELU_ERF)
          return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "epilogue: unsupported unary op %d", op.op);
        break;
      case TL_EPI_CAST:
        if (!tl_dtype_valid(op.to_dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "epilogue: cast to unknown dtype %d", op.to_dtype);
        out->idx[n] = op.to_dtype;
        break;
      default:
        return tl_set_error(ctx, TL_ERR_INVALID_ARG, "epilogue: unknown op kind %d", op.kind);
    }
    out->kind[n] = op.kind;
    out->op[n] = op.op;
    ++n;
  }
  out->n_ops = n;
  *has_ops = n > 0;
  // recognise [bias] [unary] [cast]* (a trailing cast is repeated by the store, so only
  // a cast to a type the store keeps exactly may be dropped: leave chains with casts generic
  // unless the cast is last)
  {
    int i = 0;
    out->fast = 1;
    out->fast_unary = 0;
    out->fast_bias = nullptr;
    if (i < n && out->kind[i] == TL_EPI_BIAS) out->fast_bias = out->inputs[out->idx[i++]];
    if (i < n && out->kind[i] == TL_EPI_UNARY) out->fast_unary = out->op[i++];
    if (i != n) out->fast = 0;
  }
  return TL_OK;
}

// ---------------------------------------------------------------------------
// Shape classes (classifyShape, src/backend/webgpu/matmul/types.ts:146-200)
// ---------------------------------------------------------------------------
extern "C" int32_t tl_classify_shape(int64_t m, int64_t n, int64_t k, int64_t batch) {
  if (m == 1 && n > 1) return TL_SHAPE_GEMV_ROW;
  if (m == 1 || n == 1) return TL_SHAPE_GEMV;
  if (batch > 1 && m * n < 512 * 512) return TL_SHAPE_BATCHED_SMALL;
  if (k < 64 && m * n > 100000) return TL_SHAPE_SMALL_K;
  if (double(k) / double(std::max(m, n)) > 4.0) return TL_SHAPE_LARGE_K;
  if (double(m) / double(std::max(k, n)) > 4.0) return TL_SHAPE_TALL_SKINNY;
  if (double(n) / double(std::max(k, m)) > 4.0) return TL_SHAPE_SHORT_WIDE;
  const int64_t mx = std::max(m, std::max(n, k));
  return mx < 512 ? TL_SHAPE_SQUARE_SMALL : mx < 2048 ? TL_SHAPE_SQUARE_MEDIUM : TL_SHAPE_SQUARE_LARGE;
}

extern "C" const char* tl_shape_class_name(int32_t cls) {
  static const char* const names[] = {"square_small", "square_medium", "square_large", "tall_skinny", "short_wide",
                                      "large_k", "small_k", "gemv", "gemv_row", "batched_small"};
  return cls >= 0 && cls < int(sizeof(names) / sizeof(names[0])) ? names[cls] : "?";
}

// ---------------------------------------------------------------------------
// Selection + the seam
// ---------------------------------------------------------------------------
static TuneKey make_key(int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc& q) {
  return TuneKey{m, n, k, a_dtype, q.group_size, q.scales_dtype, q.scale_convention};
}

// The tuned winner recorded for a shape, if any (the batched launch keys on the summed N).
bool tl_lookup_tuned(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc& q, tl_variant* v) {
  auto it = ctx->tuned.find(make_key(m, n, k, a_dtype, q));
  if (it == ctx->tuned.end()) return false;
  *v = it->second;
  return true;
}

static TuneKey make_class_key(int fam, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc& q) {
  return TuneKey{tl_classify_shape(m, n, k, 1), fam, 0, a_dtype, q.group_size == k ? 0 : q.group_size, q.scales_dtype,
                 q.scale_convention};
}

// A tuned winner also becomes its shape class's entry (the last shape tuned in a class wins), the
// analogue of the reference's tuningCache keyed `${shapeClass}_${dtype}_...`
// (src/backend/webgpu/matmul/dispatch.ts:146-160, autotune.ts:276-300).
void tl_record_class_winner(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc& q, const tl_variant& v) {
  ctx->class_tuned[make_class_key(v.family, m, n, k, a_dtype, q)] = v;
}

// Order of precedence follows selectMatmulChoice
// (src/backend/webgpu/matmul/dispatch.ts:171-192): explicit (forced) variant ->
// per-shape tuned winner (re-gated on applicability) -> the shape class's tuned winner
// (re-gated too) -> heuristic default.  *from_cache: 0 none, 1 exact shape, 2 shape class.
static int32_t select_variant(tl_ctx* ctx, bool gemv, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                              const tl_quant_desc& q, tl_variant* v, int* from_cache) {
  *from_cache = 0;
  const int fam = gemv ? TL_FAMILY_QGEMV : TL_FAMILY_QGEMM;
  if (ctx->has_forced && ctx->forced.family == fam) {
    if (!tl_variant_applicable(ctx, ctx->forced, m, n, k, a_dtype, q))
      return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "forced variant %s cannot run m=%lld n=%lld k=%lld G=%d %s",
                          tl_variant_name(&ctx->forced), (long long)m, (long long)n, (long long)k,
                          q.group_size, tl_dtype_name(a_dtype));
    *v = ctx->forced;
    return TL_OK;
  }
  auto it = ctx->tuned.find(make_key(m, n, k, a_dtype, q));
  if (it != ctx->tuned.end() && it->second.family == fam &&
      tl_variant_applicable(ctx, it->second, m, n, k, a_dtype, q)) {
    *v = it->second;
    *from_cache = 1;
    return TL_OK;
  }
  auto ct = ctx->class_tuned.find(make_class_key(fam, m, n, k, a_dtype, q));
  if (ct != ctx->class_tuned.end() && tl_variant_applicable(ctx, ct->second, m, n, k, a_dtype, q)) {
    *v = ct->second;
    *from_cache = 2;
    return TL_OK;
  }
  return gemv ? tl_qgemv_default_variant(ctx, (int32_t)m, n, k, a_dtype, q, v)
              : tl_qgemm_default_variant(ctx, m, n, k, a_dtype, q, v);
}

static int32_t qmatmul_impl(tl_ctx* ctx, const char* who, int route /*0 auto,1 gemv,2 gemm*/, const void* a,
                            int32_t a_dtype, const void* packed, const void* scales, void* out,
                            int32_t out_dtype, int64_t m, int64_t n, int64_t k, const tl_quant_desc* qdesc,
                            float alpha, const tl_epilogue* epilogue, tl_plan_receipt* receipt_only) {
  TL_CHECK_CTX(ctx);
  if (qdesc && qdesc->scheme == TL_SCHEME_INT4_GROUPED)  // the second value on the format axis: its own kernels
    return tl_int4_matmul(ctx, who, route, a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc, alpha, epilogue, receipt_only);
  int32_t rc = tl_check_qargs(ctx, who, receipt_only ? (const void*)16 : a, a_dtype,
                              receipt_only ? (const void*)16 : packed, receipt_only ? (const void*)16 : scales,
                              receipt_only ? (const void*)16 : out, out_dtype, m, n, k, qdesc);
  if (rc != TL_OK) return rc;
  EpiParams epi;
  bool has_ops = false;
  rc = tl_make_epi(ctx, epilogue, alpha, &epi, &has_ops);
  if (rc != TL_OK) return rc;
  bool gemv = route == 1 || (route == 0 && m <= 16);
  if (route == 1 && (m < 1 || m > 16))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: m=%lld outside the GEMV range [1,16]", who, (long long)m);
  if (m == 0 || n == 0) {
    if (receipt_only) memset(receipt_only, 0, sizeof(*receipt_only));
    return TL_OK;  // empty output: nothing to launch
  }
  DeviceGuard guard(ctx->device);
  tl_variant v;
  int from_cache = 0;
  rc = select_variant(ctx, gemv, m, n, k, a_dtype, *qdesc, &v, &from_cache);
  if (rc != TL_OK) return rc;
  if (receipt_only) {
    memset(receipt_only, 0, sizeof(*receipt_only));
    receipt_only->from_tuning_cache = from_cache;
    receipt_only->epilogue_engaged = has_ops ? 1 : 0;
  }
  if (gemv) {
    rc = tl_launch_qgemv(ctx, v, a, a_dtype, packed, scales, out, out_dtype, (int32_t)m, n, k, *qdesc, epi,
                         receipt_only);
    if (rc == TL_OK && !receipt_only) {
      ctx->counters[TL_COUNTER_QGEMV]++;
      if (has_ops) ctx->counters[TL_COUNTER_QGEMV_EPILOGUE]++;
    }
  } else {
    rc = tl_launch_qgemm(ctx, v, a, a_dtype, packed, scales, out, out_dtype, m, n, k, *qdesc, epi,
                         receipt_only);
    if (rc == TL_OK && !receipt_only) ctx->counters[TL_COUNTER_QGEMM]++;
  }
  return rc;
}

extern "C" {

int32_t tl_qgemv_nt(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed, const void* scales,
                    void* out, int32_t out_dtype, int32_t m, int64_t n, int64_t k,
                    const tl_quant_desc* qdesc, float alpha, const tl_epilogue* epilogue) {
  TlProfileScope prof(ctx, "matmul_gemv_q8", m, n, k);  // the reference's label for this route (matmul/dispatch.ts:928)
  return qmatmul_impl(ctx, "tl_qgemv_nt", 1, a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc,
                      alpha, epilogue, nullptr);
}

int32_t tl_qgemm_nt(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed, const void* scales,
                    void* out, int32_t out_dtype, int64_t m, int64_t n, int64_t k,
                    const tl_quant_desc* qdesc, float alpha, const tl_epilogue* epilogue) {
  TlProfileScope prof(ctx, "matmul_gemm_q8", m, n, k);
  return qmatmul_impl(ctx, "tl_qgemm_nt", 2, a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc,
                      alpha, epilogue, nullptr);
}

int32_t tl_qmatmul_nt(tl_ctx* ctx, const void* a, int32_t a_dtype, const void* packed, const void* scales,
                      void* out, int32_t out_dtype, int64_t m, int64_t n, int64_t k,
                      const tl_quant_desc* qdesc, float alpha, const tl_epilogue* epilogue) {
  TlProfileScope prof(ctx, m <= 16 ? "matmul_gemv_q8" : "matmul_gemm_q8", m, n, k);
  return qmatmul_impl(ctx, "tl_qmatmul_nt", 0, a, a_dtype, packed, scales, out, out_dtype, m, n, k, qdesc,
                      alpha, epilogue, nullptr);
}

int32_t tl_plan_qmatmul(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, int32_t out_dtype,
                        const tl_quant_desc* qdesc, const tl_epilogue* epilogue,
                        tl_plan_receipt* out_receipt) {
  TL_CHECK_CTX(ctx);
  if (!out_receipt) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_plan_qmatmul: null receipt");
  return qmatmul_impl(ctx, "tl_plan_qmatmul", 0, nullptr, a_dtype, nullptr, nullptr, nullptr, out_dtype, m, n,
                      k, qdesc, 1.0f, epilogue, out_receipt);
}

int32_t tl_force_variant(tl_ctx* ctx, const tl_variant* v) {
  TL_CHECK_CTX(ctx);
  if (!v) {
    ctx->has_forced = false;
    return TL_OK;
  }
  if (v->family != TL_FAMILY_QGEMV && v->family != TL_FAMILY_QGEMM && v->family != TL_FAMILY_MATMUL)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_force_variant: unknown family %d", v->family);
  ctx->forced = *v;
  ctx->has_forced = true;
  return TL_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Tensor-map encoding through the driver entry point (no libcuda link).
// ---------------------------------------------------------------------------
#include "tl_tma.cuh"

typedef CUresult (*TlEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool tl_encode_tmap_2d(CUtensorMap* map, int elem_bytes, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle) {
  static TlEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) {
      cudaGetLastError();
      return false;
    }
    fn = reinterpret_cast<TlEncodeTiledFn>(p);
  }
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                   : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                               : CU_TENSOR_MAP_SWIZZLE_NONE;
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
