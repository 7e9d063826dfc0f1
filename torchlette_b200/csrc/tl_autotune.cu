// Variant registry glue and the autotuner, re-targeted from WGSL tile configs to
// the CUDA kernel variants.  Keeps the reference's semantics
// (src/backend/webgpu/matmul/dispatch.ts:405-578, autotune.ts:309-329):
//   - candidates come from the variant that is applicable to the shape, the
//     heuristic default always among them;
//   - 2 warm-up + 3 timed runs per candidate, median, fastest wins;
//   - the winner is cached per exact (m,n,k,dtype,format); a cache hit never
//     re-runs the search; a search bumps the run counter once per new shape;
//   - a cached winner is re-gated on applicability at selection time;
//   - the cache exports to / imports from JSON text; invalid JSON is rejected
//     without touching the cache.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "tl_common.cuh"

bool tl_qgemv_variant_applicable(const tl_variant& v, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q);
bool tl_qgemm_variant_applicable(const tl_variant& v, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q);

bool tl_variant_applicable(tl_ctx* ctx, const tl_variant& v, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                           const tl_quant_desc& q) {
  (void)ctx;
  if (v.family == TL_FAMILY_QGEMV) return tl_qgemv_variant_applicable(v, m, n, k, a_dtype, q);
  if (v.family == TL_FAMILY_QGEMM) return tl_qgemm_variant_applicable(v, m, n, k, a_dtype, q);
  return false;
}

extern "C" {

const char* tl_variant_name(const tl_variant* v) {
  static thread_local char buf[96];
  if (!v) return "(null)";
  const char* fam = v->family == TL_FAMILY_QGEMV ? "qgemv" : v->family == TL_FAMILY_QGEMM ? "qgemm" : v->family == TL_FAMILY_MATMUL ? "matmul" : "?";
  const char* kern = "?";
  if (v->family == TL_FAMILY_QGEMV) kern = v->kernel == 0 ? "scalar" : v->kernel == 1 ? "simt" : v->kernel == 2 ? "mma" : v->kernel == 3 ? "sk" : v->kernel == 4 ? "ring" : v->kernel == 5 ? "tma" : v->kernel == 6 ? "bulk" : v->kernel == 7 ? "chain" : v->kernel == 8 ? "stream" : v->kernel == 9 ? "int4" : "?";
  if (v->family == TL_FAMILY_QGEMM) kern = v->kernel == 0 ? "tcgen05" : v->kernel == 1 ? "sliced" : v->kernel == 2 ? "dequant+dense" : "?";
  if (v->family == TL_FAMILY_MATMUL) kern = v->kernel == 0 ? "tiled" : v->kernel == 1 ? "gemv" : v->kernel == 2 ? "tc" : "?";
  snprintf(buf, sizeof(buf), "%s.%s[%d,%d,%d,%d]", fam, kern, v->p0, v->p1, v->p2, v->p3);
  return buf;
}

int32_t tl_autotune_set_enabled(tl_ctx* ctx, int32_t enabled) {
  TL_CHECK_CTX(ctx);
  ctx->autotune_enabled = enabled != 0;
  return TL_OK;
}

int32_t tl_autotune_is_enabled(tl_ctx* ctx) { return ctx && ctx->autotune_enabled ? 1 : 0; }

int32_t tl_tune_seed(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc* q,
                     const tl_variant* choice) {
  TL_CHECK_CTX(ctx);
  if (!q || !choice) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_tune_seed: null argument");
  ctx->tuned[TuneKey{m, n, k, a_dtype, q->group_size, q->scales_dtype, q->scale_convention}] = *choice;
  return TL_OK;
}

int32_t tl_tune_get(tl_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t a_dtype, const tl_quant_desc* q,
                    tl_variant* out_choice) {
  TL_CHECK_CTX(ctx);
  if (!q) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_tune_get: null descriptor");
  auto it = ctx->tuned.find(TuneKey{m, n, k, a_dtype, q->group_size, q->scales_dtype, q->scale_convention});
  if (it == ctx->tuned.end()) return 0;
  if (out_choice) *out_choice = it->second;
  return 1;
}

int32_t tl_tune_clear(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  ctx->tuned.clear();
  ctx->class_tuned.clear();
  return TL_OK;
}

int64_t tl_tune_run_count(tl_ctx* ctx) { return ctx ? ctx->tune_runs : -1; }

int32_t tl_pretune(tl_ctx* ctx, const tl_shape* shapes, int32_t n_shapes, int32_t a_dtype, int32_t out_dtype,
                   const tl_quant_desc* q) {
  TL_CHECK_CTX(ctx);
  if (n_shapes < 0 || (n_shapes > 0 && !shapes) || !q)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_pretune: null argument");
  if (ctx->capturing) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_pretune: not allowed during graph capture");
  // pretuneMatmulShapes returns at once unless autotuning was switched on, by setAutotuneEnabled(true)
  // or by TORCHLETTE_AUTOTUNE=1 (src/backend/webgpu/matmul/dispatch.ts:557-562)
  const char* env = std::getenv("TORCHLETTE_AUTOTUNE");
  if (!ctx->autotune_enabled && !(env && env[0] == '1')) return TL_OK;
  DeviceGuard guard(ctx->device);
  const bool debug = std::getenv("TORCHLETTE_DEBUG_AUTOTUNE") != nullptr;
  for (int32_t si = 0; si < n_shapes; ++si) {
    const int64_t m = shapes[si].m, n = shapes[si].n, k = shapes[si].k;
    int32_t rc = tl_check_qargs(ctx, "tl_pretune", (const void*)16, a_dtype, (const void*)16, (const void*)16,
                                (const void*)16, out_dtype, m, n, k, q);
    if (rc != TL_OK) return rc;
    if (m == 0 || n == 0 || k == 0) continue;
    const TuneKey key{m, n, k, a_dtype, q->group_size, q->scales_dtype, q->scale_convention};
    if (ctx->tuned.count(key)) continue;  // cache hit: no search, no counter bump
    const bool gemv = m <= 16;
    std::vector<tl_variant> cands;
    if (gemv) tl_qgemv_candidates(ctx, int32_t(m), n, k, a_dtype, *q, &cands);
    else tl_qgemm_candidates(ctx, m, n, k, a_dtype, *q, &cands);
    if (cands.empty()) continue;
    // rotate over enough weight copies that every timed run streams from HBM
    const size_t wbytes = size_t(n) * k;
    const size_t sbytes = size_t(n) * (k / q->group_size) * tl_dtype_size(q->scales_dtype);
    const size_t l2 = size_t(ctx->l2_bytes > 0 ? ctx->l2_bytes : (128 << 20));
    int copies = int(std::min<size_t>(8, std::max<size_t>(1, (2 * l2 + wbytes - 1) / wbytes)));
    void *w = nullptr, *s = nullptr, *a = nullptr, *o = nullptr;
    const size_t abytes = size_t(m) * k * tl_dtype_size(a_dtype), obytes = size_t(m) * n * tl_dtype_size(out_dtype);
    auto cleanup = [&]() {
      cudaFree(w); cudaFree(s); cudaFree(a); cudaFree(o);
    };
    if (cudaMalloc(&w, wbytes * copies) != cudaSuccess || cudaMalloc(&s, sbytes * copies) != cudaSuccess ||
        cudaMalloc(&a, abytes) != cudaSuccess || cudaMalloc(&o, obytes) != cudaSuccess) {
      cudaGetLastError();
      cleanup();
      return tl_set_error(ctx, TL_ERR_OOM, "tl_pretune: cannot allocate bench buffers for %lldx%lldx%lld",
                          (long long)m, (long long)n, (long long)k);
    }
    cudaMemsetAsync(w, 0x11, wbytes * copies, ctx->stream);
    cudaMemsetAsync(s, 0, sbytes * copies, ctx->stream);
    cudaMemsetAsync(a, 0, abytes, ctx->stream);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    EpiParams epi;
    bool has_ops;
    tl_make_epi(ctx, nullptr, 1.0f, &epi, &has_ops);
    double best_ms = 1e30;
    tl_variant best = cands[0];
    bool any = false;
    const int64_t saved_launches = ctx->counters[TL_COUNTER_KERNEL_LAUNCHES];
    for (const tl_variant& v : cands) {
      std::vector<float> times;
      bool ok = true;
      for (int rep = 0; rep < 5 && ok; ++rep) {  // 2 warm-up + 3 timed
        cudaEventRecord(e0, ctx->stream);
        for (int c = 0; c < copies && ok; ++c) {
          const void* wp = (const uint8_t*)w + size_t(c) * wbytes;
          const void* sp = (const uint8_t*)s + size_t(c) * sbytes;
          int32_t r = gemv ? tl_launch_qgemv(ctx, v, a, a_dtype, wp, sp, o, out_dtype, int32_t(m), n, k, *q, epi, nullptr)
                           : tl_launch_qgemm(ctx, v, a, a_dtype, wp, sp, o, out_dtype, m, n, k, *q, epi, nullptr);
          ok = r == TL_OK;
        }
        cudaEventRecord(e1, ctx->stream);
        if (cudaEventSynchronize(e1) != cudaSuccess) ok = false;
        float ms = 0.f;
        if (ok) cudaEventElapsedTime(&ms, e0, e1);
        if (ok && rep >= 2) times.push_back(ms / copies);
      }
      if (!ok || times.empty()) continue;  // a failing candidate is skipped (all-fail -> default)
      std::sort(times.begin(), times.end());
      const double med = times[times.size() / 2];
      if (debug)
        fprintf(stderr, "[tl autotune] %lldx%lldx%lld %s: %.3f us\n", (long long)m, (long long)n, (long long)k,
                tl_variant_name(&v), med * 1e3);
      if (med < best_ms) { best_ms = med; best = v; any = true; }
    }
    ctx->counters[TL_COUNTER_KERNEL_LAUNCHES] = saved_launches;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaStreamSynchronize(ctx->stream);
    cleanup();
    cudaGetLastError();
    ctx->tuned[key] = any ? best : cands[0];
    if (any) tl_record_class_winner(ctx, m, n, k, a_dtype, *q, best);
    ctx->tune_runs++;
  }
  return TL_OK;
}

// JSON: {"version":1,"entries":[{"m":..,"n":..,"k":..,"a_dtype":..,"group":..,"scales_dtype":..,
//        "convention":..,"family":..,"kernel":..,"p":[p0,p1,p2,p3]}, ...]}
int32_t tl_tune_export_json(tl_ctx* ctx, char* buf, size_t cap, size_t* out_len) {
  TL_CHECK_CTX(ctx);
  std::ostringstream os;
  os << "{\"version\":1,\"entries\":[";
  bool first = true;
  for (const auto& kv : ctx->tuned) {
    if (!first) os << ",";
    first = false;
    const TuneKey& t = kv.first;
    const tl_variant& v = kv.second;
    os << "{\"m\":" << t.m << ",\"n\":" << t.n << ",\"k\":" << t.k << ",\"a_dtype\":" << t.a_dtype
       << ",\"group\":" << t.group << ",\"scales_dtype\":" << t.scales_dtype << ",\"convention\":" << t.convention
       << ",\"family\":" << v.family << ",\"kernel\":" << v.kernel << ",\"p\":[" << v.p0 << "," << v.p1 << ","
       << v.p2 << "," << v.p3 << "]}";
  }
  os << "]}";
  const std::string s = os.str();
  if (out_len) *out_len = s.size() + 1;
  if (buf && cap > 0) {
    const size_t nb = std::min(cap - 1, s.size());
    std::memcpy(buf, s.data(), nb);
    buf[nb] = 0;
  }
  return TL_OK;
}

namespace {
// Minimal parser for the exact schema above (whitespace tolerant).
struct Cur {
  const char* p;
  void ws() { while (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r') ++p; }
  bool lit(const char* s) {
    ws();
    const size_t n = std::strlen(s);
    if (std::strncmp(p, s, n) != 0) return false;
    p += n;
    return true;
  }
  bool num(int64_t* out) {
    ws();
    char* end = nullptr;
    const long long v = std::strtoll(p, &end, 10);
    if (end == p) return false;
    p = end;
    *out = v;
    return true;
  }
  bool key(const char* name) {
    std::string k = std::string("\"") + name + "\"";
    return lit(k.c_str()) && lit(":");
  }
};
}  // namespace

int32_t tl_tune_import_json(tl_ctx* ctx, const char* json) {
  TL_CHECK_CTX(ctx);
  if (!json) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_tune_import_json: null text");
  Cur c{json};
  std::map<TuneKey, tl_variant> parsed;
  int64_t ver = 0;
  bool ok = c.lit("{") && c.key("version") && c.num(&ver) && ver == 1 && c.lit(",") && c.key("entries") && c.lit("[");
  if (ok && !c.lit("]")) {
    while (ok) {
      int64_t m, n, k, ad, g, sd, cv, fam, kern, p[4];
      ok = c.lit("{") && c.key("m") && c.num(&m) && c.lit(",") && c.key("n") && c.num(&n) && c.lit(",") &&
           c.key("k") && c.num(&k) && c.lit(",") && c.key("a_dtype") && c.num(&ad) && c.lit(",") &&
           c.key("group") && c.num(&g) && c.lit(",") && c.key("scales_dtype") && c.num(&sd) && c.lit(",") &&
           c.key("convention") && c.num(&cv) && c.lit(",") && c.key("family") && c.num(&fam) && c.lit(",") &&
           c.key("kernel") && c.num(&kern) && c.lit(",") && c.key("p") && c.lit("[") && c.num(&p[0]) &&
           c.lit(",") && c.num(&p[1]) && c.lit(",") && c.num(&p[2]) && c.lit(",") && c.num(&p[3]) && c.lit("]") &&
           c.lit("}");
      if (!ok) break;
      tl_variant v{int32_t(fam), int32_t(kern), int32_t(p[0]), int32_t(p[1]), int32_t(p[2]), int32_t(p[3])};
      parsed[TuneKey{m, n, k, int32_t(ad), int32_t(g), int32_t(sd), int32_t(cv)}] = v;
      if (c.lit(",")) continue;
      ok = c.lit("]");
      break;
    }
  }
  ok = ok && c.lit("}");
  if (ok) { c.ws(); ok = *c.p == 0; }
  if (!ok) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_tune_import_json: invalid tuning-cache JSON near offset %zu", size_t(c.p - json));
  for (const auto& kv : parsed) {
    ctx->tuned[kv.first] = kv.second;
    const tl_quant_desc q{TL_SCHEME_INT8_GROUPED, kv.first.group, kv.first.scales_dtype, kv.first.convention};
    tl_record_class_winner(ctx, kv.first.m, kv.first.n, kv.first.k, kv.first.a_dtype, q, kv.second);  // classes follow the shapes
  }
  return TL_OK;
}

}  // extern "C"
