/*
 * N-API addon over libtlcuda.so: the shim a torchlette `cuda` backend loads
 * (require("./tlcuda.node")).  Each export maps 1:1 to a function of
 * include/tlcuda.h; a non-zero status becomes a thrown JS Error carrying
 * tl_last_error().  Device pointers cross the boundary as BigInt.
 *
 * node_api.h is not available where this was written, so the handful of N-API
 * prototypes used here are declared locally (they are ABI-stable; the symbols
 * resolve when node loads the addon).  Build:
 *   gcc -shared -fPIC tl_napi.c -I ../../../include -L .. -ltlcuda -o tlcuda.node
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#include "tlcuda.h"

/* ---- minimal N-API surface (node_api.h, ABI-stable) ------------------------ */
typedef struct napi_env__* napi_env;
typedef struct napi_value__* napi_value;
typedef struct napi_callback_info__* napi_callback_info;
typedef enum { napi_ok = 0 } napi_status;
typedef napi_value (*napi_callback)(napi_env, napi_callback_info);
typedef struct {
  const char* utf8name; napi_value name; napi_callback method; napi_callback getter; napi_callback setter;
  napi_value value; int attributes; void* data;
} napi_property_descriptor;
extern napi_status napi_get_cb_info(napi_env, napi_callback_info, size_t*, napi_value*, napi_value*, void**);
extern napi_status napi_get_value_int32(napi_env, napi_value, int32_t*);
extern napi_status napi_get_value_int64(napi_env, napi_value, int64_t*);
extern napi_status napi_get_value_double(napi_env, napi_value, double*);
extern napi_status napi_get_value_bigint_uint64(napi_env, napi_value, uint64_t*, int*);
extern napi_status napi_create_bigint_uint64(napi_env, uint64_t, napi_value*);
extern napi_status napi_create_int32(napi_env, int32_t, napi_value*);
extern napi_status napi_create_double(napi_env, double, napi_value*);
extern napi_status napi_get_undefined(napi_env, napi_value*);
extern napi_status napi_throw_error(napi_env, const char*, const char*);
extern napi_status napi_get_typedarray_info(napi_env, napi_value, int*, size_t*, void**, napi_value*, size_t*);
extern napi_status napi_get_arraybuffer_info(napi_env, napi_value, void**, size_t*);
extern napi_status napi_define_properties(napi_env, napi_value, size_t, const napi_property_descriptor*);
extern napi_status napi_get_array_length(napi_env, napi_value, uint32_t*);
extern napi_status napi_get_element(napi_env, napi_value, uint32_t, napi_value*);
extern napi_status napi_get_named_property(napi_env, napi_value, const char*, napi_value*);
extern napi_status napi_typeof(napi_env, napi_value, int*);

#define ARGS(n) size_t argc = n; napi_value argv[n]; napi_get_cb_info(env, info, &argc, argv, NULL, NULL)
static uint64_t u64(napi_env env, napi_value v) { uint64_t r = 0; int lossless = 0; napi_get_value_bigint_uint64(env, v, &r, &lossless); return r; }
static int32_t i32(napi_env env, napi_value v) { int32_t r = 0; napi_get_value_int32(env, v, &r); return r; }
static int64_t i64(napi_env env, napi_value v) { int64_t r = 0; napi_get_value_int64(env, v, &r); return r; }
static double f64(napi_env env, napi_value v) { double r = 0; napi_get_value_double(env, v, &r); return r; }
static napi_value undef(napi_env env) { napi_value u; napi_get_undefined(env, &u); return u; }
static napi_value big(napi_env env, uint64_t v) { napi_value r; napi_create_bigint_uint64(env, v, &r); return r; }
static napi_value check(napi_env env, tl_ctx* ctx, int32_t status) {
  if (status != TL_OK) napi_throw_error(env, NULL, tl_last_error(ctx));
  return undef(env);
}
static void* host_ptr(napi_env env, napi_value typed, size_t* bytes) {
  int type; size_t len; void* data; napi_value ab; size_t off;
  napi_get_typedarray_info(env, typed, &type, &len, &data, &ab, &off);
  void* base; size_t total; napi_get_arraybuffer_info(env, ab, &base, &total);
  if (bytes) *bytes = total - off;
  return data;
}

/* ctxCreate(device) -> BigInt handle */
static napi_value CtxCreate(napi_env env, napi_callback_info info) {
  ARGS(1); tl_ctx* ctx = NULL;
  int32_t st = tl_ctx_create(i32(env, argv[0]), &ctx);
  if (st != TL_OK) { napi_throw_error(env, NULL, tl_last_error(NULL)); return undef(env); }
  return big(env, (uint64_t)(uintptr_t)ctx);
}
static napi_value CtxDestroy(napi_env env, napi_callback_info info) { ARGS(1); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); return check(env, NULL, tl_ctx_destroy(c)); }
static napi_value Sync(napi_env env, napi_callback_info info) { ARGS(1); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); return check(env, c, tl_sync(c)); }
/* alloc(ctx, bytes) -> BigInt device pointer ; free(ctx, ptr) */
static napi_value Alloc(napi_env env, napi_callback_info info) {
  ARGS(2); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); void* p = NULL;
  int32_t st = tl_alloc(c, (size_t)i64(env, argv[1]), &p);
  if (st != TL_OK) { napi_throw_error(env, NULL, tl_last_error(c)); return undef(env); }
  return big(env, (uint64_t)(uintptr_t)p);
}
static napi_value Free(napi_env env, napi_callback_info info) { ARGS(2); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); return check(env, c, tl_free(c, (void*)(uintptr_t)u64(env, argv[1]))); }
/* upload(ctx, dptr, typedArray) ; download(ctx, typedArray, dptr) — both followed by tl_sync so the
 * JS side may reuse the buffer; a Promise-returning variant would run them through napi_async_work. */
static napi_value Upload(napi_env env, napi_callback_info info) {
  ARGS(3); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); size_t n; void* h = host_ptr(env, argv[2], &n);
  int32_t st = tl_upload(c, (void*)(uintptr_t)u64(env, argv[1]), h, n);
  if (st == TL_OK) st = tl_sync(c);
  return check(env, c, st);
}
static napi_value Download(napi_env env, napi_callback_info info) {
  ARGS(3); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); size_t n; void* h = host_ptr(env, argv[1], &n);
  int32_t st = tl_download(c, h, (void*)(uintptr_t)u64(env, argv[2]), n);
  if (st == TL_OK) st = tl_sync(c);
  return check(env, c, st);
}
/* quantize(weightF32, n, k, group, packedU32, scalesU16) */
static napi_value Quantize(napi_env env, napi_callback_info info) {
  ARGS(6);
  return check(env, NULL, tl_quantize_linear_weight((const float*)host_ptr(env, argv[0], NULL), i64(env, argv[1]), i64(env, argv[2]),
                                                    i32(env, argv[3]), (uint32_t*)host_ptr(env, argv[4], NULL),
                                                    (uint16_t*)host_ptr(env, argv[5], NULL)));
}
/* epilogue: JS passes {ops: Int32Array(4*n) [kind,op,inputIndex,toDtype]..., inputs: BigUint64Array} or undefined */
static const tl_epilogue* read_epilogue(napi_env env, napi_value v, tl_epilogue* e) {
  int t = 0; napi_typeof(env, v, &t);
  if (t != 6 /* napi_object */) return NULL;
  memset(e, 0, sizeof(*e));
  napi_value ops, inputs; napi_get_named_property(env, v, "ops", &ops); napi_get_named_property(env, v, "inputs", &inputs);
  size_t ob = 0, ib = 0; int32_t* o = (int32_t*)host_ptr(env, ops, &ob); uint64_t* in = (uint64_t*)host_ptr(env, inputs, &ib);
  e->n_ops = (int32_t)(ob / 16); if (e->n_ops > TL_EPI_MAX_OPS) e->n_ops = TL_EPI_MAX_OPS + 1; /* rejected by the library */
  for (int i = 0; i < e->n_ops && i < TL_EPI_MAX_OPS; ++i) { e->ops[i].kind = o[4*i]; e->ops[i].op = o[4*i+1]; e->ops[i].input_index = o[4*i+2]; e->ops[i].to_dtype = o[4*i+3]; }
  e->n_inputs = (int32_t)(ib / 8); if (e->n_inputs > TL_EPI_MAX_INPUTS) e->n_inputs = TL_EPI_MAX_INPUTS + 1;
  for (int i = 0; i < e->n_inputs && i < TL_EPI_MAX_INPUTS; ++i) e->inputs[i] = (const void*)(uintptr_t)in[i];
  return e;
}
/* qmatmul(ctx, a, aDtype, packed, scales, out, outDtype, m, n, k, group, scalesDtype, convention, alpha, epilogue?, route)
 * route: 0 = seam (tl_qmatmul_nt), 1 = tl_qgemv_nt, 2 = tl_qgemm_nt */
static napi_value QMatmul(napi_env env, napi_callback_info info) {
  ARGS(16); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]);
  tl_quant_desc q = {TL_SCHEME_INT8_GROUPED, i32(env, argv[10]), i32(env, argv[11]), i32(env, argv[12])};
  tl_epilogue e; const tl_epilogue* ep = read_epilogue(env, argv[14], &e);
  const void* a = (const void*)(uintptr_t)u64(env, argv[1]); const void* w = (const void*)(uintptr_t)u64(env, argv[3]);
  const void* s = (const void*)(uintptr_t)u64(env, argv[4]); void* out = (void*)(uintptr_t)u64(env, argv[5]);
  int64_t m = i64(env, argv[7]), n = i64(env, argv[8]), k = i64(env, argv[9]); float alpha = (float)f64(env, argv[13]);
  int route = i32(env, argv[15]); int32_t st;
  if (route == 1) st = tl_qgemv_nt(c, a, i32(env, argv[2]), w, s, out, i32(env, argv[6]), (int32_t)m, n, k, &q, alpha, ep);
  else if (route == 2) st = tl_qgemm_nt(c, a, i32(env, argv[2]), w, s, out, i32(env, argv[6]), m, n, k, &q, alpha, ep);
  else st = tl_qmatmul_nt(c, a, i32(env, argv[2]), w, s, out, i32(env, argv[6]), m, n, k, &q, alpha, ep);
  return check(env, c, st);
}
/* dequant(ctx, packed, scales, out, outDtype, n, k, group, scalesDtype, convention) */
static napi_value Dequant(napi_env env, napi_callback_info info) {
  ARGS(10); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]);
  tl_quant_desc q = {TL_SCHEME_INT8_GROUPED, i32(env, argv[7]), i32(env, argv[8]), i32(env, argv[9])};
  return check(env, c, tl_dequant_int8(c, (const void*)(uintptr_t)u64(env, argv[1]), (const void*)(uintptr_t)u64(env, argv[2]),
                                       (void*)(uintptr_t)u64(env, argv[3]), i32(env, argv[4]), i64(env, argv[5]), i64(env, argv[6]), &q));
}
static napi_value CounterGet(napi_env env, napi_callback_info info) {
  ARGS(2); napi_value r; napi_create_double(env, (double)tl_counter_get((tl_ctx*)(uintptr_t)u64(env, argv[0]), i32(env, argv[1])), &r); return r;
}
static napi_value AsyncErrors(napi_env env, napi_callback_info info) {
  ARGS(1); napi_value r; napi_create_double(env, (double)tl_async_error_count((tl_ctx*)(uintptr_t)u64(env, argv[0])), &r); return r;
}
static napi_value AutotuneSet(napi_env env, napi_callback_info info) { ARGS(2); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); return check(env, c, tl_autotune_set_enabled(c, i32(env, argv[1]))); }
static napi_value AutotuneGet(napi_env env, napi_callback_info info) { ARGS(1); napi_value r; napi_create_int32(env, tl_autotune_is_enabled((tl_ctx*)(uintptr_t)u64(env, argv[0])), &r); return r; }
/* pretune(ctx, shapesBigInt64Array[m,n,k...], aDtype, outDtype, group, scalesDtype, convention) */
static napi_value Pretune(napi_env env, napi_callback_info info) {
  ARGS(7); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); size_t bytes = 0; int64_t* sh = (int64_t*)host_ptr(env, argv[1], &bytes);
  tl_quant_desc q = {TL_SCHEME_INT8_GROUPED, i32(env, argv[4]), i32(env, argv[5]), i32(env, argv[6])};
  return check(env, c, tl_pretune(c, (const tl_shape*)sh, (int32_t)(bytes / sizeof(tl_shape)), i32(env, argv[2]), i32(env, argv[3]), &q));
}
static napi_value GraphBegin(napi_env env, napi_callback_info info) { ARGS(1); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); return check(env, c, tl_graph_begin(c)); }
static napi_value GraphEnd(napi_env env, napi_callback_info info) {
  ARGS(1); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); tl_graph* g = NULL; int32_t st = tl_graph_end(c, &g);
  if (st != TL_OK) { napi_throw_error(env, NULL, tl_last_error(c)); return undef(env); }
  return big(env, (uint64_t)(uintptr_t)g);
}
static napi_value GraphLaunch(napi_env env, napi_callback_info info) { ARGS(2); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); return check(env, c, tl_graph_launch(c, (tl_graph*)(uintptr_t)u64(env, argv[1]))); }
static napi_value GraphDestroy(napi_env env, napi_callback_info info) { ARGS(2); tl_ctx* c = (tl_ctx*)(uintptr_t)u64(env, argv[0]); return check(env, c, tl_graph_destroy(c, (tl_graph*)(uintptr_t)u64(env, argv[1]))); }

napi_value napi_register_module_v1(napi_env env, napi_value exports) {
  const napi_property_descriptor props[] = {
      {"ctxCreate", 0, CtxCreate, 0, 0, 0, 0, 0},   {"ctxDestroy", 0, CtxDestroy, 0, 0, 0, 0, 0},
      {"sync", 0, Sync, 0, 0, 0, 0, 0},             {"alloc", 0, Alloc, 0, 0, 0, 0, 0},
      {"free", 0, Free, 0, 0, 0, 0, 0},             {"upload", 0, Upload, 0, 0, 0, 0, 0},
      {"download", 0, Download, 0, 0, 0, 0, 0},     {"quantize", 0, Quantize, 0, 0, 0, 0, 0},
      {"qmatmul", 0, QMatmul, 0, 0, 0, 0, 0},       {"dequant", 0, Dequant, 0, 0, 0, 0, 0},
      {"counterGet", 0, CounterGet, 0, 0, 0, 0, 0}, {"asyncErrorCount", 0, AsyncErrors, 0, 0, 0, 0, 0},
      {"autotuneSetEnabled", 0, AutotuneSet, 0, 0, 0, 0, 0}, {"autotuneIsEnabled", 0, AutotuneGet, 0, 0, 0, 0, 0},
      {"pretune", 0, Pretune, 0, 0, 0, 0, 0},       {"graphBegin", 0, GraphBegin, 0, 0, 0, 0, 0},
      {"graphEnd", 0, GraphEnd, 0, 0, 0, 0, 0},     {"graphLaunch", 0, GraphLaunch, 0, 0, 0, 0, 0},
      {"graphDestroy", 0, GraphDestroy, 0, 0, 0, 0, 0},
  };
  napi_define_properties(env, exports, sizeof(props) / sizeof(props[0]), props);
  return exports;
}
