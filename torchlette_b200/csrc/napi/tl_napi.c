/*
 * N-API addon over libtlcuda.so: the shim a torchlette `cuda` backend loads
 * (require("./tlcuda.node")).  Every function of include/tlcuda.h has one export here
 * (tl_xxx_yyy -> xxxYyy); a non-zero status becomes a thrown JS Error carrying tl_last_error().
 *
 * Handles.  A context is an external value; ctxDestroy ends it and later calls on it throw.
 * Device memory from `alloc` is an external value whose finalizer frees the allocation when
 * the JS object is collected (unless `free` already did, or the context is gone), so a dropped
 * tensor does not leak; `view(buf, byteOffset)` makes a non-owning handle into the same
 * allocation (it keeps the parent alive) -- the ownsBuffer = false case of BackendTensor
 * (src/backend/types.ts:5-27).  Wherever a device pointer is expected, a buffer handle, a
 * BigInt address (a peer's pointer, say) or null may be passed.
 *
 * Host data.  Typed arrays are read through their own byte length (element count x element
 * size), never through the size of the ArrayBuffer underneath: a subarray or a pooled Buffer
 * view hands over exactly its own bytes.
 *
 * Blocking.  `upload` returns once the copy is enqueued (a copy from pageable memory has left
 * the caller's buffer by then).  `download` blocks the JS thread until the bytes have arrived;
 * `downloadAsync` does not: it enqueues the copy into pinned staging memory, records an event,
 * and waits for the event on a libuv worker (napi_async_work); the Promise resolves on the JS
 * thread after the staging bytes have been copied into the typed array.
 *
 * With -DTL_NAPI_USE_NODE_HEADER the real <node_api.h> is included; otherwise the N-API
 * prototypes used here are declared locally (they are ABI-stable, and the symbols resolve when
 * node loads the addon).  Build:
 *   gcc -shared -fPIC tl_napi.c -I ../../../include -L .. -ltlcuda -o tlcuda.node
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "tlcuda.h"

#ifdef TL_NAPI_USE_NODE_HEADER
#include <node_api.h>
#else
/* ---- the N-API surface used below (node_api.h / js_native_api.h) ------------ */
typedef struct napi_env__* napi_env;
typedef struct napi_value__* napi_value;
typedef struct napi_ref__* napi_ref;
typedef struct napi_deferred__* napi_deferred;
typedef struct napi_callback_info__* napi_callback_info;
typedef struct napi_async_work__* napi_async_work;
typedef enum { napi_ok = 0 } napi_status;
typedef enum {
  napi_undefined, napi_null, napi_boolean, napi_number, napi_string, napi_symbol, napi_object, napi_function,
  napi_external, napi_bigint
} napi_valuetype;
typedef enum {
  napi_int8_array, napi_uint8_array, napi_uint8_clamped_array, napi_int16_array, napi_uint16_array, napi_int32_array,
  napi_uint32_array, napi_float32_array, napi_float64_array, napi_bigint64_array, napi_biguint64_array
} napi_typedarray_type;
typedef napi_value (*napi_callback)(napi_env, napi_callback_info);
typedef void (*napi_finalize)(napi_env, void* data, void* hint);
typedef void (*napi_async_execute_callback)(napi_env, void* data);
typedef void (*napi_async_complete_callback)(napi_env, napi_status, void* data);
typedef struct {
  const char* utf8name; napi_value name; napi_callback method; napi_callback getter; napi_callback setter;
  napi_value value; int attributes; void* data;
} napi_property_descriptor;
extern napi_status napi_get_cb_info(napi_env, napi_callback_info, size_t*, napi_value*, napi_value*, void**);
extern napi_status napi_typeof(napi_env, napi_value, napi_valuetype*);
extern napi_status napi_get_value_int32(napi_env, napi_value, int32_t*);
extern napi_status napi_get_value_int64(napi_env, napi_value, int64_t*);
extern napi_status napi_get_value_double(napi_env, napi_value, double*);
extern napi_status napi_get_value_bigint_uint64(napi_env, napi_value, uint64_t*, int*);
extern napi_status napi_get_value_string_utf8(napi_env, napi_value, char*, size_t, size_t*);
extern napi_status napi_get_value_external(napi_env, napi_value, void**);
extern napi_status napi_create_bigint_uint64(napi_env, uint64_t, napi_value*);
extern napi_status napi_create_int32(napi_env, int32_t, napi_value*);
extern napi_status napi_create_double(napi_env, double, napi_value*);
extern napi_status napi_create_string_utf8(napi_env, const char*, size_t, napi_value*);
extern napi_status napi_create_external(napi_env, void*, napi_finalize, void*, napi_value*);
extern napi_status napi_create_arraybuffer(napi_env, size_t, void**, napi_value*);
extern napi_status napi_create_external_arraybuffer(napi_env, void*, size_t, napi_finalize, void*, napi_value*);
extern napi_status napi_create_typedarray(napi_env, napi_typedarray_type, size_t, napi_value, size_t, napi_value*);
extern napi_status napi_get_undefined(napi_env, napi_value*);
extern napi_status napi_throw_error(napi_env, const char*, const char*);
extern napi_status napi_get_typedarray_info(napi_env, napi_value, napi_typedarray_type*, size_t*, void**, napi_value*, size_t*);
extern napi_status napi_get_arraybuffer_info(napi_env, napi_value, void**, size_t*);
extern napi_status napi_define_properties(napi_env, napi_value, size_t, const napi_property_descriptor*);
extern napi_status napi_get_array_length(napi_env, napi_value, uint32_t*);
extern napi_status napi_get_element(napi_env, napi_value, uint32_t, napi_value*);
extern napi_status napi_get_named_property(napi_env, napi_value, const char*, napi_value*);
extern napi_status napi_create_reference(napi_env, napi_value, uint32_t, napi_ref*);
extern napi_status napi_delete_reference(napi_env, napi_ref);
extern napi_status napi_get_reference_value(napi_env, napi_ref, napi_value*);
extern napi_status napi_create_promise(napi_env, napi_deferred*, napi_value*);
extern napi_status napi_resolve_deferred(napi_env, napi_deferred, napi_value);
extern napi_status napi_reject_deferred(napi_env, napi_deferred, napi_value);
extern napi_status napi_create_error(napi_env, napi_value code, napi_value msg, napi_value*);
extern napi_status napi_create_async_work(napi_env, napi_value, napi_value, napi_async_execute_callback,
                                          napi_async_complete_callback, void*, napi_async_work*);
extern napi_status napi_queue_async_work(napi_env, napi_async_work);
extern napi_status napi_delete_async_work(napi_env, napi_async_work);
#endif

/* ---- handles ------------------------------------------------------------------ */
typedef struct CtxBox {
  tl_ctx* ctx;      /* NULL once destroyed */
  int64_t holders;  /* JS objects (the context value, buffers, pinned blocks, jobs) that point here */
} CtxBox;
typedef struct DevBuf {
  CtxBox* box;
  void* ptr;        /* NULL once freed */
  size_t bytes;
  int owns;
  napi_ref parent;  /* a view keeps its allocation alive */
} DevBuf;
typedef struct PinBlock {
  CtxBox* box;
  void* ptr;
  struct PinBlock* next;
} PinBlock;
static PinBlock* g_pinned = NULL;

static void box_release(CtxBox* box) {
  if (--box->holders == 0) {
    if (box->ctx) tl_ctx_destroy(box->ctx);
    free(box);
  }
}
static void ctx_finalize(napi_env env, void* data, void* hint) { (void)env; (void)hint; box_release((CtxBox*)data); }
static void buf_finalize(napi_env env, void* data, void* hint) {
  (void)hint;
  DevBuf* b = (DevBuf*)data;
  if (b->owns && b->ptr && b->box->ctx) tl_free(b->box->ctx, b->ptr);
  if (b->parent) napi_delete_reference(env, b->parent);
  box_release(b->box);
  free(b);
}
static void pin_finalize(napi_env env, void* data, void* hint) {
  (void)env; (void)data;
  PinBlock* p = (PinBlock*)hint;
  if (p->ptr && p->box->ctx) tl_host_free_pinned(p->box->ctx, p->ptr);
  for (PinBlock** q = &g_pinned; *q; q = &(*q)->next)
    if (*q == p) { *q = p->next; break; }
  box_release(p->box);
  free(p);
}

/* ---- argument helpers --------------------------------------------------------- */
#define ARGS(n) size_t argc = n; napi_value argv[n]; memset(argv, 0, sizeof(argv)); napi_get_cb_info(env, info, &argc, argv, NULL, NULL)
#define FN(name) static napi_value name(napi_env env, napi_callback_info info)
#define CTX(i) CtxBox* box = ctx_box(env, argv[i]); if (!box) return undef(env); tl_ctx* c = box->ctx

static napi_value undef(napi_env env) { napi_value u; napi_get_undefined(env, &u); return u; }
static napi_valuetype type_of(napi_env env, napi_value v) {
  napi_valuetype t = napi_undefined;
  if (v) napi_typeof(env, v, &t);
  return t;
}
static int32_t i32(napi_env env, napi_value v) { int32_t r = 0; napi_get_value_int32(env, v, &r); return r; }
static int64_t i64(napi_env env, napi_value v) {
  if (type_of(env, v) == napi_bigint) { uint64_t r = 0; int ok = 0; napi_get_value_bigint_uint64(env, v, &r, &ok); return (int64_t)r; }
  int64_t r = 0; napi_get_value_int64(env, v, &r); return r;
}
static double f64(napi_env env, napi_value v) { double r = 0; napi_get_value_double(env, v, &r); return r; }
static napi_value num(napi_env env, double v) { napi_value r; napi_create_double(env, v, &r); return r; }
static napi_value big(napi_env env, uint64_t v) { napi_value r; napi_create_bigint_uint64(env, v, &r); return r; }
static napi_value str(napi_env env, const char* s) { napi_value r; napi_create_string_utf8(env, s ? s : "", (size_t)-1, &r); return r; }
static napi_value check(napi_env env, tl_ctx* ctx, int32_t status) {
  if (status != TL_OK) napi_throw_error(env, NULL, tl_last_error(ctx));
  return undef(env);
}
static CtxBox* ctx_box(napi_env env, napi_value v) {
  void* p = NULL;
  if (type_of(env, v) == napi_external) napi_get_value_external(env, v, &p);
  CtxBox* box = (CtxBox*)p;
  if (!box || !box->ctx) { napi_throw_error(env, NULL, "tlcuda: not a live context"); return NULL; }
  return box;
}
/* a device pointer: buffer handle | BigInt address | null | undefined */
static void* dptr(napi_env env, napi_value v) {
  napi_valuetype t = type_of(env, v);
  if (t == napi_external) { void* p = NULL; napi_get_value_external(env, v, &p); return p ? ((DevBuf*)p)->ptr : NULL; }
  if (t == napi_bigint) { uint64_t r = 0; int ok = 0; napi_get_value_bigint_uint64(env, v, &r, &ok); return (void*)(uintptr_t)r; }
  return NULL;
}
/* a handle made by this addon that is not a buffer (graph, event, chain): BigInt of its address */
static void* hptr(napi_env env, napi_value v) {
  uint64_t r = 0; int ok = 0;
  if (type_of(env, v) == napi_bigint) napi_get_value_bigint_uint64(env, v, &r, &ok);
  return (void*)(uintptr_t)r;
}
static const size_t kElemBytes[] = {1, 1, 1, 2, 2, 4, 4, 4, 8, 8, 8};
/* the typed array's own bytes: element count x element size */
static void* host_ptr(napi_env env, napi_value typed, size_t* bytes) {
  napi_typedarray_type type = napi_uint8_array; size_t len = 0; void* data = NULL; napi_value ab; size_t off = 0;
  if (bytes) *bytes = 0;
  if (type_of(env, typed) != napi_object) return NULL;
  if (napi_get_typedarray_info(env, typed, &type, &len, &data, &ab, &off) != napi_ok) return NULL;
  if (bytes) *bytes = len * ((unsigned)type < sizeof(kElemBytes) / sizeof(kElemBytes[0]) ? kElemBytes[type] : 1);
  return data;
}
static napi_value make_i32_array(napi_env env, const int32_t* src, size_t count) {
  void* data = NULL; napi_value ab, arr;
  napi_create_arraybuffer(env, count * 4, &data, &ab);
  memcpy(data, src, count * 4);
  napi_create_typedarray(env, napi_int32_array, count, ab, 0, &arr);
  return arr;
}
static napi_value make_u8_array(napi_env env, const void* src, size_t count) {
  void* data = NULL; napi_value ab, arr;
  napi_create_arraybuffer(env, count, &data, &ab);
  memcpy(data, src, count);
  napi_create_typedarray(env, napi_uint8_array, count, ab, 0, &arr);
  return arr;
}
/* quant descriptor: Int32Array [scheme, groupSize, scalesDtype, scaleConvention] (the struct's layout) */
static int read_qdesc(napi_env env, napi_value v, tl_quant_desc* q) {
  size_t bytes = 0; const int32_t* p = (const int32_t*)host_ptr(env, v, &bytes);
  if (!p || bytes != sizeof(tl_quant_desc)) { napi_throw_error(env, NULL, "tlcuda: quant descriptor must be an Int32Array(4)"); return 0; }
  memcpy(q, p, sizeof(*q));
  return 1;
}
/* variant: Int32Array [family, kernel, p0, p1, p2, p3] */
static int read_variant(napi_env env, napi_value v, tl_variant* out) {
  size_t bytes = 0; const int32_t* p = (const int32_t*)host_ptr(env, v, &bytes);
  if (!p || bytes != sizeof(tl_variant)) { napi_throw_error(env, NULL, "tlcuda: variant must be an Int32Array(6)"); return 0; }
  memcpy(out, p, sizeof(*out));
  return 1;
}
/* epilogue: { ops: Int32Array(4 n) of [kind, op, inputIndex, toDtype], inputs: Array of device pointers } | undefined */
static const tl_epilogue* read_epilogue(napi_env env, napi_value v, tl_epilogue* e) {
  if (type_of(env, v) != napi_object) return NULL;
  memset(e, 0, sizeof(*e));
  napi_value ops, inputs;
  napi_get_named_property(env, v, "ops", &ops);
  napi_get_named_property(env, v, "inputs", &inputs);
  size_t ob = 0; const int32_t* o = (const int32_t*)host_ptr(env, ops, &ob);
  e->n_ops = (int32_t)(ob / 16);
  if (e->n_ops > TL_EPI_MAX_OPS) e->n_ops = TL_EPI_MAX_OPS + 1; /* the library rejects it with its own message */
  for (int i = 0; i < e->n_ops && i < TL_EPI_MAX_OPS; ++i) {
    e->ops[i].kind = o[4 * i]; e->ops[i].op = o[4 * i + 1]; e->ops[i].input_index = o[4 * i + 2]; e->ops[i].to_dtype = o[4 * i + 3];
  }
  uint32_t n_in = 0;
  if (type_of(env, inputs) == napi_object) napi_get_array_length(env, inputs, &n_in);
  e->n_inputs = n_in > TL_EPI_MAX_INPUTS ? TL_EPI_MAX_INPUTS + 1 : (int32_t)n_in;
  for (uint32_t i = 0; i < n_in && i < TL_EPI_MAX_INPUTS; ++i) {
    napi_value el; napi_get_element(env, inputs, i, &el);
    e->inputs[i] = dptr(env, el);
  }
  return e;
}
static napi_value receipt_value(napi_env env, const tl_plan_receipt* r) {
  /* Int32Array [family, kernel, p0, p1, p2, p3, grid x, y, z, block, splitK, fromTuningCache, epilogueEngaged] */
  return make_i32_array(env, (const int32_t*)r, sizeof(*r) / 4);
}

/* ---- context ------------------------------------------------------------------ */
FN(CtxCreate) {
  ARGS(1); tl_ctx* ctx = NULL;
  if (tl_ctx_create(i32(env, argv[0]), &ctx) != TL_OK) { napi_throw_error(env, NULL, tl_last_error(NULL)); return undef(env); }
  CtxBox* box = (CtxBox*)calloc(1, sizeof(CtxBox));
  box->ctx = ctx; box->holders = 1;
  napi_value v; napi_create_external(env, box, ctx_finalize, NULL, &v);
  return v;
}
FN(CtxDestroy) {
  ARGS(1); CTX(0);
  box->ctx = NULL; /* buffers that outlive the context skip their tl_free */
  if (tl_ctx_destroy(c) != TL_OK) napi_throw_error(env, NULL, "tlcuda: tl_ctx_destroy failed");
  return undef(env);
}
FN(Sync) { ARGS(1); CTX(0); return check(env, c, tl_sync(c)); }
FN(AsyncErrorCount) { ARGS(1); CTX(0); return num(env, (double)tl_async_error_count(c)); }
FN(LastError) { ARGS(1); CtxBox* box = NULL; void* p = NULL; if (type_of(env, argv[0]) == napi_external) { napi_get_value_external(env, argv[0], &p); box = (CtxBox*)p; } return str(env, tl_last_error(box ? box->ctx : NULL)); }
FN(CtxStream) { ARGS(1); CTX(0); void* s = NULL; if (tl_ctx_stream(c, &s) != TL_OK) return check(env, c, -1); return big(env, (uint64_t)(uintptr_t)s); }
FN(DeviceSmCount) { ARGS(1); CTX(0); int32_t n = 0; if (tl_device_sm_count(c, &n) != TL_OK) return check(env, c, -1); return num(env, n); }
FN(SetOption) { ARGS(3); CTX(0); char name[64]; size_t len = 0; napi_get_value_string_utf8(env, argv[1], name, sizeof(name), &len); return check(env, c, tl_set_option(c, name, i64(env, argv[2]))); }
FN(GetOption) {
  ARGS(2); CTX(0); char name[64]; size_t len = 0; int64_t v = 0;
  napi_get_value_string_utf8(env, argv[1], name, sizeof(name), &len);
  if (tl_get_option(c, name, &v) != TL_OK) return check(env, c, -1);
  return big(env, (uint64_t)v); /* BigInt: some options are addresses */
}

/* ---- memory ------------------------------------------------------------------- */
/* alloc(ctx, bytes) -> owning buffer handle */
FN(Alloc) {
  ARGS(2); CTX(0); void* p = NULL; size_t bytes = (size_t)i64(env, argv[1]);
  if (tl_alloc(c, bytes, &p) != TL_OK) return check(env, c, -1);
  DevBuf* b = (DevBuf*)calloc(1, sizeof(DevBuf));
  b->box = box; b->ptr = p; b->bytes = bytes; b->owns = 1; box->holders++;
  napi_value v; napi_create_external(env, b, buf_finalize, NULL, &v);
  return v;
}
/* view(buf, byteOffset) -> non-owning handle into the same allocation */
FN(View) {
  ARGS(2); void* p = NULL;
  if (type_of(env, argv[0]) != napi_external) { napi_throw_error(env, NULL, "tlcuda: view() needs a buffer handle"); return undef(env); }
  napi_get_value_external(env, argv[0], &p);
  DevBuf* src = (DevBuf*)p; size_t off = (size_t)i64(env, argv[1]);
  if (!src->ptr || off > src->bytes) { napi_throw_error(env, NULL, "tlcuda: view() outside the allocation"); return undef(env); }
  DevBuf* b = (DevBuf*)calloc(1, sizeof(DevBuf));
  b->box = src->box; b->ptr = (char*)src->ptr + off; b->bytes = src->bytes - off; b->owns = 0; src->box->holders++;
  napi_create_reference(env, argv[0], 1, &b->parent);
  napi_value v; napi_create_external(env, b, buf_finalize, NULL, &v);
  return v;
}
/* free(ctx, buf): frees now (an owning handle only); the finalizer then has nothing left to do */
FN(Free) {
  ARGS(2); CTX(0);
  if (type_of(env, argv[1]) == napi_external) {
    void* p = NULL; napi_get_value_external(env, argv[1], &p); DevBuf* b = (DevBuf*)p;
    int32_t st = TL_OK;
    if (b->owns && b->ptr) st = tl_free(c, b->ptr);
    b->ptr = NULL;
    return check(env, c, st);
  }
  return check(env, c, tl_free(c, dptr(env, argv[1])));
}
FN(PtrOf) { ARGS(1); return big(env, (uint64_t)(uintptr_t)dptr(env, argv[0])); }
FN(Upload) {
  ARGS(3); CTX(0); size_t n = 0; void* h = host_ptr(env, argv[2], &n);
  return check(env, c, tl_upload(c, dptr(env, argv[1]), h, n));
}
FN(Download) {
  ARGS(3); CTX(0); size_t n = 0; void* h = host_ptr(env, argv[1], &n);
  int32_t st = tl_download(c, h, dptr(env, argv[2]), n);
  if (st == TL_OK) st = tl_sync(c);
  return check(env, c, st);
}
typedef struct DlJob {
  napi_async_work work; napi_deferred deferred; napi_ref keep;
  CtxBox* box; tl_ctx* ctx; void* staging; size_t bytes; tl_event* ev; int32_t st;
} DlJob;
static void dl_execute(napi_env env, void* data) { (void)env; DlJob* j = (DlJob*)data; j->st = tl_event_synchronize(j->ctx, j->ev); }
static void dl_complete(napi_env env, napi_status status, void* data) {
  DlJob* j = (DlJob*)data; napi_value target, result;
  napi_get_reference_value(env, j->keep, &target);
  size_t n = 0; void* dst = host_ptr(env, target, &n);
  const int ok = status == napi_ok && j->st == TL_OK && dst && n == j->bytes && j->box->ctx;
  if (ok) memcpy(dst, j->staging, n);
  if (j->box->ctx) { tl_event_destroy(j->box->ctx, j->ev); tl_host_free_pinned(j->box->ctx, j->staging); }
  if (ok) napi_resolve_deferred(env, j->deferred, target);
  else { napi_create_error(env, NULL, str(env, "tlcuda: downloadAsync failed (device error, or the context or the target array went away)"), &result); napi_reject_deferred(env, j->deferred, result); }
  napi_delete_reference(env, j->keep);
  napi_delete_async_work(env, j->work);
  box_release(j->box);
  free(j);
}
/* downloadAsync(ctx, typedArray, src) -> Promise<typedArray> */
FN(DownloadAsync) {
  ARGS(3); CTX(0); size_t n = 0; void* h = host_ptr(env, argv[1], &n);
  if (!h && n) { napi_throw_error(env, NULL, "tlcuda: downloadAsync needs a typed array"); return undef(env); }
  DlJob* j = (DlJob*)calloc(1, sizeof(DlJob));
  j->box = box; j->ctx = c; j->bytes = n;
  int32_t st = tl_host_alloc_pinned(c, n ? n : 1, &j->staging);
  if (st == TL_OK) st = tl_download(c, j->staging, dptr(env, argv[2]), n);
  if (st == TL_OK) st = tl_event_create(c, &j->ev);
  if (st == TL_OK) st = tl_event_record(c, j->ev);
  if (st != TL_OK) {
    if (j->ev) tl_event_destroy(c, j->ev);
    if (j->staging) tl_host_free_pinned(c, j->staging);
    free(j);
    return check(env, c, st);
  }
  box->holders++;
  napi_value promise;
  napi_create_promise(env, &j->deferred, &promise);
  napi_create_reference(env, argv[1], 1, &j->keep);
  napi_create_async_work(env, NULL, str(env, "tlcuda.downloadAsync"), dl_execute, dl_complete, j, &j->work);
  napi_queue_async_work(env, j->work);
  return promise;
}
/* hostAllocPinned(ctx, bytes) -> ArrayBuffer over page-locked memory (freed when collected, or by hostFreePinned) */
FN(HostAllocPinned) {
  ARGS(2); CTX(0); void* p = NULL; size_t bytes = (size_t)i64(env, argv[1]);
  if (tl_host_alloc_pinned(c, bytes, &p) != TL_OK) return check(env, c, -1);
  PinBlock* pb = (PinBlock*)calloc(1, sizeof(PinBlock));
  pb->box = box; pb->ptr = p; pb->next = g_pinned; g_pinned = pb; box->holders++;
  napi_value ab; napi_create_external_arraybuffer(env, p, bytes, pin_finalize, pb, &ab);
  return ab;
}
/* hostFreePinned(ctx, arrayBuffer): releases the pages now; the ArrayBuffer must not be used afterwards */
FN(HostFreePinned) {
  ARGS(2); CTX(0); void* data = NULL; size_t len = 0;
  napi_get_arraybuffer_info(env, argv[1], &data, &len);
  for (PinBlock* p = g_pinned; p; p = p->next)
    if (p->ptr == data && data) { p->ptr = NULL; return check(env, c, tl_host_free_pinned(c, data)); }
  napi_throw_error(env, NULL, "tlcuda: hostFreePinned: not a pinned block of this addon");
  return undef(env);
}
FN(Memset) { ARGS(4); CTX(0); return check(env, c, tl_memset(c, dptr(env, argv[1]), i32(env, argv[2]), (size_t)i64(env, argv[3]))); }
/* copy2d(ctx, dst, dstPitch, src, srcPitch, widthBytes, height) */
FN(Copy2d) {
  ARGS(7); CTX(0);
  return check(env, c, tl_copy2d(c, dptr(env, argv[1]), (size_t)i64(env, argv[2]), dptr(env, argv[3]), (size_t)i64(env, argv[4]),
                                 (size_t)i64(env, argv[5]), (size_t)i64(env, argv[6])));
}

/* ---- quantizer ---------------------------------------------------------------- */
/* quantizeLinearWeight(weightF32, n, k, group, packedU32, scalesU16): host arrays, lengths checked here */
FN(QuantizeLinearWeight) {
  ARGS(6); size_t wb = 0, pb = 0, sb = 0;
  const float* w = (const float*)host_ptr(env, argv[0], &wb); uint32_t* p = (uint32_t*)host_ptr(env, argv[4], &pb);
  uint16_t* s = (uint16_t*)host_ptr(env, argv[5], &sb);
  int64_t n = i64(env, argv[1]), k = i64(env, argv[2]); int32_t g = i32(env, argv[3]);
  if (g <= 0 || n < 0 || k < 0 || wb != (size_t)(n * k) * 4 || pb != (size_t)(n * k) || sb != (size_t)(n * (k / g)) * 2) {
    napi_throw_error(env, NULL, "quantizeLinearWeight: array lengths do not match n, k and the group size");
    return undef(env);
  }
  return check(env, NULL, tl_quantize_linear_weight(w, n, k, g, p, s));
}
/* quantizeLinearWeightDevice(ctx, weight, n, k, group, packed, scales): device pointers */
FN(QuantizeLinearWeightDevice) {
  ARGS(7); CTX(0);
  return check(env, c, tl_quantize_linear_weight_device(c, (const float*)dptr(env, argv[1]), i64(env, argv[2]), i64(env, argv[3]),
                                                        i32(env, argv[4]), (uint32_t*)dptr(env, argv[5]), (uint16_t*)dptr(env, argv[6])));
}
FN(F32ToF16Bits) { ARGS(1); return num(env, tl_f32_to_f16_bits((float)f64(env, argv[0]))); }
FN(F16BitsToF32) { ARGS(1); return num(env, tl_f16_bits_to_f32((uint32_t)i64(env, argv[0]))); }

/* ---- quantized products --------------------------------------------------------
 * Common argument list: (ctx, a, aDtype, packed, scales, out, outDtype, m, n, k, qdesc, alpha, epilogue?) */
typedef int32_t (*qfn64)(tl_ctx*, const void*, int32_t, const void*, const void*, void*, int32_t, int64_t, int64_t, int64_t,
                         const tl_quant_desc*, float, const tl_epilogue*);
static napi_value q_call64(napi_env env, napi_callback_info info, qfn64 fn) {
  ARGS(13); CTX(0); tl_quant_desc q; tl_epilogue e;
  if (!read_qdesc(env, argv[10], &q)) return undef(env);
  const tl_epilogue* ep = read_epilogue(env, argv[12], &e);
  return check(env, c, fn(c, dptr(env, argv[1]), i32(env, argv[2]), dptr(env, argv[3]), dptr(env, argv[4]), dptr(env, argv[5]),
                          i32(env, argv[6]), i64(env, argv[7]), i64(env, argv[8]), i64(env, argv[9]), &q, (float)f64(env, argv[11]), ep));
}
typedef int32_t (*qfn32)(tl_ctx*, const void*, int32_t, const void*, const void*, void*, int32_t, int32_t, int64_t, int64_t,
                         const tl_quant_desc*, float, const tl_epilogue*);
static napi_value q_call32(napi_env env, napi_callback_info info, qfn32 fn) {
  ARGS(13); CTX(0); tl_quant_desc q; tl_epilogue e;
  if (!read_qdesc(env, argv[10], &q)) return undef(env);
  const tl_epilogue* ep = read_epilogue(env, argv[12], &e);
  return check(env, c, fn(c, dptr(env, argv[1]), i32(env, argv[2]), dptr(env, argv[3]), dptr(env, argv[4]), dptr(env, argv[5]),
                          i32(env, argv[6]), i32(env, argv[7]), i64(env, argv[8]), i64(env, argv[9]), &q, (float)f64(env, argv[11]), ep));
}
typedef int32_t (*qfn_noepi)(tl_ctx*, const void*, int32_t, const void*, const void*, void*, int32_t, int32_t, int64_t, int64_t,
                             const tl_quant_desc*, float);
static napi_value q_call_noepi(napi_env env, napi_callback_info info, qfn_noepi fn) {
  ARGS(12); CTX(0); tl_quant_desc q;
  if (!read_qdesc(env, argv[10], &q)) return undef(env);
  return check(env, c, fn(c, dptr(env, argv[1]), i32(env, argv[2]), dptr(env, argv[3]), dptr(env, argv[4]), dptr(env, argv[5]),
                          i32(env, argv[6]), i32(env, argv[7]), i64(env, argv[8]), i64(env, argv[9]), &q, (float)f64(env, argv[11])));
}
FN(QgemvNt) { return q_call32(env, info, tl_qgemv_nt); }
FN(QgemvNtStaticScratch) { return q_call32(env, info, tl_qgemv_nt_static_scratch); }
FN(QgemmNt) { return q_call64(env, info, tl_qgemm_nt); }
FN(QmatmulNt) { return q_call64(env, info, tl_qmatmul_nt); }
FN(QgemvNtAllreduce) { return q_call_noepi(env, info, tl_qgemv_nt_allreduce); }
FN(QgemvNtPush) { return q_call_noepi(env, info, tl_qgemv_nt_push); }
FN(ReducePending) { ARGS(1); CTX(0); return check(env, c, tl_reduce_pending(c)); }

/* items: Array of { packed, scales, out, n, alpha, epilogue? }; the epilogues live in `store` */
static int read_items(napi_env env, napi_value arr, tl_qgemv_item* items, tl_epilogue* store, int max_items) {
  uint32_t n = 0;
  if (type_of(env, arr) == napi_object) napi_get_array_length(env, arr, &n);
  if (n > (uint32_t)max_items) return -1;
  for (uint32_t i = 0; i < n; ++i) {
    napi_value it, v;
    napi_get_element(env, arr, i, &it);
    napi_get_named_property(env, it, "packed", &v); items[i].packed = dptr(env, v);
    napi_get_named_property(env, it, "scales", &v); items[i].scales = dptr(env, v);
    napi_get_named_property(env, it, "out", &v); items[i].out = dptr(env, v);
    napi_get_named_property(env, it, "n", &v); items[i].n = i64(env, v);
    napi_get_named_property(env, it, "alpha", &v); items[i].alpha = type_of(env, v) == napi_number ? (float)f64(env, v) : 1.0f;
    napi_get_named_property(env, it, "epilogue", &v); items[i].epilogue = read_epilogue(env, v, &store[i]);
  }
  return (int)n;
}
/* qgemvNtBatched(ctx, a, aDtype, items, outDtype, m, k, qdesc) */
FN(QgemvNtBatched) {
  ARGS(8); CTX(0); tl_quant_desc q; tl_qgemv_item items[16]; tl_epilogue store[16];
  if (!read_qdesc(env, argv[7], &q)) return undef(env);
  int n = read_items(env, argv[3], items, store, 16);
  if (n < 0) { napi_throw_error(env, NULL, "qgemvNtBatched: at most 16 items"); return undef(env); }
  return check(env, c, tl_qgemv_nt_batched(c, dptr(env, argv[1]), i32(env, argv[2]), items, n, i32(env, argv[4]), i32(env, argv[5]),
                                           i64(env, argv[6]), &q));
}
/* qgemvChainCreate(ctx, phases, aDtype, m, scalesDtype, convention) -> BigInt chain handle;
 * phases: Array of { a, k, groupSize, outDtype, items } with at most 4 items each */
FN(QgemvChainCreate) {
  ARGS(6); CTX(0); uint32_t np = 0;
  if (type_of(env, argv[1]) == napi_object) napi_get_array_length(env, argv[1], &np);
  if (np == 0 || np > 1024) { napi_throw_error(env, NULL, "qgemvChainCreate: 1..1024 phases"); return undef(env); }
  tl_chain_phase* ph = (tl_chain_phase*)calloc(np, sizeof(tl_chain_phase));
  tl_epilogue* store = (tl_epilogue*)calloc((size_t)np * 4, sizeof(tl_epilogue));
  int bad = 0;
  for (uint32_t i = 0; i < np && !bad; ++i) {
    napi_value p, v;
    napi_get_element(env, argv[1], i, &p);
    napi_get_named_property(env, p, "a", &v); ph[i].a = dptr(env, v);
    napi_get_named_property(env, p, "k", &v); ph[i].k = i64(env, v);
    napi_get_named_property(env, p, "groupSize", &v); ph[i].group_size = i32(env, v);
    napi_get_named_property(env, p, "outDtype", &v); ph[i].out_dtype = i32(env, v);
    napi_get_named_property(env, p, "items", &v);
    int n = read_items(env, v, ph[i].items, store + (size_t)i * 4, 4);
    if (n < 0) bad = 1; else ph[i].n_items = n;
  }
  tl_chain* chain = NULL; int32_t st = TL_ERR_INVALID_ARG;
  if (!bad) st = tl_qgemv_chain_create(c, ph, (int32_t)np, i32(env, argv[2]), i32(env, argv[3]), i32(env, argv[4]), i32(env, argv[5]), &chain);
  free(ph); free(store); /* the library flattens the description at create time */
  if (bad) { napi_throw_error(env, NULL, "qgemvChainCreate: at most 4 items per phase"); return undef(env); }
  if (st != TL_OK) return check(env, c, st);
  return big(env, (uint64_t)(uintptr_t)chain);
}
FN(QgemvChainLaunch) { ARGS(2); CTX(0); return check(env, c, tl_qgemv_chain_launch(c, (tl_chain*)hptr(env, argv[1]))); }
FN(QgemvChainDestroy) { ARGS(2); CTX(0); return check(env, c, tl_qgemv_chain_destroy(c, (tl_chain*)hptr(env, argv[1]))); }
/* dequantInt8(ctx, packed, scales, out, outDtype, n, k, qdesc) */
FN(DequantInt8) {
  ARGS(8); CTX(0); tl_quant_desc q;
  if (!read_qdesc(env, argv[7], &q)) return undef(env);
  return check(env, c, tl_dequant_int8(c, dptr(env, argv[1]), dptr(env, argv[2]), dptr(env, argv[3]), i32(env, argv[4]), i64(env, argv[5]),
                                       i64(env, argv[6]), &q));
}
/* quantizeLinearWeightInt4(weightF32, n, k, group, packedU32 [n, k/8], scalesU16) */
FN(QuantizeLinearWeightInt4) {
  ARGS(6); size_t wb = 0, pb = 0, sb = 0;
  const float* w = (const float*)host_ptr(env, argv[0], &wb); uint32_t* p = (uint32_t*)host_ptr(env, argv[4], &pb);
  uint16_t* s = (uint16_t*)host_ptr(env, argv[5], &sb);
  int64_t n = i64(env, argv[1]), k = i64(env, argv[2]); int32_t g = i32(env, argv[3]);
  if (g <= 0 || n < 0 || k < 0 || wb != (size_t)(n * k) * 4 || pb != (size_t)(n * k) / 2 || sb != (size_t)(n * (k / g)) * 2) {
    napi_throw_error(env, NULL, "quantizeLinearWeightInt4: array lengths do not match n, k and the group size");
    return undef(env);
  }
  return check(env, NULL, tl_quantize_linear_weight_int4(w, n, k, g, p, s));
}
FN(DequantInt4) {
  ARGS(8); CTX(0); tl_quant_desc q;
  if (!read_qdesc(env, argv[7], &q)) return undef(env);
  return check(env, c, tl_dequant_int4(c, dptr(env, argv[1]), dptr(env, argv[2]), dptr(env, argv[3]), i32(env, argv[4]), i64(env, argv[5]),
                                       i64(env, argv[6]), &q));
}
FN(UnpackInt4) { ARGS(5); CTX(0); return check(env, c, tl_unpack_int4(c, dptr(env, argv[1]), dptr(env, argv[2]), i64(env, argv[3]), i64(env, argv[4]))); }
FN(UnpackInt8) { ARGS(5); CTX(0); return check(env, c, tl_unpack_int8(c, dptr(env, argv[1]), dptr(env, argv[2]), i64(env, argv[3]), i64(env, argv[4]))); }

/* ---- companion ops ---------------------------------------------------------------- */
/* unaryOp(ctx, op, in, inDtype, out, outDtype, count) ; op 0 = cast / copy */
FN(UnaryOp) { ARGS(7); CTX(0); return check(env, c, tl_unary_op(c, i32(env, argv[1]), dptr(env, argv[2]), i32(env, argv[3]), dptr(env, argv[4]), i32(env, argv[5]), i64(env, argv[6]))); }
/* binaryOp(ctx, op, a, aDtype, b, bDtype, out, outDtype, rows, cols, bIsRow) */
FN(BinaryOp) {
  ARGS(11); CTX(0);
  return check(env, c, tl_binary_op(c, i32(env, argv[1]), dptr(env, argv[2]), i32(env, argv[3]), dptr(env, argv[4]), i32(env, argv[5]),
                                    dptr(env, argv[6]), i32(env, argv[7]), i64(env, argv[8]), i64(env, argv[9]), i32(env, argv[10])));
}
/* transpose2d(ctx, in, out, batch, rows, cols, elemBytes) */
FN(Transpose2d) { ARGS(7); CTX(0); return check(env, c, tl_transpose2d(c, dptr(env, argv[1]), dptr(env, argv[2]), i64(env, argv[3]), i64(env, argv[4]), i64(env, argv[5]), i32(env, argv[6]))); }

/* rmsnorm(ctx, x, xDtype, weight, weightDtype, out, outDtype, rows, cols, eps) */
FN(Rmsnorm) {
  ARGS(10); CTX(0);
  return check(env, c, tl_rmsnorm(c, dptr(env, argv[1]), i32(env, argv[2]), dptr(env, argv[3]), i32(env, argv[4]), dptr(env, argv[5]), i32(env, argv[6]),
                                  i64(env, argv[7]), i64(env, argv[8]), (float)f64(env, argv[9])));
}
/* rope(ctx, qk, dtype, cos, sin, out, outer, seqLen, headDim, sinScale, cosOffset, sinOffset) */
FN(Rope) {
  ARGS(12); CTX(0);
  return check(env, c, tl_rope(c, dptr(env, argv[1]), i32(env, argv[2]), (const float*)dptr(env, argv[3]), (const float*)dptr(env, argv[4]), dptr(env, argv[5]),
                               i64(env, argv[6]), i64(env, argv[7]), i64(env, argv[8]), (float)f64(env, argv[9]), i64(env, argv[10]), i64(env, argv[11])));
}
/* decodeAttention(ctx, q, kCache, vCache, out, dtype, batch, heads, kvHeads, headDim, kvLen, kvCapacity, scale, mask | null) */
FN(DecodeAttention) {
  ARGS(14); CTX(0);
  return check(env, c, tl_decode_attention(c, dptr(env, argv[1]), dptr(env, argv[2]), dptr(env, argv[3]), dptr(env, argv[4]), i32(env, argv[5]), i64(env, argv[6]),
                                           i64(env, argv[7]), i64(env, argv[8]), i64(env, argv[9]), i64(env, argv[10]), i64(env, argv[11]),
                                           (float)f64(env, argv[12]), (const float*)dptr(env, argv[13])));
}

/* attention(ctx, q, kCache, vCache, out, dtype, batch, heads, kvHeads, qLen, headDim, kvLen, kvCapacity, scale, mask | null, causal) */
FN(Attention) {
  ARGS(16); CTX(0);
  return check(env, c, tl_attention(c, dptr(env, argv[1]), dptr(env, argv[2]), dptr(env, argv[3]), dptr(env, argv[4]), i32(env, argv[5]), i64(env, argv[6]),
                                    i64(env, argv[7]), i64(env, argv[8]), i64(env, argv[9]), i64(env, argv[10]), i64(env, argv[11]), i64(env, argv[12]),
                                    (float)f64(env, argv[13]), (const float*)dptr(env, argv[14]), i32(env, argv[15])));
}

/* ---- dense matmul ---------------------------------------------------------------
 * matmul(ctx, a, b, out, m, n, k, batch, strideA, strideB, strideC, transA, transB, alpha, dtypeA, dtypeB, outDtype,
 *        castA, castB, epilogue?, planOnly) -> undefined, or the receipt (Int32Array) when planOnly */
FN(Matmul) {
  ARGS(21); CTX(0); tl_epilogue e; const tl_epilogue* ep = read_epilogue(env, argv[19], &e);
  tl_plan_receipt r; memset(&r, 0, sizeof(r));
  const int plan_only = i32(env, argv[20]) != 0;
  int32_t st = tl_matmul(c, dptr(env, argv[1]), dptr(env, argv[2]), dptr(env, argv[3]), i64(env, argv[4]), i64(env, argv[5]), i64(env, argv[6]),
                         i64(env, argv[7]), i64(env, argv[8]), i64(env, argv[9]), i64(env, argv[10]), i32(env, argv[11]), i32(env, argv[12]),
                         (float)f64(env, argv[13]), i32(env, argv[14]), i32(env, argv[15]), i32(env, argv[16]), i32(env, argv[17]),
                         i32(env, argv[18]), ep, plan_only ? &r : NULL);
  if (st != TL_OK || !plan_only) return check(env, c, st);
  return receipt_value(env, &r);
}

/* ---- selection, counters, autotune ------------------------------------------------ */
/* planQmatmul(ctx, m, n, k, aDtype, outDtype, qdesc, epilogue?) -> receipt Int32Array */
FN(PlanQmatmul) {
  ARGS(8); CTX(0); tl_quant_desc q; tl_epilogue e; tl_plan_receipt r;
  if (!read_qdesc(env, argv[6], &q)) return undef(env);
  const tl_epilogue* ep = read_epilogue(env, argv[7], &e);
  if (tl_plan_qmatmul(c, i64(env, argv[1]), i64(env, argv[2]), i64(env, argv[3]), i32(env, argv[4]), i32(env, argv[5]), &q, ep, &r) != TL_OK)
    return check(env, c, -1);
  return receipt_value(env, &r);
}
FN(VariantName) { ARGS(1); tl_variant v; if (!read_variant(env, argv[0], &v)) return undef(env); return str(env, tl_variant_name(&v)); }
/* forceVariant(ctx, variant | null) */
FN(ForceVariant) {
  ARGS(2); CTX(0); tl_variant v;
  if (type_of(env, argv[1]) != napi_object) return check(env, c, tl_force_variant(c, NULL));
  if (!read_variant(env, argv[1], &v)) return undef(env);
  return check(env, c, tl_force_variant(c, &v));
}
FN(ClassifyShape) { ARGS(4); return num(env, tl_classify_shape(i64(env, argv[0]), i64(env, argv[1]), i64(env, argv[2]), i64(env, argv[3]))); }
FN(ShapeClassName) { ARGS(1); return str(env, tl_shape_class_name(i32(env, argv[0]))); }
FN(CounterGet) { ARGS(2); CTX(0); return num(env, (double)tl_counter_get(c, i32(env, argv[1]))); }
FN(CountersReset) { ARGS(1); CTX(0); return check(env, c, tl_counters_reset(c)); }
FN(AutotuneSetEnabled) { ARGS(2); CTX(0); return check(env, c, tl_autotune_set_enabled(c, i32(env, argv[1]))); }
FN(AutotuneIsEnabled) { ARGS(1); CTX(0); return num(env, tl_autotune_is_enabled(c)); }
/* pretune(ctx, shapes BigInt64Array [m, n, k, ...], aDtype, outDtype, qdesc): the shape count is the array's own length / 3 */
FN(Pretune) {
  ARGS(5); CTX(0); size_t bytes = 0; const int64_t* sh = (const int64_t*)host_ptr(env, argv[1], &bytes); tl_quant_desc q;
  if (!read_qdesc(env, argv[4], &q)) return undef(env);
  if (bytes % sizeof(tl_shape) != 0) { napi_throw_error(env, NULL, "pretune: shapes must hold whole [m, n, k] triples"); return undef(env); }
  return check(env, c, tl_pretune(c, (const tl_shape*)sh, (int32_t)(bytes / sizeof(tl_shape)), i32(env, argv[2]), i32(env, argv[3]), &q));
}
/* tuneSeed(ctx, m, n, k, aDtype, qdesc, variant) */
FN(TuneSeed) {
  ARGS(7); CTX(0); tl_quant_desc q; tl_variant v;
  if (!read_qdesc(env, argv[5], &q) || !read_variant(env, argv[6], &v)) return undef(env);
  return check(env, c, tl_tune_seed(c, i64(env, argv[1]), i64(env, argv[2]), i64(env, argv[3]), i32(env, argv[4]), &q, &v));
}
/* tuneGet(ctx, m, n, k, aDtype, qdesc) -> variant Int32Array | undefined */
FN(TuneGet) {
  ARGS(6); CTX(0); tl_quant_desc q; tl_variant v;
  if (!read_qdesc(env, argv[5], &q)) return undef(env);
  int32_t st = tl_tune_get(c, i64(env, argv[1]), i64(env, argv[2]), i64(env, argv[3]), i32(env, argv[4]), &q, &v);
  if (st < 0) return check(env, c, st);
  return st == 1 ? make_i32_array(env, (const int32_t*)&v, 6) : undef(env);
}
FN(TuneClear) { ARGS(1); CTX(0); return check(env, c, tl_tune_clear(c)); }
FN(TuneRunCount) { ARGS(1); CTX(0); return num(env, (double)tl_tune_run_count(c)); }
FN(TuneExportJson) {
  ARGS(1); CTX(0); size_t need = 0;
  if (tl_tune_export_json(c, NULL, 0, &need) != TL_OK) return check(env, c, -1);
  char* buf = (char*)malloc(need + 1);
  int32_t st = tl_tune_export_json(c, buf, need + 1, &need);
  napi_value r = st == TL_OK ? str(env, buf) : check(env, c, st);
  free(buf);
  return r;
}
FN(TuneImportJson) {
  ARGS(2); CTX(0); size_t len = 0;
  napi_get_value_string_utf8(env, argv[1], NULL, 0, &len);
  char* buf = (char*)malloc(len + 1);
  napi_get_value_string_utf8(env, argv[1], buf, len + 1, &len);
  int32_t st = tl_tune_import_json(c, buf);
  free(buf);
  return check(env, c, st);
}

/* ---- graphs and events ------------------------------------------------------------ */
FN(GraphBegin) { ARGS(1); CTX(0); return check(env, c, tl_graph_begin(c)); }
FN(GraphEnd) { ARGS(1); CTX(0); tl_graph* g = NULL; if (tl_graph_end(c, &g) != TL_OK) return check(env, c, -1); return big(env, (uint64_t)(uintptr_t)g); }
FN(GraphLaunch) { ARGS(2); CTX(0); return check(env, c, tl_graph_launch(c, (tl_graph*)hptr(env, argv[1]))); }
FN(GraphDestroy) { ARGS(2); CTX(0); return check(env, c, tl_graph_destroy(c, (tl_graph*)hptr(env, argv[1]))); }
FN(EventCreate) { ARGS(1); CTX(0); tl_event* e = NULL; if (tl_event_create(c, &e) != TL_OK) return check(env, c, -1); return big(env, (uint64_t)(uintptr_t)e); }
FN(EventRecord) { ARGS(2); CTX(0); return check(env, c, tl_event_record(c, (tl_event*)hptr(env, argv[1]))); }
FN(EventElapsedMs) {
  ARGS(3); CTX(0); float ms = 0.f;
  if (tl_event_elapsed_ms(c, (tl_event*)hptr(env, argv[1]), (tl_event*)hptr(env, argv[2]), &ms) != TL_OK) return check(env, c, -1);
  return num(env, ms);
}
FN(EventSynchronize) {
  ARGS(2); CTX(0);
  if (tl_event_synchronize(c, (tl_event*)hptr(env, argv[1])) != TL_OK) napi_throw_error(env, NULL, "tlcuda: eventSynchronize failed");
  return undef(env);
}
FN(EventDestroy) { ARGS(2); CTX(0); return check(env, c, tl_event_destroy(c, (tl_event*)hptr(env, argv[1]))); }

/* ---- multi-GPU -------------------------------------------------------------------- */
FN(CommUniqueId) { ARGS(1); (void)argv; uint8_t id[TL_COMM_ID_BYTES]; if (tl_comm_unique_id(id) != TL_OK) { napi_throw_error(env, NULL, tl_last_error(NULL)); return undef(env); } return make_u8_array(env, id, sizeof(id)); }
/* commInit(ctx, rank, world, id Uint8Array(128)) */
FN(CommInit) {
  ARGS(4); CTX(0); size_t n = 0; const void* id = host_ptr(env, argv[3], &n);
  if (n != TL_COMM_ID_BYTES) { napi_throw_error(env, NULL, "commInit: the id is 128 bytes"); return undef(env); }
  return check(env, c, tl_comm_init(c, i32(env, argv[1]), i32(env, argv[2]), id));
}
FN(CommDestroy) { ARGS(1); CTX(0); return check(env, c, tl_comm_destroy(c)); }
FN(AllgatherCols) { ARGS(6); CTX(0); return check(env, c, tl_allgather_cols(c, dptr(env, argv[1]), dptr(env, argv[2]), i64(env, argv[3]), i64(env, argv[4]), i32(env, argv[5]))); }
FN(AllreduceSum) { ARGS(4); CTX(0); return check(env, c, tl_allreduce_sum(c, dptr(env, argv[1]), i64(env, argv[2]), i32(env, argv[3]))); }
/* p2pCreate(ctx, maxBytes) -> Uint8Array(64) handle to send to the peers */
FN(P2pCreate) {
  ARGS(2); CTX(0); uint8_t h[TL_P2P_HANDLE_BYTES];
  if (tl_p2p_create(c, (size_t)i64(env, argv[1]), h) != TL_OK) return check(env, c, -1);
  return make_u8_array(env, h, sizeof(h));
}
/* p2pAttach(ctx, handles Uint8Array(world * 64), in rank order) */
FN(P2pAttach) {
  ARGS(2); CTX(0); size_t n = 0; const void* h = host_ptr(env, argv[1], &n);
  if (n == 0 || n % TL_P2P_HANDLE_BYTES != 0) { napi_throw_error(env, NULL, "p2pAttach: handles are 64 bytes per rank"); return undef(env); }
  return check(env, c, tl_p2p_attach(c, h));
}
FN(P2pAttachLoopback) { ARGS(2); CTX(0); return check(env, c, tl_p2p_attach_loopback(c, i32(env, argv[1]))); }
FN(P2pReset) { ARGS(1); CTX(0); return check(env, c, tl_p2p_reset(c)); }
FN(AllreduceSumP2p) { ARGS(5); CTX(0); return check(env, c, tl_allreduce_sum_p2p(c, dptr(env, argv[1]), dptr(env, argv[2]), i64(env, argv[3]), i32(env, argv[4]))); }

/* allreduceSumP2pF32To(ctx, srcF32, dst, dstDtype, count) */
FN(AllreduceSumP2pF32To) { ARGS(5); CTX(0); return check(env, c, tl_allreduce_sum_p2p_f32_to(c, (const float*)dptr(env, argv[1]), dptr(env, argv[2]), i32(env, argv[3]), i64(env, argv[4]))); }

#define EXPORT(js, fn) {js, 0, fn, 0, 0, 0, 0, 0}
napi_value napi_register_module_v1(napi_env env, napi_value exports) {
  const napi_property_descriptor props[] = {
      EXPORT("ctxCreate", CtxCreate), EXPORT("ctxDestroy", CtxDestroy), EXPORT("sync", Sync),
      EXPORT("asyncErrorCount", AsyncErrorCount), EXPORT("lastError", LastError), EXPORT("ctxStream", CtxStream),
      EXPORT("deviceSmCount", DeviceSmCount), EXPORT("setOption", SetOption), EXPORT("getOption", GetOption),
      EXPORT("alloc", Alloc), EXPORT("view", View), EXPORT("free", Free), EXPORT("ptrOf", PtrOf), EXPORT("upload", Upload),
      EXPORT("download", Download), EXPORT("downloadAsync", DownloadAsync), EXPORT("hostAllocPinned", HostAllocPinned),
      EXPORT("hostFreePinned", HostFreePinned), EXPORT("memset", Memset), EXPORT("copy2d", Copy2d),
      EXPORT("quantizeLinearWeight", QuantizeLinearWeight), EXPORT("quantizeLinearWeightDevice", QuantizeLinearWeightDevice),
      EXPORT("f32ToF16Bits", F32ToF16Bits), EXPORT("f16BitsToF32", F16BitsToF32),
      EXPORT("qgemvNt", QgemvNt), EXPORT("qgemvNtBatched", QgemvNtBatched), EXPORT("qgemvChainCreate", QgemvChainCreate),
      EXPORT("qgemvChainLaunch", QgemvChainLaunch), EXPORT("qgemvChainDestroy", QgemvChainDestroy),
      EXPORT("qgemvNtStaticScratch", QgemvNtStaticScratch), EXPORT("qgemmNt", QgemmNt), EXPORT("qmatmulNt", QmatmulNt),
      EXPORT("dequantInt8", DequantInt8), EXPORT("unpackInt8", UnpackInt8), EXPORT("quantizeLinearWeightInt4", QuantizeLinearWeightInt4),
      EXPORT("dequantInt4", DequantInt4), EXPORT("unpackInt4", UnpackInt4), EXPORT("matmul", Matmul),
      EXPORT("rmsnorm", Rmsnorm), EXPORT("rope", Rope), EXPORT("decodeAttention", DecodeAttention), EXPORT("attention", Attention),
      EXPORT("unaryOp", UnaryOp), EXPORT("binaryOp", BinaryOp), EXPORT("transpose2d", Transpose2d),
      EXPORT("planQmatmul", PlanQmatmul), EXPORT("variantName", VariantName), EXPORT("forceVariant", ForceVariant),
      EXPORT("classifyShape", ClassifyShape), EXPORT("shapeClassName", ShapeClassName),
      EXPORT("counterGet", CounterGet), EXPORT("countersReset", CountersReset),
      EXPORT("autotuneSetEnabled", AutotuneSetEnabled), EXPORT("autotuneIsEnabled", AutotuneIsEnabled), EXPORT("pretune", Pretune),
      EXPORT("tuneSeed", TuneSeed), EXPORT("tuneGet", TuneGet), EXPORT("tuneClear", TuneClear), EXPORT("tuneRunCount", TuneRunCount),
      EXPORT("tuneExportJson", TuneExportJson), EXPORT("tuneImportJson", TuneImportJson),
      EXPORT("graphBegin", GraphBegin), EXPORT("graphEnd", GraphEnd), EXPORT("graphLaunch", GraphLaunch),
      EXPORT("graphDestroy", GraphDestroy), EXPORT("eventCreate", EventCreate), EXPORT("eventRecord", EventRecord),
      EXPORT("eventElapsedMs", EventElapsedMs), EXPORT("eventSynchronize", EventSynchronize), EXPORT("eventDestroy", EventDestroy),
      EXPORT("commUniqueId", CommUniqueId), EXPORT("commInit", CommInit), EXPORT("commDestroy", CommDestroy),
      EXPORT("allgatherCols", AllgatherCols), EXPORT("allreduceSum", AllreduceSum), EXPORT("p2pCreate", P2pCreate),
      EXPORT("p2pAttach", P2pAttach), EXPORT("p2pAttachLoopback", P2pAttachLoopback), EXPORT("p2pReset", P2pReset),
      EXPORT("allreduceSumP2p", AllreduceSumP2p), EXPORT("allreduceSumP2pF32To", AllreduceSumP2pF32To), EXPORT("qgemvNtAllreduce", QgemvNtAllreduce), EXPORT("qgemvNtPush", QgemvNtPush),
      EXPORT("reducePending", ReducePending),
  };
  napi_define_properties(env, exports, sizeof(props) / sizeof(props[0]), props);
  return exports;
}
