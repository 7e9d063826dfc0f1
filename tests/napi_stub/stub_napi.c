/*
 * A fake of the N-API calls that tl_napi.c makes, fakes of the handful of tl_* functions the
 * scenarios below reach, and a main() that drives the addon's exports the way node would.
 * Test infrastructure only (there is no node runtime where the tests run): it checks what the
 * shim hands to the C ABI -- byte counts for subarray views, shape counts, epilogue inputs,
 * finalizer behaviour, the Promise path of downloadAsync -- and prints one "ok <name>" line
 * per check; any failed check prints "FAIL ..." and exits 1.
 * Linked with: gcc tl_napi.c stub_napi.c -Wl,--unresolved-symbols=ignore-all (the tl_*
 * functions no scenario calls stay undefined).
 */
#define _POSIX_C_SOURCE 200809L
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "tlcuda.h"

typedef struct V V;
typedef V* napi_value;
typedef struct Env* napi_env;
typedef V* napi_ref;
typedef V* napi_deferred;
typedef struct CbInfo* napi_callback_info;
typedef struct Work* napi_async_work;
typedef int napi_status;
typedef napi_value (*napi_callback)(napi_env, napi_callback_info);
typedef void (*napi_finalize)(napi_env, void*, void*);
typedef void (*exec_cb)(napi_env, void*);
typedef void (*done_cb)(napi_env, napi_status, void*);
typedef struct { const char* utf8name; napi_value name; napi_callback method; napi_callback getter; napi_callback setter; napi_value value; int attributes; void* data; } napi_property_descriptor;
enum { T_UNDEF, T_NULL, T_BOOL, T_NUM, T_STR, T_SYM, T_OBJ, T_FN, T_EXT, T_BIG };
struct V {
  int type; double num; uint64_t big; char* s;
  void* ext; napi_finalize fin; void* hint;                       /* external / external arraybuffer */
  int is_typed, ta_type; size_t len, off; void* data; V* ab;     /* typed array */
  int is_ab; size_t ab_len;                                       /* array buffer */
  int is_array, n; V* elems[16]; const char* keys[16];           /* array / object */
  int settled; V* result;                                         /* promise: 1 resolved, 2 rejected */
};
struct CbInfo { size_t argc; V** argv; };
struct Work { exec_cb exec; done_cb done; void* data; };
struct Env { char thrown[512]; int has_thrown; };

static V* nv(int type) { V* v = (V*)calloc(1, sizeof(V)); v->type = type; return v; }

napi_status napi_get_cb_info(napi_env e, napi_callback_info i, size_t* argc, napi_value* argv, napi_value* t, void** d) {
  (void)e; (void)t; (void)d;
  for (size_t k = 0; k < *argc; ++k) argv[k] = k < i->argc ? i->argv[k] : nv(T_UNDEF);
  return 0;
}
napi_status napi_typeof(napi_env e, napi_value v, int* t) { (void)e; *t = v->type; return 0; }
napi_status napi_get_value_int32(napi_env e, napi_value v, int32_t* r) { (void)e; *r = (int32_t)v->num; return v->type == T_NUM ? 0 : 1; }
napi_status napi_get_value_int64(napi_env e, napi_value v, int64_t* r) { (void)e; *r = (int64_t)v->num; return v->type == T_NUM ? 0 : 1; }
napi_status napi_get_value_double(napi_env e, napi_value v, double* r) { (void)e; *r = v->num; return v->type == T_NUM ? 0 : 1; }
napi_status napi_get_value_bigint_uint64(napi_env e, napi_value v, uint64_t* r, int* ok) { (void)e; *r = v->big; *ok = 1; return 0; }
napi_status napi_get_value_string_utf8(napi_env e, napi_value v, char* buf, size_t cap, size_t* len) {
  (void)e; size_t n = v->s ? strlen(v->s) : 0;
  if (!buf) { *len = n; return 0; }
  if (n > cap - 1) n = cap - 1;
  memcpy(buf, v->s, n); buf[n] = 0; if (len) *len = n; return 0;
}
napi_status napi_get_value_external(napi_env e, napi_value v, void** p) { (void)e; *p = v->ext; return 0; }
napi_status napi_create_bigint_uint64(napi_env e, uint64_t x, napi_value* r) { (void)e; *r = nv(T_BIG); (*r)->big = x; return 0; }
napi_status napi_create_int32(napi_env e, int32_t x, napi_value* r) { (void)e; *r = nv(T_NUM); (*r)->num = x; return 0; }
napi_status napi_create_double(napi_env e, double x, napi_value* r) { (void)e; *r = nv(T_NUM); (*r)->num = x; return 0; }
napi_status napi_create_string_utf8(napi_env e, const char* s, size_t n, napi_value* r) { (void)e; (void)n; *r = nv(T_STR); (*r)->s = strdup(s); return 0; }
napi_status napi_create_external(napi_env e, void* d, napi_finalize f, void* h, napi_value* r) { (void)e; *r = nv(T_EXT); (*r)->ext = d; (*r)->fin = f; (*r)->hint = h; return 0; }
napi_status napi_create_arraybuffer(napi_env e, size_t n, void** d, napi_value* r) { (void)e; *r = nv(T_OBJ); (*r)->is_ab = 1; (*r)->ab_len = n; (*r)->data = calloc(1, n ? n : 1); *d = (*r)->data; return 0; }
napi_status napi_create_external_arraybuffer(napi_env e, void* d, size_t n, napi_finalize f, void* h, napi_value* r) { (void)e; *r = nv(T_OBJ); (*r)->is_ab = 1; (*r)->ab_len = n; (*r)->data = d; (*r)->fin = f; (*r)->hint = h; return 0; }
napi_status napi_create_typedarray(napi_env e, int type, size_t len, napi_value ab, size_t off, napi_value* r) {
  (void)e; *r = nv(T_OBJ); (*r)->is_typed = 1; (*r)->ta_type = type; (*r)->len = len; (*r)->off = off; (*r)->ab = ab; (*r)->data = (char*)ab->data + off; return 0;
}
napi_status napi_get_undefined(napi_env e, napi_value* r) { (void)e; *r = nv(T_UNDEF); return 0; }
napi_status napi_throw_error(napi_env e, const char* code, const char* msg) { (void)code; e->has_thrown = 1; snprintf(e->thrown, sizeof(e->thrown), "%s", msg ? msg : ""); return 0; }
napi_status napi_get_typedarray_info(napi_env e, napi_value v, int* type, size_t* len, void** data, napi_value* ab, size_t* off) {
  (void)e; if (!v->is_typed) return 1;
  *type = v->ta_type; *len = v->len; *data = v->data; *ab = v->ab; *off = v->off; return 0;
}
napi_status napi_get_arraybuffer_info(napi_env e, napi_value v, void** d, size_t* n) { (void)e; *d = v->data; *n = v->ab_len; return 0; }
static napi_property_descriptor g_props[128]; static size_t g_nprops;
napi_status napi_define_properties(napi_env e, napi_value o, size_t n, const napi_property_descriptor* p) { (void)e; (void)o; memcpy(g_props, p, n * sizeof(*p)); g_nprops = n; return 0; }
napi_status napi_get_array_length(napi_env e, napi_value v, uint32_t* n) { (void)e; *n = v->is_array ? (uint32_t)v->n : 0; return 0; }
napi_status napi_get_element(napi_env e, napi_value v, uint32_t i, napi_value* r) { (void)e; *r = v->elems[i]; return 0; }
napi_status napi_get_named_property(napi_env e, napi_value v, const char* k, napi_value* r) {
  (void)e;
  for (int i = 0; i < v->n; ++i) if (v->keys[i] && !strcmp(v->keys[i], k)) { *r = v->elems[i]; return 0; }
  *r = nv(T_UNDEF); return 0;
}
napi_status napi_create_reference(napi_env e, napi_value v, uint32_t c, napi_ref* r) { (void)e; (void)c; *r = v; return 0; }
napi_status napi_delete_reference(napi_env e, napi_ref r) { (void)e; (void)r; return 0; }
napi_status napi_get_reference_value(napi_env e, napi_ref r, napi_value* v) { (void)e; *v = r; return 0; }
napi_status napi_create_promise(napi_env e, napi_deferred* d, napi_value* p) { (void)e; *p = nv(T_OBJ); *d = *p; return 0; }
napi_status napi_resolve_deferred(napi_env e, napi_deferred d, napi_value v) { (void)e; d->settled = 1; d->result = v; return 0; }
napi_status napi_reject_deferred(napi_env e, napi_deferred d, napi_value v) { (void)e; d->settled = 2; d->result = v; return 0; }
napi_status napi_create_error(napi_env e, napi_value c, napi_value m, napi_value* r) { (void)e; (void)c; *r = m; return 0; }
static struct Work* g_queued;
napi_status napi_create_async_work(napi_env e, napi_value a, napi_value b, exec_cb x, done_cb d, void* data, napi_async_work* w) {
  (void)e; (void)a; (void)b; *w = (struct Work*)calloc(1, sizeof(struct Work)); (*w)->exec = x; (*w)->done = d; (*w)->data = data; return 0;
}
napi_status napi_queue_async_work(napi_env e, napi_async_work w) { (void)e; g_queued = w; return 0; }  /* run later by the test */
napi_status napi_delete_async_work(napi_env e, napi_async_work w) { (void)e; free(w); return 0; }

/* ---- fakes of the C ABI ---------------------------------------------------------- */
struct tl_ctx { int dummy; };
struct tl_event { int recorded; };
static struct { size_t upload_bytes, download_bytes; const void* upload_src; void* download_dst; int n_shapes; int frees; void* last_free;
                int pinned_live; int events_live; int fail_upload; tl_epilogue epi; int qmatmul_calls; tl_quant_desc q; int64_t shapes[6];
                int ctx_destroyed; } rec;
int32_t tl_ctx_create(int32_t d, tl_ctx** out) { (void)d; *out = (tl_ctx*)calloc(1, sizeof(tl_ctx)); return 0; }
int32_t tl_ctx_destroy(tl_ctx* c) { free(c); rec.ctx_destroyed++; return 0; }
const char* tl_last_error(tl_ctx* c) { (void)c; return "fake: last error text"; }
int32_t tl_sync(tl_ctx* c) { (void)c; return 0; }
int32_t tl_alloc(tl_ctx* c, size_t n, void** p) { (void)c; *p = calloc(1, n); return 0; }
int32_t tl_free(tl_ctx* c, void* p) { (void)c; rec.frees++; rec.last_free = p; free(p); return 0; }
int32_t tl_upload(tl_ctx* c, void* dst, const void* src, size_t n) { (void)c; if (rec.fail_upload) return -1; rec.upload_bytes = n; rec.upload_src = src; memcpy(dst, src, n); return 0; }
int32_t tl_download(tl_ctx* c, void* dst, const void* src, size_t n) { (void)c; rec.download_bytes = n; rec.download_dst = dst; memcpy(dst, src, n); return 0; }
int32_t tl_host_alloc_pinned(tl_ctx* c, size_t n, void** p) { (void)c; *p = calloc(1, n); rec.pinned_live++; return 0; }
int32_t tl_host_free_pinned(tl_ctx* c, void* p) { (void)c; free(p); rec.pinned_live--; return 0; }
int32_t tl_event_create(tl_ctx* c, tl_event** e) { (void)c; *e = (tl_event*)calloc(1, sizeof(tl_event)); rec.events_live++; return 0; }
int32_t tl_event_record(tl_ctx* c, tl_event* e) { (void)c; e->recorded = 1; return 0; }
int32_t tl_event_synchronize(tl_ctx* c, tl_event* e) { (void)c; return e->recorded ? 0 : -3; }
int32_t tl_event_destroy(tl_ctx* c, tl_event* e) { (void)c; free(e); rec.events_live--; return 0; }
int32_t tl_pretune(tl_ctx* c, const tl_shape* s, int32_t n, int32_t a, int32_t o, const tl_quant_desc* q) {
  (void)c; (void)a; (void)o; rec.n_shapes = n; rec.q = *q; memcpy(rec.shapes, s, sizeof(int64_t) * 3 * (n > 2 ? 2 : n)); return 0;
}
int32_t tl_qmatmul_nt(tl_ctx* c, const void* a, int32_t ad, const void* w, const void* s, void* out, int32_t od, int64_t m, int64_t n, int64_t k,
                      const tl_quant_desc* q, float alpha, const tl_epilogue* e) {
  (void)c; (void)a; (void)ad; (void)w; (void)s; (void)out; (void)od; (void)m; (void)n; (void)k; (void)alpha;
  rec.qmatmul_calls++; rec.q = *q; if (e) rec.epi = *e; else memset(&rec.epi, 0, sizeof(rec.epi)); return 0;
}

/* ---- driver ------------------------------------------------------------------- */
extern napi_value napi_register_module_v1(napi_env, napi_value);
static struct Env g_env;
static void fail(const char* fmt, ...) { va_list ap; va_start(ap, fmt); printf("FAIL "); vprintf(fmt, ap); printf("\n"); va_end(ap); exit(1); }
#define EXPECT(cond, name) do { if (!(cond)) fail("%s (line %d)", name, __LINE__); printf("ok %s\n", name); } while (0)
static V* call(const char* name, size_t argc, V** argv) {
  for (size_t i = 0; i < g_nprops; ++i)
    if (!strcmp(g_props[i].utf8name, name)) { struct CbInfo info = {argc, argv}; g_env.has_thrown = 0; return g_props[i].method(&g_env, &info); }
  fail("no export named %s", name); return NULL;
}
static V* number(double x) { V* v = nv(T_NUM); v->num = x; return v; }
static V* typed(int type, V* ab, size_t off, size_t len) { V* r; napi_create_typedarray(&g_env, type, len, ab, off, &r); return r; }
static V* arraybuffer(size_t n) { V* ab; void* d; napi_create_arraybuffer(&g_env, n, &d, &ab); return ab; }
static void finalize(V* v) { if (v->fin) v->fin(&g_env, v->type == T_EXT ? v->ext : v->data, v->hint); v->fin = NULL; }

int main(int argc, char** argv) {
  if (argc > 1 && !strcmp(argv[1], "--list")) {
    napi_register_module_v1(&g_env, nv(T_OBJ));
    for (size_t i = 0; i < g_nprops; ++i) printf("%s\n", g_props[i].utf8name);
    return 0;
  }
  napi_register_module_v1(&g_env, nv(T_OBJ));
  EXPECT(g_nprops >= 68, "exports registered");
  V* a1[1] = {number(0)};
  V* ctx = call("ctxCreate", 1, a1);
  EXPECT(ctx->type == T_EXT && !g_env.has_thrown, "ctxCreate returns an external");

  /* a 1024-byte ArrayBuffer; the view is Float32Array(4) at byte offset 16 */
  V* ab = arraybuffer(1024);
  for (int i = 0; i < 1024; ++i) ((uint8_t*)ab->data)[i] = (uint8_t)i;
  V* view = typed(7 /* float32 */, ab, 16, 4);
  V* a2[2] = {ctx, number(16)};
  V* buf = call("alloc", 2, a2);
  EXPECT(buf->type == T_EXT, "alloc returns an external");
  V* a3[3] = {ctx, buf, view};
  call("upload", 3, a3);
  EXPECT(rec.upload_bytes == 16 && rec.upload_src == (char*)ab->data + 16, "upload copies the view's own 16 bytes");

  V* ab2 = arraybuffer(1024);
  V* view2 = typed(4 /* uint16 */, ab2, 100, 8);
  V* a4[3] = {ctx, view2, buf};
  call("download", 3, a4);
  EXPECT(rec.download_bytes == 16 && rec.download_dst == (char*)ab2->data + 100, "download fills the view's own 16 bytes");
  EXPECT(((uint8_t*)ab2->data)[99] == 0 && ((uint8_t*)ab2->data)[116] == 0 && ((uint8_t*)ab2->data)[100] == 16, "download leaves the rest of the ArrayBuffer alone");

  /* pretune: BigInt64Array(6) inside a 30-element buffer -> exactly 2 shapes */
  V* ab3 = arraybuffer(30 * 8);
  int64_t* sh = (int64_t*)((char*)ab3->data + 24);
  sh[0] = 1; sh[1] = 4096; sh[2] = 14336; sh[3] = 16; sh[4] = 151936; sh[5] = 4096;
  V* shapes = typed(9 /* bigint64 */, ab3, 24, 6);
  V* qab = arraybuffer(16); int32_t qd[4] = {1, 64, 1, 0}; memcpy(qab->data, qd, 16);
  V* q = typed(5 /* int32 */, qab, 0, 4);
  V* a5[5] = {ctx, shapes, number(1), number(1), q};
  call("pretune", 5, a5);
  EXPECT(rec.n_shapes == 2 && rec.shapes[1] == 4096 && rec.shapes[3] == 16 && rec.q.group_size == 64, "pretune passes 2 shapes and the descriptor");

  /* epilogue with one bias input given as a buffer handle */
  V* opsab = arraybuffer(16); int32_t ops[4] = {TL_EPI_BIAS, 0, 0, 0}; memcpy(opsab->data, ops, 16);
  V* inputs = nv(T_OBJ); inputs->is_array = 1; inputs->n = 1; inputs->elems[0] = buf;
  V* epi = nv(T_OBJ); epi->n = 2; epi->keys[0] = "ops"; epi->elems[0] = typed(5, opsab, 0, 4); epi->keys[1] = "inputs"; epi->elems[1] = inputs;
  V* big0 = nv(T_BIG); big0->big = 0x1000;
  V* a13[13] = {ctx, buf, number(1), big0, buf, buf, number(0), number(1), number(8), number(64), q, number(1.0), epi};
  call("qmatmulNt", 13, a13);
  void* bufptr = NULL; { V* pa[1] = {buf}; V* p = call("ptrOf", 1, pa); bufptr = (void*)(uintptr_t)p->big; }
  EXPECT(rec.qmatmul_calls == 1 && rec.epi.n_ops == 1 && rec.epi.ops[0].kind == TL_EPI_BIAS && rec.epi.n_inputs == 1 && rec.epi.inputs[0] == bufptr,
         "epilogue ops and inputs reach the library");

  /* an error status becomes a thrown Error with the library's text */
  rec.fail_upload = 1; call("upload", 3, a3); rec.fail_upload = 0;
  EXPECT(g_env.has_thrown && strstr(g_env.thrown, "fake: last error text"), "a failing call throws tl_last_error");

  /* downloadAsync: nothing lands in the array until the work item has run and completed */
  memset(ab2->data, 0, 1024);
  V* promise = call("downloadAsync", 3, a4);
  EXPECT(promise->settled == 0 && g_queued && ((uint8_t*)ab2->data)[100] == 0 && rec.pinned_live == 1, "downloadAsync returns a pending Promise");
  g_queued->exec(&g_env, g_queued->data);
  EXPECT(promise->settled == 0, "the worker-side wait does not settle the Promise");
  g_queued->done(&g_env, 0, g_queued->data);
  EXPECT(promise->settled == 1 && promise->result == view2 && ((uint8_t*)ab2->data)[100] == 16 && ((uint8_t*)ab2->data)[115] == 31 &&
         ((uint8_t*)ab2->data)[116] == 0 && rec.pinned_live == 0 && rec.events_live == 0, "downloadAsync resolves with the filled view and frees its staging");

  /* views and finalizers */
  V* av[2] = {buf, number(8)};
  V* sub = call("view", 2, av);
  { V* pa[1] = {sub}; V* p = call("ptrOf", 1, pa); EXPECT((void*)(uintptr_t)p->big == (char*)bufptr + 8, "view points 8 bytes into the allocation"); }
  rec.frees = 0;
  finalize(sub);
  EXPECT(rec.frees == 0, "a view's finalizer frees nothing");
  finalize(buf);
  EXPECT(rec.frees == 1 && rec.last_free == bufptr, "a dropped owning buffer is freed once by its finalizer");
  V* buf2 = call("alloc", 2, a2);
  V* af[2] = {ctx, buf2};
  call("free", 2, af);
  finalize(buf2);
  EXPECT(rec.frees == 2, "free() followed by collection frees once");
  V* buf3 = call("alloc", 2, a2);
  V* ad[1] = {ctx};
  call("ctxDestroy", 1, ad);
  EXPECT(rec.ctx_destroyed == 1, "ctxDestroy destroys the context");
  finalize(buf3);
  EXPECT(rec.frees == 2, "a buffer collected after its context is gone is not freed through it");
  call("sync", 1, ad);
  EXPECT(g_env.has_thrown, "a call on a destroyed context throws");
  finalize(ctx);
  EXPECT(rec.ctx_destroyed == 1, "the context is destroyed exactly once");
  printf("ALL OK\n");
  return 0;
}
