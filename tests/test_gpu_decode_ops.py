"""The other ops of one Qwen3 decode step (row f2) against f64 numpy restatements of the reference's
definitions -- rmsnorm (src/ops/semantic/composite.ts:156-170), the half-split rotation
(src/backend/webgpu/rope-kernel.ts:1-93), the decomposed decode attention with repeated KV heads
(packages/qwen3-browser/src/model.ts:171-180, 292-312) -- and one whole decoder layer step
(model.ts:220-420) with int8-64 quantized projections through the backend, end to end."""
import numpy as np
import pytest

from oracle import oracle as orc
from torchlette_b200 import backend as tb

pytestmark = pytest.mark.gpu


def np_rmsnorm(x, w, eps):
    x = x.astype(np.float64)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w.astype(np.float64)


def np_rope(qk, cos, sin, sin_scale=1.0):
    """qk [..., S, D]; cos / sin [S, D/2]."""
    qk = qk.astype(np.float64)
    half = qk.shape[-1] // 2
    a, b = qk[..., :half], qk[..., half:]
    c, s = cos.astype(np.float64), sin.astype(np.float64) * sin_scale
    return np.concatenate([a * c - b * s, b * c + a * s], -1)


def np_decode_attention(q, k, v, scale, mask=None):
    """q [B,H,D]; k, v [B,kvH,L,D] -> [B,H,D]."""
    b, h, d = q.shape
    rep = h // k.shape[1]
    ke, ve = np.repeat(k.astype(np.float64), rep, axis=1), np.repeat(v.astype(np.float64), rep, axis=1)
    s = np.einsum("bhd,bhld->bhl", q.astype(np.float64), ke) * scale
    if mask is not None:
        s = s + mask.astype(np.float64)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    return np.einsum("bhl,bhld->bhd", p, ve)


def _f32(be, arr, shape=None):
    arr = np.ascontiguousarray(arr, dtype=np.float32)
    return be.ops.tensorFromArray(arr, list(shape or arr.shape), "f32")


@pytest.mark.parametrize("rows,cols", [(1, 4096), (16, 128), (7, 300), (64, 64)])
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_rmsnorm(backend, rows, cols, dtype):
    be = backend
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 3
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    xt = be.ops.tensorFromArray(x.astype(np.float16) if dtype == "f16" else x, [rows, cols], dtype)
    xv = x.astype(np.float16).astype(np.float32) if dtype == "f16" else x
    wt = _f32(be, w)
    y = be.ops.rmsnorm(xt, wt, 1e-6)
    ref = np_rmsnorm(xv, w, 1e-6)
    np.testing.assert_allclose(np.asarray(be.ops.read(y), np.float64), ref, rtol=2e-3 if dtype == "f16" else 2e-6, atol=2e-3 if dtype == "f16" else 2e-6)
    for t in (xt, wt, y):
        t.destroy()


def test_rope_offsets_and_inverse(backend):
    be = backend
    b, h, s, d, max_s = 2, 3, 4, 64, 32
    rng = np.random.default_rng(4)
    qk = rng.standard_normal((b, h, s, d)).astype(np.float32)
    pos = np.arange(max_s)[:, None] * (1.0 / 10000 ** (np.arange(d // 2)[None, :] / (d // 2)))
    cos, sin = np.cos(pos).astype(np.float32), np.sin(pos).astype(np.float32)
    qt, ct, st = _f32(be, qk), _f32(be, cos), _f32(be, sin)
    start = 5  # a narrow() view of the persistent tables: rows [start, start + s)
    y = be.ops.fusedRoPE(qt, ct, st, {"cosOffset": start * (d // 2), "sinOffset": start * (d // 2)})
    ref = np_rope(qk, cos[start:start + s], sin[start:start + s])
    np.testing.assert_allclose(be.ops.read(y), ref, rtol=1e-5, atol=1e-5)
    back = be.ops.fusedRoPE(y, ct, st, {"cosOffset": start * (d // 2), "sinOffset": start * (d // 2), "sinScale": -1.0})
    np.testing.assert_allclose(be.ops.read(back), qk, rtol=1e-5, atol=1e-5)
    odd = _f32(be, np.zeros((1, 1, 3), np.float32))
    with pytest.raises(tb.TlError):
        be.ops.fusedRoPE(odd, ct, st)
    for t in (qt, ct, st, y, back, odd):
        t.destroy()


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("kv_len,masked", [(1, False), (37, False), (600, True)])
def test_decode_attention_with_repeated_kv_heads(backend, dtype, kv_len, masked):
    be = backend
    b, h, kvh, d, cap = 2, 8, 2, 64, 640
    rng = np.random.default_rng(kv_len)
    q = rng.standard_normal((b, h, 1, d)).astype(np.float32)
    k = rng.standard_normal((b, kvh, cap, d)).astype(np.float32)
    v = rng.standard_normal((b, kvh, cap, d)).astype(np.float32)
    mask = np.where(rng.uniform(size=kv_len) < 0.2, -1e9, 0.0).astype(np.float32) if masked else None
    if masked:
        mask[0] = 0.0
    conv = (lambda a: a.astype(np.float16)) if dtype == "f16" else (lambda a: a)
    qt = be.ops.tensorFromArray(conv(q), list(q.shape), dtype)
    kt = be.ops.tensorFromArray(conv(k), list(k.shape), dtype)
    vt = be.ops.tensorFromArray(conv(v), list(v.shape), dtype)
    mt = _f32(be, mask) if masked else None
    out = be.ops.decodeAttention(qt, kt, vt, kv_len, 1.0 / np.sqrt(d), mt)
    assert out.shape == [b, 1, h * d]
    f = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == "f16" else (lambda a: a)
    ref = np_decode_attention(f(q)[:, :, 0], f(k)[:, :, :kv_len], f(v)[:, :, :kv_len], 1.0 / np.sqrt(d), mask)
    tol = 3e-3 if dtype == "f16" else 2e-5
    np.testing.assert_allclose(np.asarray(be.ops.read(out), np.float64).reshape(b, h, d), ref, rtol=tol, atol=tol)
    for t in (qt, kt, vt, out) + ((mt,) if mt else ()):
        t.destroy()


def test_one_decoder_layer_step_end_to_end(backend):
    """model.ts:220-420 for one new token per sequence with a KV cache: input norm, q / k / v (int8-64),
    per-head q / k norm, RoPE at the current position, cache append, attention over the cache, o_proj,
    residual, post-attention norm, silu(gate) * up, down_proj, residual."""
    be = backend
    B_, hidden, heads, kvh, hd, inter, cap, pos, eps = 2, 256, 4, 2, 64, 512, 16, 5, 1e-6
    rng = np.random.default_rng(2024)
    G = 64

    def qweight(n, k):
        w = (rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32)
        packed, scales = be.quantizeLinearWeight(w, G)
        return be.createQuantizedWeight(packed, scales, n, k, tb.resolveWeightFormat("int8-64")), orc.dequantize_to_f32(packed, scales, k, G)

    (wq, wq_r), (wk, wk_r), (wv, wv_r) = qweight(heads * hd, hidden), qweight(kvh * hd, hidden), qweight(kvh * hd, hidden)
    (wo, wo_r), (wg, wg_r), (wu, wu_r), (wd, wd_r) = qweight(hidden, heads * hd), qweight(inter, hidden), qweight(inter, hidden), qweight(hidden, inter)
    n_in, n_post = rng.uniform(0.5, 1.5, hidden).astype(np.float32), rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    n_q, n_k = rng.uniform(0.5, 1.5, hd).astype(np.float32), rng.uniform(0.5, 1.5, hd).astype(np.float32)
    x = rng.standard_normal((B_, 1, hidden)).astype(np.float32)
    k_past = rng.standard_normal((B_, kvh, cap, hd)).astype(np.float32)
    v_past = rng.standard_normal((B_, kvh, cap, hd)).astype(np.float32)
    k_past[:, :, pos:] = 0
    v_past[:, :, pos:] = 0
    ang = np.arange(cap)[:, None] * (1.0 / 1e6 ** (np.arange(hd // 2)[None, :] / (hd // 2)))
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)

    # ---- the backend ----
    ops = be.ops
    xt = _f32(be, x.reshape(B_, hidden))
    t_in, t_post, t_q, t_k = _f32(be, n_in), _f32(be, n_post), _f32(be, n_q), _f32(be, n_k)
    ct, st = _f32(be, cos), _f32(be, sin)
    kc, vc = _f32(be, k_past), _f32(be, v_past)
    h0 = ops.rmsnorm(xt, t_in, eps)
    q, k, v = be.linear(h0, wq), be.linear(h0, wk), be.linear(h0, wv)
    qn = ops.rmsnorm(ops.reshape(q, [B_, heads, hd]), t_q, eps)
    kn = ops.rmsnorm(ops.reshape(k, [B_, kvh, hd]), t_k, eps)
    off = {"cosOffset": pos * (hd // 2), "sinOffset": pos * (hd // 2)}
    qr = ops.fusedRoPE(ops.reshape(qn, [B_, heads, 1, hd]), ct, st, off)
    kr = ops.fusedRoPE(ops.reshape(kn, [B_, kvh, 1, hd]), ct, st, off)
    ops.kvAppend(kc, kr, pos)
    ops.kvAppend(vc, v, pos)
    attn = ops.decodeAttention(qr, kc, vc, pos + 1, 1.0 / np.sqrt(hd))
    o = be.linear(ops.reshape(attn, [B_, heads * hd]), wo)
    h1 = ops.add(xt, o)
    h1n = ops.rmsnorm(h1, t_post, eps)
    gu = be.swiglu(h1n, wg, wu, "f32")
    d = be.linear(gu, wd)
    out = ops.add(h1, d)
    got = np.asarray(ops.read(out), np.float64)

    # ---- f64 numpy restatement of the same step on the dequantized weights ----
    def lin(a, w):
        return a.astype(np.float64) @ w.astype(np.float64).T
    x2 = x.reshape(B_, hidden)
    r0 = np_rmsnorm(x2, n_in, eps)
    rq = np_rmsnorm(lin(r0, wq_r).reshape(B_, heads, hd), n_q, eps)
    rk = np_rmsnorm(lin(r0, wk_r).reshape(B_, kvh, hd), n_k, eps)
    rv = lin(r0, wv_r).reshape(B_, kvh, hd)
    rq = np_rope(rq[:, :, None, :], cos[pos:pos + 1], sin[pos:pos + 1])[:, :, 0]
    rk = np_rope(rk[:, :, None, :], cos[pos:pos + 1], sin[pos:pos + 1])[:, :, 0]
    kk, vv = k_past.astype(np.float64).copy(), v_past.astype(np.float64).copy()
    kk[:, :, pos], vv[:, :, pos] = rk, rv
    ra = np_decode_attention(rq, kk[:, :, :pos + 1], vv[:, :, :pos + 1], 1.0 / np.sqrt(hd)).reshape(B_, heads * hd)
    r1 = x2 + lin(ra, wo_r)
    r1n = np_rmsnorm(r1, n_post, eps)
    g = lin(r1n, wg_r)
    ref = r1 + lin(g / (1 + np.exp(-g)) * lin(r1n, wu_r), wd_r)
    assert float(np.max(np.abs(got - ref) / np.maximum(1.0, np.abs(ref)))) <= 1e-3
    # the cache now holds this step's rotated k and its v at `pos`
    np.testing.assert_allclose(ops.read(kc)[:, :, pos], rk, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(ops.read(vc)[:, :, pos], rv, rtol=1e-4, atol=1e-4)
    assert be.getGpuUncapturedErrorCount() == 0


def np_causal_attention(q, k, v, scale):
    """q [B,H,S,D]; k, v [B,kvH,L,D], L >= S; query s sees keys <= L - S + s.  Returns [B,S,H,D]."""
    b, h, s, d = q.shape
    length = k.shape[2]
    rep = h // k.shape[1]
    ke, ve = np.repeat(k.astype(np.float64), rep, axis=1), np.repeat(v.astype(np.float64), rep, axis=1)
    sc = np.einsum("bhsd,bhld->bhsl", q.astype(np.float64), ke) * scale
    vis = np.arange(length)[None, :] <= (length - s + np.arange(s))[:, None]
    sc = np.where(vis[None, None], sc, -np.inf)
    sc = sc - sc.max(-1, keepdims=True)
    p = np.exp(sc)
    p /= p.sum(-1, keepdims=True)
    return np.einsum("bhsl,bhld->bshd", p, ve)


@pytest.mark.parametrize("s_q,kv_len", [(7, 7), (5, 12), (1, 9), (33, 33)])
def test_causal_attention_prefill_and_multi_token_with_cache(backend, s_q, kv_len):
    be = backend
    b, h, kvh, d, cap = 2, 6, 3, 32, 40
    rng = np.random.default_rng(s_q * 100 + kv_len)
    q = rng.standard_normal((b, h, s_q, d)).astype(np.float32)
    k = rng.standard_normal((b, kvh, cap, d)).astype(np.float32)
    v = rng.standard_normal((b, kvh, cap, d)).astype(np.float32)
    qt, kt, vt = _f32(be, q), _f32(be, k), _f32(be, v)
    out = be.ops.attention(qt, kt, vt, kv_len, 1.0 / np.sqrt(d), causal=True)
    assert out.shape == [b, s_q, h * d]
    ref = np_causal_attention(q, k[:, :, :kv_len], v[:, :, :kv_len], 1.0 / np.sqrt(d))
    np.testing.assert_allclose(np.asarray(be.ops.read(out), np.float64).reshape(b, s_q, h, d), ref, rtol=2e-5, atol=2e-5)
    with pytest.raises(tb.TlError):
        be.ops.attention(qt, kt, vt, s_q - 1 if s_q > 1 else 0, 1.0, causal=True)  # fewer keys than queries
    for t in (qt, kt, vt, out):
        t.destroy()
