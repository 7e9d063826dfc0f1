"""GPU parity of the dense matmul / GEMV + epilogue (tl_matmul through the backend's
dispatchMatmul) against the CPU oracle.

Inputs and tolerances follow the reference's own tests of this op:
test/webgpu/matmul-epilogue.spec.ts:21-27 (values ((i + off) % 7) - 3, rtol = atol = 1e-3,
1e-2 with gelu, including the non-tile-aligned 50 x 70 x 60 product) and
examples/qwen3/probe-gemv.ts:38-39 (GEMV vs f64 over K, N in {33, 128, 1024, 2048}, NN and NT,
f32 x f32 and f32 x f16, relative error <= 5e-4; epilogue battery <= 1e-4 relative).
"""
import numpy as np
import pytest

from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B

pytestmark = pytest.mark.gpu


def _pattern(count, off):
    return (((np.arange(count) + off) % 7) - 3).astype(np.float32)


def _to_dev(be, arr_f32, shape, dtype):
    if dtype == "f32":
        return be.ops.tensorFromArray(arr_f32, shape, "f32"), arr_f32.reshape(shape)
    if dtype == "f16":
        h = arr_f32.astype(np.float16)
        return be.ops.tensorFromArray(h, shape, "f16"), h.astype(np.float32).reshape(shape)
    bits = orc.bf16_bits_rne(arr_f32)
    return be.ops.tensorFromArray(bits, shape, "bf16"), orc.bf16_bits_to_f32(bits).reshape(shape)


def _read_f32(be, t):
    r = be.ops.read(t)
    return orc.bf16_bits_to_f32(r) if t.dtype == "bf16" else np.asarray(r, dtype=np.float32)


def _ref(a, b, bias=None, act=None, alpha=1.0):
    """a [M,K], b [K,N] as f32 values: f64 sequential-k accumulate (the oracle's matmul)."""
    return orc.linear_reference(np.ascontiguousarray(a), np.ascontiguousarray(b.T), bias, act, alpha)


EPILOGUES = [None, ("bias", None), (None, "relu"), (None, "gelu"), (None, "silu"), ("bias", "relu"), ("bias", "gelu")]


@pytest.mark.parametrize("m,k,n", [(64, 64, 64), (50, 70, 60), (1, 128, 96), (130, 33, 257)])
@pytest.mark.parametrize("epi", EPILOGUES)
def test_dense_matmul_epilogue_battery(backend, m, k, n, epi):
    be = backend
    a, a_v = _to_dev(be, _pattern(m * k, 0), [m, k], "f32")
    b, b_v = _to_dev(be, _pattern(k * n, 3), [k, n], "f32")
    bias_v = _pattern(n, 5) * 0.5
    bias_t = be.ops.tensorFromArray(bias_v, [n], "f32")
    chain, act = [], None
    if epi is not None:
        if epi[0]:
            chain.append(("add", bias_t))
        if epi[1]:
            chain.append((epi[1], None))
            act = epi[1]
    opts = {}
    if chain:
        plan = tb.detectMatmulEpilogue(chain)
        opts["epilogue"], opts["epilogueInputs"], _ = plan
    y = be.ops.matmul(a, b, opts)
    got = _read_f32(be, y)
    ref = _ref(a_v, b_v, bias_v if (epi and epi[0]) else None, act)
    tol = 1e-2 if act == "gelu" else 1e-3
    np.testing.assert_allclose(got, ref.reshape(got.shape), rtol=tol, atol=tol)
    for t in (a, b, bias_t, y):
        t.destroy()


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("dtypes", [("f32", "f32", "f32"), ("f16", "f16", "f32"), ("f32", "f16", "f32"),
                                    ("bf16", "bf16", "bf16"), ("f16", "f16", "f16")])
def test_dense_matmul_layouts_and_dtypes(backend, trans_a, trans_b, dtypes):
    be = backend
    m, k, n = 37, 100, 45
    rng = np.random.default_rng(1234)
    av = rng.uniform(-1, 1, m * k).astype(np.float32)
    bv = rng.uniform(-1, 1, k * n).astype(np.float32)
    # the stored buffers: [K,M] when A is a transposed view, [N,K] when B is
    a_t, a_stored = _to_dev(be, av, [k, m] if trans_a else [m, k], dtypes[0])
    b_t, b_stored = _to_dev(be, bv, [n, k] if trans_b else [k, n], dtypes[1])
    a_view = be.ops.transpose(a_t) if trans_a else a_t
    b_view = be.ops.transpose(b_t) if trans_b else b_t
    a_log = a_stored.T if trans_a else a_stored
    b_log = b_stored.T if trans_b else b_stored
    assert be.planMatmul(m, n, k, dtypes[0], dtypes[1], transA=trans_a, transB=trans_b)["variant"].startswith("matmul.tiled")
    y = be.ops.matmul(a_view, b_view, {"outputDtype": dtypes[2]})
    got = _read_f32(be, y)
    ref = _ref(a_log, b_log)
    tol = 1e-4 if dtypes[2] == "f32" else 2e-2
    np.testing.assert_allclose(got, ref, rtol=tol, atol=tol * (1 if dtypes[2] == "f32" else 4))
    for t in (a_t, b_t, y):
        t.destroy()


def test_dense_matmul_cast_on_load_matches_rounded_operands(backend):
    be = backend
    m, k, n = 20, 96, 24
    rng = np.random.default_rng(7)
    av = rng.uniform(-2, 2, m * k).astype(np.float32)
    bv = rng.uniform(-2, 2, k * n).astype(np.float32)
    a, a_v = _to_dev(be, av, [m, k], "f32")
    b, b_v = _to_dev(be, bv, [k, n], "f32")
    y = be.ops.matmul(a, b, {"inputCastA": "f16", "inputCastB": "bf16"})
    a_r = a_v.astype(np.float16).astype(np.float32)
    b_r = orc.bf16_bits_to_f32(orc.bf16_bits_rne(b_v.reshape(-1))).reshape(k, n)
    np.testing.assert_allclose(_read_f32(be, y), _ref(a_r, b_r), rtol=1e-5, atol=1e-5)
    # and differs from the unrounded product: the prologue really ran
    assert np.abs(_read_f32(be, y) - _ref(a_v, b_v)).max() > 1e-4
    for t in (a, b, y):
        t.destroy()


def test_dense_matmul_batched_with_broadcast(backend):
    be = backend
    bs, m, k, n = 3, 18, 40, 22
    rng = np.random.default_rng(99)
    av = rng.uniform(-1, 1, bs * m * k).astype(np.float32)
    bv = rng.uniform(-1, 1, bs * k * n).astype(np.float32)
    a, a_v = _to_dev(be, av, [bs, m, k], "f32")
    b, b_v = _to_dev(be, bv, [bs, k, n], "f32")
    b1, b1_v = _to_dev(be, bv[: k * n], [k, n], "f32")
    a1, a1_v = _to_dev(be, av[: m * k], [m, k], "f32")
    y = be.ops.matmul(a, b)          # both batched
    yb = be.ops.matmul(a, b1)        # B broadcast (flattened to one [bs*m, k] product)
    ya = be.ops.matmul(a1, b)        # A broadcast (stride 0)
    g, gb, ga = _read_f32(be, y), _read_f32(be, yb), _read_f32(be, ya)
    assert g.shape == (bs, m, n) and gb.shape == (bs, m, n) and ga.shape == (bs, m, n)
    for i in range(bs):
        np.testing.assert_allclose(g[i], _ref(a_v[i], b_v[i]), rtol=1e-4, atol=1e-4)
        np.testing.assert_allclose(gb[i], _ref(a_v[i], b1_v), rtol=1e-4, atol=1e-4)
        np.testing.assert_allclose(ga[i], _ref(a1_v, b_v[i]), rtol=1e-4, atol=1e-4)
    for t in (a, b, b1, a1, y, yb, ya):
        t.destroy()


def _rel(x, ref):
    return float(np.max(np.abs(x - ref) / np.maximum(1.0, np.abs(ref))))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m", [1, 4, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(33, 128), (128, 1024), (1024, 2048), (2048, 6144), (4096, 32)])
def test_dense_gemv_nt_routes_to_tensor_core_gemv(backend, dtype, m, n, k):
    be = backend
    rng = np.random.default_rng(n * 31 + k + m)
    xv = rng.uniform(-1, 1, m * k).astype(np.float32)
    wv = rng.uniform(-1, 1, n * k).astype(np.float32)
    x, x_v = _to_dev(be, xv, [m, k], dtype)
    w, w_v = _to_dev(be, wv, [n, k], dtype)
    assert be.planMatmul(m, n, k, dtype, dtype, transB=True)["variant"].startswith("matmul.gemv")
    be.resetCounters()
    y = be.ops.matmul(x, be.ops.transpose(w))
    assert be.getGemvDispatchCount() == 1 and be.getTiledMatmulDispatchCount() == 0
    got = _read_f32(be, y)
    ref = _ref(x_v, w_v.T)
    assert _rel(got, ref) <= 5e-4
    # forcing the tiled kernel gives the same answer through the other route
    be.forceVariant((3, 0, 0, 0, 0, 0))
    try:
        be.resetCounters()
        y2 = be.ops.matmul(x, be.ops.transpose(w))
        assert be.getGemvDispatchCount() == 0 and be.getTiledMatmulDispatchCount() == 1
    finally:
        be.forceVariant(None)
    assert _rel(_read_f32(be, y2), ref) <= 5e-4
    for t in (x, w, y, y2):
        t.destroy()


@pytest.mark.parametrize("epi", [("bias", None), ("bias", "gelu"), ("bias", "silu"), (None, "silu")])
def test_dense_gemv_epilogue_battery(backend, epi):
    be = backend
    m, n, k = 1, 1024, 2048
    rng = np.random.default_rng(5)
    x, x_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], "f16")
    w, w_v = _to_dev(be, (rng.uniform(-1, 1, n * k) * 0.1).astype(np.float32), [n, k], "f16")
    bias_v = rng.uniform(-1, 1, n).astype(np.float32)
    bias_t = be.ops.tensorFromArray(bias_v, [n], "f32")
    be.resetCounters()
    y = be.linear(x, w, bias_t if epi[0] else None, epi[1], "f32")
    assert be.getGemvDispatchCount() == 1 and be.getGemvEpilogueDispatchCount() == 1
    ref = _ref(x_v, w_v.T, bias_v if epi[0] else None, epi[1])
    assert _rel(_read_f32(be, y), ref) <= 1e-4
    for t in (x, w, bias_t, y):
        t.destroy()


def test_dense_matmul_argument_errors(backend):
    be = backend
    a = be.ops.tensorFromArray(np.zeros(12, np.float32), [3, 4], "f32")
    b = be.ops.tensorFromArray(np.zeros(15, np.float32), [5, 3], "f32")
    with pytest.raises(tb.TlError):
        be.ops.matmul(a, b)  # inner dims differ
    for t in (a, b):
        t.destroy()


# ---------------------------------------------------------------------------
# companion ops: the unfused sequence the reference's tests use as the control
# (test/webgpu/matmul-epilogue.spec.ts:77-100): matmul -> add bias -> activation -> cast
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("act", ["relu", "silu", "gelu", "sigmoid", "tanh"])
def test_unfused_sequence_matches_fused_epilogue_and_oracle(backend, act):
    be = backend
    m, k, n = 50, 70, 60
    a, a_v = _to_dev(be, _pattern(m * k, 0) * 0.25, [m, k], "f32")
    b, b_v = _to_dev(be, _pattern(k * n, 3) * 0.25, [k, n], "f32")
    bias_v = _pattern(n, 5) * 0.5
    bias_t = be.ops.tensorFromArray(bias_v, [n], "f32")
    y0 = be.ops.matmul(a, b)
    y1 = be.ops.add(y0, bias_t)
    y2 = getattr(be.ops, act)(y1)
    y3 = be.ops.cast(y2, "f16")
    plan = tb.detectMatmulEpilogue([("add", bias_t), (act, None), ("cast", "f16")])
    fused = be.ops.matmul(a, b, {"epilogue": plan[0], "epilogueInputs": plan[1]})
    assert fused.dtype == "f16"
    ref = _ref(a_v, b_v, bias_v, act)
    np.testing.assert_allclose(_read_f32(be, y2), ref, rtol=1e-5, atol=1e-5)
    # fused and unfused round the same f32 value to f16 once: identical bits
    np.testing.assert_array_equal(be.ops.read(y3).view(np.uint16), be.ops.read(fused).view(np.uint16))
    for t in (a, b, bias_t, y0, y1, y2, y3, fused):
        t.destroy()


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_contiguous_of_a_transposed_view(backend, dtype):
    be = backend
    rows, cols = 45, 70
    t, t_v = _to_dev(be, np.arange(rows * cols, dtype=np.float32) % 251, [rows, cols], dtype)
    c = be.ops.contiguous(be.ops.transpose(t))
    assert c.shape == [cols, rows] and not c.transposed
    np.testing.assert_array_equal(_read_f32(be, c), t_v.T)
    c2 = be.ops.contiguous(t)
    np.testing.assert_array_equal(_read_f32(be, c2), t_v)
    # the materialized transposition feeds a plain NN product
    x, x_v = _to_dev(be, _pattern(8 * rows, 1), [8, rows], dtype)
    y = be.ops.matmul(x, t)
    np.testing.assert_allclose(_read_f32(be, y), _ref(x_v, t_v), rtol=2e-2, atol=2e-2)
    for u in (t, c, c2, x, y):
        u.destroy()


def test_binary_ops_and_cast_round_trip(backend):
    be = backend
    rng = np.random.default_rng(3)
    av = rng.uniform(-4, 4, 33 * 65).astype(np.float32)
    bv = rng.uniform(-4, 4, 33 * 65).astype(np.float32)
    a, a_v = _to_dev(be, av, [33, 65], "f32")
    b, b_v = _to_dev(be, bv, [33, 65], "f32")
    for name, fn in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply)):
        r = getattr(be.ops, name)(a, b)
        np.testing.assert_array_equal(_read_f32(be, r), fn(a_v, b_v))
        r.destroy()
    h = be.ops.cast(a, "f16")
    np.testing.assert_array_equal(be.ops.read(h), a_v.astype(np.float16))
    bf = be.ops.cast(a, "bf16")
    np.testing.assert_array_equal(be.ops.read(bf).reshape(-1), orc.bf16_bits_rne(a_v.reshape(-1)))
    back = be.ops.cast(h, "f32")
    np.testing.assert_array_equal(_read_f32(be, back), a_v.astype(np.float16).astype(np.float32))
    for t in (a, b, h, bf, back):
        t.destroy()


# ---------------------------------------------------------------------------
# the tensor-core route (tcgen05, both operands from shared memory)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,k,n", [(128, 64, 128), (256, 256, 512), (130, 72, 200), (33, 200, 201), (512, 1024, 1000)])
def test_dense_tensor_core_route_nt(backend, dtype, m, k, n):
    be = backend
    rng = np.random.default_rng(m + 7 * n + 13 * k)
    x, x_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], dtype)
    w, w_v = _to_dev(be, rng.uniform(-1, 1, n * k).astype(np.float32), [n, k], dtype)
    assert be.planMatmul(m, n, k, dtype, dtype, transB=True)["variant"].startswith("matmul.tc")
    y = be.ops.matmul(x, be.ops.transpose(w))
    ref = _ref(x_v, w_v.T)
    assert _rel(_read_f32(be, y), ref) <= 1e-3
    # the exactly representable pattern inputs give exact sums: bit-equal to the oracle
    xp, xp_v = _to_dev(be, _pattern(m * k, 0), [m, k], dtype)
    wp, wp_v = _to_dev(be, _pattern(n * k, 3), [n, k], dtype)
    yp = be.ops.matmul(xp, be.ops.transpose(wp))
    np.testing.assert_array_equal(_read_f32(be, yp), _ref(xp_v, wp_v.T))
    for t in (x, w, y, xp, wp, yp):
        t.destroy()


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (True, True)])
def test_dense_tensor_core_route_other_layouts(backend, trans_a, trans_b):
    be = backend
    m, k, n = 96, 136, 264
    rng = np.random.default_rng(11)
    a_t, a_stored = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [k, m] if trans_a else [m, k], "f16")
    b_t, b_stored = _to_dev(be, rng.uniform(-1, 1, k * n).astype(np.float32), [n, k] if trans_b else [k, n], "f16")
    a_view = be.ops.transpose(a_t) if trans_a else a_t
    b_view = be.ops.transpose(b_t) if trans_b else b_t
    assert be.planMatmul(m, n, k, "f16", "f16", transA=trans_a, transB=trans_b)["variant"].startswith("matmul.tc")
    y = be.ops.matmul(a_view, b_view)
    ref = _ref(a_stored.T if trans_a else a_stored, b_stored.T if trans_b else b_stored)
    assert _rel(_read_f32(be, y), ref) <= 1e-3
    for t in (a_t, b_t, y):
        t.destroy()


@pytest.mark.parametrize("out_dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("epi", [("bias", None), ("bias", "gelu"), (None, "silu"), ("bias", "relu"), "residual"])
def test_dense_tensor_core_epilogues(backend, out_dtype, epi):
    be = backend
    m, k, n = 160, 128, 272
    rng = np.random.default_rng(2)
    x, x_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], "bf16")
    w, w_v = _to_dev(be, (rng.uniform(-1, 1, n * k) * 0.2).astype(np.float32), [n, k], "bf16")
    bias_v = rng.uniform(-1, 1, n).astype(np.float32)
    bias_t = be.ops.tensorFromArray(bias_v, [n], "f32")
    res_v = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    res_t = be.ops.tensorFromArray(res_v, [m, n], "f32")
    if epi == "residual":
        chain = [("add", res_t), ("relu", None)]
        ref = orc.unary("relu", (_ref(x_v, w_v.T) + res_v).astype(np.float32))
    else:
        chain = ([("add", bias_t)] if epi[0] else []) + ([(epi[1], None)] if epi[1] else [])
        ref = _ref(x_v, w_v.T, bias_v if epi[0] else None, epi[1])
    if out_dtype != "f32":
        chain.append(("cast", out_dtype))
    plan = tb.detectMatmulEpilogue(chain)
    y = be.ops.matmul(x, be.ops.transpose(w), {"epilogue": plan[0], "epilogueInputs": plan[1]})
    assert y.dtype == out_dtype
    assert _rel(_read_f32(be, y), ref) <= (1e-3 if out_dtype == "f32" else 1e-2)
    for t in (x, w, bias_t, res_t, y):
        t.destroy()


def test_dense_tensor_core_batched(backend):
    be = backend
    bs, m, k, n = 3, 64, 128, 128
    rng = np.random.default_rng(4)
    a, a_v = _to_dev(be, rng.uniform(-1, 1, bs * m * k).astype(np.float32), [bs, m, k], "f16")
    b, b_v = _to_dev(be, rng.uniform(-1, 1, bs * k * n).astype(np.float32), [bs, k, n], "f16")
    y = be.ops.matmul(a, b)
    g = _read_f32(be, y)
    for i in range(bs):
        assert _rel(g[i], _ref(a_v[i], b_v[i])) <= 1e-3
    for t in (a, b, y):
        t.destroy()


# every tile shape of the tensor-core kernel, forced: (BN, MH) with MH row halves of 128 per tile
_TC_TILES = [(256, 1), (224, 1), (192, 1), (160, 1), (128, 1), (256, 2), (240, 2), (224, 2), (208, 2), (192, 2), (176, 2), (160, 2)]


@pytest.mark.parametrize("bn,mh", _TC_TILES)
def test_dense_tensor_core_every_tile_shape_ragged(backend, bn, mh):
    """m, n and k off every tile boundary (the second row half of the last tile is partly out of range,
    the last column tile is ragged, k ends inside a 64-k stage), bias + gelu, f16 in and out."""
    be = backend
    m, k, n = 300, 200, 2 * bn + 40
    rng = np.random.default_rng(bn + mh)
    x, x_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], "f16")
    w, w_v = _to_dev(be, (rng.uniform(-1, 1, n * k) * 0.2).astype(np.float32), [n, k], "f16")
    bias_v = rng.uniform(-1, 1, n).astype(np.float32)
    bias_t = be.ops.tensorFromArray(bias_v, [n], "f32")
    plan = tb.detectMatmulEpilogue([("add", bias_t), ("gelu", None), ("cast", "f16")])
    be.forceVariant((B.TL_FAMILY_MATMUL, 2, bn, 0, mh, 0))
    try:
        receipt = be.planMatmul(m, n, k, "f16", "f16", transB=True)
        assert receipt["variant"].startswith("matmul.tc") and receipt["choice"][2] == bn and receipt["choice"][4] == mh
        y = be.ops.matmul(x, be.ops.transpose(w), {"epilogue": plan[0], "epilogueInputs": plan[1]})
        assert _rel(_read_f32(be, y), _ref(x_v, w_v.T, bias_v, "gelu")) <= 1e-2
        # exactly representable inputs: bit-equal to the oracle, f32 out (the un-approximated path)
        xp, xp_v = _to_dev(be, _pattern(m * k, 0), [m, k], "f16")
        wp, wp_v = _to_dev(be, _pattern(n * k, 3), [n, k], "f16")
        yp = be.ops.matmul(xp, be.ops.transpose(wp))
        np.testing.assert_array_equal(_read_f32(be, yp), _ref(xp_v, wp_v.T))
    finally:
        be.forceVariant(None)
    for t in (x, w, bias_t, y, xp, wp, yp):
        t.destroy()


@pytest.mark.parametrize("bn,mh", [(160, 2), (256, 2), (128, 1)])
def test_dense_tensor_core_several_tiles_per_cta(backend, bn, mh):
    """More tiles than SMs: every CTA walks several tiles, so the accumulators in TMEM are handed back
    and forth between the MMA warp and the epilogue warps (one set when MH = 2, two when MH = 1)."""
    be = backend
    m, k, n = 2048, 192, 20 * bn
    rng = np.random.default_rng(5)
    x, x_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], "bf16")
    w, w_v = _to_dev(be, rng.uniform(-1, 1, n * k).astype(np.float32), [n, k], "bf16")
    be.forceVariant((B.TL_FAMILY_MATMUL, 2, bn, 0, mh, 0))
    try:
        y = be.ops.matmul(x, be.ops.transpose(w))
        assert _rel(_read_f32(be, y), _ref(x_v, w_v.T)) <= 1e-3
    finally:
        be.forceVariant(None)
    for t in (x, w, y):
        t.destroy()


@pytest.mark.parametrize("out_dtype", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["relu", "silu", "gelu", "gelu_erf", "sigmoid", "tanh"])
def test_dense_tensor_core_unary_modes_on_two_half_tiles(backend, out_dtype, act):
    be = backend
    m, k, n = 260, 128, 330
    rng = np.random.default_rng(9)
    x, x_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], "bf16")
    w, w_v = _to_dev(be, (rng.uniform(-1, 1, n * k) * 0.2).astype(np.float32), [n, k], "bf16")
    chain = [("gelu", {"approximate": "none"}) if act == "gelu_erf" else (act, None)]
    if out_dtype != "f32":
        chain.append(("cast", out_dtype))
    plan = tb.detectMatmulEpilogue(chain)
    be.forceVariant((B.TL_FAMILY_MATMUL, 2, 160, 0, 2, 0))
    try:
        y = be.ops.matmul(x, be.ops.transpose(w), {"epilogue": plan[0], "epilogueInputs": plan[1]})
        assert _rel(_read_f32(be, y), _ref(x_v, w_v.T, None, act)) <= (1e-3 if out_dtype == "f32" else 1e-2)
    finally:
        be.forceVariant(None)
    for t in (x, w, y):
        t.destroy()


def test_dense_tensor_core_full_size_sampled_rows(backend):
    """The benchmark's dense shape (2048 x 4096 -> 14336, bf16, gelu, bf16 out) with the tile the library picks
    for it; the oracle runs on token rows that cover every 128- and 256-row tile edge, over all N."""
    be = backend
    m, k, n = 2048, 4096, 14336
    rng = np.random.default_rng(17)
    x, x_v = _to_dev(be, rng.standard_normal(m * k, dtype=np.float32), [m, k], "bf16")
    w, w_v = _to_dev(be, rng.standard_normal(n * k, dtype=np.float32) * np.float32(0.02), [n, k], "bf16")
    plan = tb.detectMatmulEpilogue([("gelu", None), ("cast", "bf16")])
    receipt = be.planMatmul(m, n, k, "bf16", "bf16", transB=True)
    assert receipt["variant"].startswith("matmul.tc")
    y = be.ops.matmul(x, be.ops.transpose(w), {"epilogue": plan[0], "epilogueInputs": plan[1]})
    got = _read_f32(be, y)
    rows = sorted({0, 1, 127, 128, 129, 255, 256, 257, 1023, 1024, 1919, 1920, 2046, 2047} |
                  set(rng.integers(0, m, 10).tolist()))
    ref = _ref(x_v[rows], w_v.T, None, "gelu")
    assert _rel(got[rows], ref) <= 1e-2
    for t in (x, w, y):
        t.destroy()


@pytest.mark.parametrize("bn,mh", [(128, 1), (192, 1), (256, 1), (192, 2), (256, 2)])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_dense_tensor_core_nn_layout_without_a_transposed_copy(backend, bn, mh, dtype):
    """matmul(a, b) with b stored [K, N]: the tensor-core kernel stages and multiplies B MN-major (64-column
    slabs), so nothing is transposed into scratch.  Ragged m, n, k; bias + gelu; bit-exact on representable inputs."""
    be = backend
    m, k, n = 300, 200, 1000
    rng = np.random.default_rng(bn + mh)
    a, a_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], dtype)
    b, b_v = _to_dev(be, (rng.uniform(-1, 1, k * n) * 0.2).astype(np.float32), [k, n], dtype)
    bias_v = rng.uniform(-1, 1, n).astype(np.float32)
    bias_t = be.ops.tensorFromArray(bias_v, [n], "f32")
    plan = tb.detectMatmulEpilogue([("add", bias_t), ("gelu", None)])
    be.forceVariant((B.TL_FAMILY_MATMUL, 2, bn, 0, mh, 0))
    try:
        launches0 = be.getKernelLaunchCount()
        y = be.ops.matmul(a, b, {"epilogue": plan[0], "epilogueInputs": plan[1]})
        assert be.getKernelLaunchCount() == launches0 + 1  # one kernel: no transposition pass in front of it
        assert _rel(_read_f32(be, y), _ref(a_v, b_v, bias_v, "gelu")) <= 1e-2
        ap, ap_v = _to_dev(be, _pattern(m * k, 0), [m, k], dtype)
        bp, bp_v = _to_dev(be, _pattern(k * n, 3), [k, n], dtype)
        yp = be.ops.matmul(ap, bp)
        np.testing.assert_array_equal(_read_f32(be, yp), _ref(ap_v, bp_v))
    finally:
        be.forceVariant(None)
    for t in (a, b, bias_t, y, ap, bp, yp):
        t.destroy()


def test_dense_tensor_core_nn_layout_odd_n_takes_the_transposition_pass(backend):
    be = backend
    m, k, n = 160, 128, 1001  # a row pitch of 2002 bytes cannot be a TMA map
    rng = np.random.default_rng(3)
    a, a_v = _to_dev(be, rng.uniform(-1, 1, m * k).astype(np.float32), [m, k], "f16")
    b, b_v = _to_dev(be, rng.uniform(-1, 1, k * n).astype(np.float32), [k, n], "f16")
    assert be.planMatmul(m, n, k, "f16", "f16")["variant"].startswith("matmul.tc")
    launches0 = be.getKernelLaunchCount()
    y = be.ops.matmul(a, b)
    assert be.getKernelLaunchCount() == launches0 + 2  # transposition, then the NT kernel
    assert _rel(_read_f32(be, y), _ref(a_v, b_v)) <= 1e-3
    for t in (a, b, y):
        t.destroy()


@pytest.mark.parametrize("bn,mh", [(128, 1), (256, 1), (192, 2), (256, 2)])
@pytest.mark.parametrize("trans_b", [False, True])
def test_dense_tensor_core_transposed_a_without_a_transposed_copy(backend, bn, mh, trans_b):
    """matmul(transpose(a), b) with a stored [K, M]: A is staged and multiplied MN-major too (TN and TT)."""
    be = backend
    m, k, n = 296, 200, 1000
    rng = np.random.default_rng(bn + mh + int(trans_b))
    a, a_v = _to_dev(be, rng.uniform(-1, 1, k * m).astype(np.float32), [k, m], "bf16")
    b, b_v = _to_dev(be, (rng.uniform(-1, 1, k * n) * 0.2).astype(np.float32), [n, k] if trans_b else [k, n], "bf16")
    be.forceVariant((B.TL_FAMILY_MATMUL, 2, bn, 0, mh, 0))
    try:
        launches0 = be.getKernelLaunchCount()
        y = be.ops.matmul(be.ops.transpose(a), be.ops.transpose(b) if trans_b else b)
        assert be.getKernelLaunchCount() == launches0 + 1
        assert _rel(_read_f32(be, y), _ref(a_v.T, b_v.T if trans_b else b_v)) <= 1e-3
        ap, ap_v = _to_dev(be, _pattern(k * m, 1), [k, m], "bf16")
        bp, bp_v = _to_dev(be, _pattern(k * n, 4), [n, k] if trans_b else [k, n], "bf16")
        yp = be.ops.matmul(be.ops.transpose(ap), be.ops.transpose(bp) if trans_b else bp)
        np.testing.assert_array_equal(_read_f32(be, yp), _ref(ap_v.T, bp_v.T if trans_b else bp_v))
    finally:
        be.forceVariant(None)
    for t in (a, b, y, ap, bp, yp):
        t.destroy()
