"""GPU parity of the int4-grouped scheme (row f4) through the C ABI against the CPU oracle: unpacked
nibbles and dequantized weights bit-exact, f32-accumulated outputs within 1e-3 and 16-bit outputs
within 1e-2 on the reference probes' metric |x - ref| / max(1, |ref|); routes counted like the int8
path (m <= 16: fused-dequant GEMV; larger m: explicit dequant + dense matmul)."""
import numpy as np
import pytest

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb

pytestmark = pytest.mark.gpu


def _weight(be, n, k, g, seed):
    rng = np.random.default_rng(seed)
    w = (rng.uniform(-1, 1, (n, k)) * 0.1).astype(np.float32)
    packed, scales = be.quantizeLinearWeight(w, g, scheme="int4-grouped")
    op, os_ = orc.quantize_linear_weight_int4(w, g)
    assert np.array_equal(packed, op) and np.array_equal(scales, os_)
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int4-grouped", g, "f16"))
    return be.createQuantizedWeight(packed, scales, n, k, fmt), orc.dequantize_int4_to_f32(packed, scales, k, g), packed


@pytest.mark.parametrize("n,k,g", [(128, 128, 32), (300, 1024, 128), (33, 64, 8), (1024, 2048, 32)])
def test_int4_unpack_and_dequant_bit_exact(backend, n, k, g):
    be = backend
    w, ref, packed = _weight(be, n, k, g, seed=n + k)
    assert np.array_equal(be.unpackInt4(w, n, k), orc.unpack_int4(packed, k))
    d = be.dequantize(w, "f32")
    assert np.array_equal(be.ops.read(d).view(np.uint32), ref.view(np.uint32))
    h = be.dequantize(w, "f16")
    assert np.array_equal(be.ops.read(h), ref.astype(np.float16))
    for t in (d, h, w.scales, w):
        t.destroy()


@pytest.mark.parametrize("act_dtype,out_dtype", [("f32", "f32"), ("f16", "f32"), ("f16", "f16"), ("bf16", "bf16")])
@pytest.mark.parametrize("m", [1, 3, 4, 8, 16])
@pytest.mark.parametrize("n,k,g", [(128, 128, 32), (512, 1024, 128), (37, 264, 8)])
def test_int4_gemv_matches_oracle(backend, act_dtype, out_dtype, m, n, k, g):
    be = backend
    w, wref, _ = _weight(be, n, k, g, seed=7 * n + k + m)
    rng = np.random.default_rng(m)
    xv = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    if act_dtype == "f16":
        x = be.ops.tensorFromArray(xv.astype(np.float16), [m, k], "f16")
        xv = xv.astype(np.float16).astype(np.float32)
    elif act_dtype == "bf16":
        bits = orc.bf16_bits_rne(xv.reshape(-1))
        x = be.ops.tensorFromArray(bits, [m, k], "bf16")
        xv = orc.bf16_bits_to_f32(bits).reshape(m, k)
    else:
        x = be.ops.tensorFromArray(xv, [m, k], "f32")
    be.resetCounters()
    y = be.linear(x, w, None, None, out_dtype)
    assert be.getQuantGemvDispatchCount() == 1 and be.getDequantI8DispatchCount() == 0
    got = be.ops.read(y)
    got = orc.bf16_bits_to_f32(got) if out_dtype == "bf16" else np.asarray(got, np.float32)
    ref = orc.linear_reference(xv, wref)
    assert cases.rel_err(got, ref) <= (1e-3 if out_dtype == "f32" else 1e-2)
    for t in (x, y, w.scales, w):
        t.destroy()


@pytest.mark.parametrize("act", [None, "relu", "gelu", "silu"])
def test_int4_gemv_epilogue(backend, act):
    be = backend
    n, k, g, m = 256, 512, 32, 4
    w, wref, _ = _weight(be, n, k, g, seed=99)
    rng = np.random.default_rng(5)
    xv = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    x = be.ops.tensorFromArray(xv, [m, k], "f16")
    bt = be.ops.tensorFromArray(bias, [n], "f32")
    be.resetCounters()
    y = be.linear(x, w, bt, act, "f32")
    assert be.getGemvEpilogueDispatchCount() == 1
    ref = orc.linear_reference(xv.astype(np.float32), wref, bias, act)
    assert cases.rel_err(be.ops.read(y), ref) <= 1e-3
    for t in (x, bt, y, w.scales, w):
        t.destroy()


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_int4_large_m_takes_the_dequant_plus_dense_route(backend, dtype):
    be = backend
    n, k, g, m = 256, 512, 128, 96
    w, wref, _ = _weight(be, n, k, g, seed=3)
    rng = np.random.default_rng(8)
    xv = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    if dtype == "f16":
        x = be.ops.tensorFromArray(xv.astype(np.float16), [m, k], "f16")
        xv = xv.astype(np.float16).astype(np.float32)
        wr = wref.astype(np.float16).astype(np.float32)   # the dense operand is the dequantized weight in the activation type
    elif dtype == "bf16":
        bits = orc.bf16_bits_rne(xv.reshape(-1))
        x = be.ops.tensorFromArray(bits, [m, k], "bf16")
        xv = orc.bf16_bits_to_f32(bits).reshape(m, k)
        wr = orc.bf16_bits_to_f32(orc.bf16_bits_rne(wref.reshape(-1))).reshape(n, k)
    else:
        x = be.ops.tensorFromArray(xv, [m, k], "f32")
        wr = wref
    be.resetCounters()
    y = be.linear(x, w, None, "relu", "f32")
    assert be.getQuantGemvDispatchCount() == 0 and be.getDequantI8DispatchCount() == 1
    ref = orc.linear_reference(xv, wr, None, "relu")
    assert cases.rel_err(be.ops.read(y), ref) <= 1e-3
    plan = be.planQuantizedMatmul(m, n, k, dtype, "f32", w.format.packing)
    assert plan["family"] == "gemm"
    assert be.planQuantizedMatmul(4, n, k, dtype, "f32", w.format.packing)["family"] == "gemv"
    for t in (x, y, w.scales, w):
        t.destroy()


def test_int4_argument_errors(backend):
    be = backend
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int4-grouped", 32, "f16"))
    with pytest.raises(tb.TlError):
        be.createQuantizedWeight(np.zeros(10, np.uint32), np.zeros(4, np.uint16), 4, 36, fmt)  # K % 8
    with pytest.raises(tb.TlError):
        be.quantizeLinearWeight(np.zeros((2, 36), np.float32), 12, scheme="int4-grouped")


@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("g", [128, 256, 1024])
def test_int4_tensor_core_and_simt_forms_agree(backend, m, g):
    """K and the group multiples of 128 take the mma.sync form; forcing {QGEMV, simt} takes the f32
    form.  Both against the oracle, and against each other within f32 summation-order noise."""
    be = backend
    n, k = 264, 1024
    w, wref, _ = _weight(be, n, k, g, seed=g + m)
    rng = np.random.default_rng(g)
    xv = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    x = be.ops.tensorFromArray(xv, [m, k], "f16")
    y1 = be.linear(x, w, None, None, "f32")
    be.forceVariant((1, 1, 8, 1, 1, 0))
    try:
        y2 = be.linear(x, w, None, None, "f32")
    finally:
        be.forceVariant(None)
    ref = orc.linear_reference(xv.astype(np.float32), wref)
    a, b = be.ops.read(y1), be.ops.read(y2)
    assert cases.rel_err(a, ref) <= 1e-3 and cases.rel_err(b, ref) <= 1e-3
    assert cases.rel_err(a, b) <= 1e-4
    for t in (x, y1, y2, w.scales, w):
        t.destroy()
