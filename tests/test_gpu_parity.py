"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle on the same seeded inputs.

Tolerances (stated by the path's specification): unpacked int8 and dequantized
f32 weights bit-exact; f32-accumulated f32 outputs within 1e-3; f16/bf16 outputs
within 1e-2; both measured with the reference probes' metric
|x - ref| / max(1, |ref|) (examples/qwen3/probe-quant-gemv.ts:166-177).
"""
import ctypes as C

import numpy as np
import pytest

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_HALF = 1e-2

GEMV_VARIANTS_F32 = [(1, 0, 8, 0, 1, 0), (1, 1, 8, 1, 1, 0), (1, 1, 8, 2, 1, 0), (1, 1, 4, 4, 1, 0)]
GEMV_VARIANTS_HALF = GEMV_VARIANTS_F32 + [(1, 2, 8, 4, 1, 0), (1, 2, 4, 2, 1, 0), (1, 2, 16, 2, 1, 0),
                                          (1, 3, 4, 4, 0, 0), (1, 3, 2, 2, 0, 0), (1, 3, 8, 4, 0, 0),
                                          (1, 4, 4, 4, 0, 0), (1, 4, 2, 8, 0, 0), (1, 4, 16, 2, 0, 0),
                                          (1, 5, 6, 0, 0, 0), (1, 5, 4, 0, 0, 0),
                                          (1, 6, 16, 32, 0, 0), (1, 6, 8, 64, 0, 0),
                                          (1, 8, 8, 3, 2, 16), (1, 8, 8, 5, 2, 16), (1, 8, 8, 2, 1, 16), (1, 8, 8, 3, 2, 32)]


def _out_to_f32(arr, dtype):
    if dtype == "bf16":
        return orc.bf16_bits_to_f32(arr)
    return np.asarray(arr, dtype=np.float32)


def _upload_act(be, cs, m, k, dtype):
    if dtype == "f32":
        return be.ops.tensorFromArray(cs["x"], [m, k], "f32")
    return be.ops.tensorFromArray(cs["x_bits"], [m, k], dtype)


def _run_direct(be, cs, m, n, k, act_dtype, out_dtype, variant=None, bias=False, act=None, alpha=1.0):
    """Per-channel f32 'direct' case through linear(); returns (gpu f32, oracle f32)."""
    fmt = tb.perChannelFormat(k)
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, fmt)
    x = _upload_act(be, cs, m, k, act_dtype)
    bt = be.ops.tensorFromArray(cs["bias"], [n], "f32") if bias else None
    be.forceVariant(variant)
    try:
        y = be.linear(x, w, bt, act, out_dtype)
    finally:
        be.forceVariant(None)
    got = _out_to_f32(be.ops.read(y), out_dtype)
    wref = orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k)
    ref = orc.linear_reference(cs["x"], wref, cs["bias"] if bias else None, act, alpha)
    for t in (w.scales, w, x, y) + ((bt,) if bt else ()):
        t.destroy()
    return got, ref


# ---------------------------------------------------------------------------
# integer unpack + dequant: bit-exact
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("n,k,group", [(128, 128, 64), (96, 384, 128), (33, 256, 32), (7, 64, 4)])
def test_unpack_and_dequant_snorm_bit_exact(backend, n, k, group):
    be = backend
    w, _ = orc.lcg_fill(0x51A7EE ^ n, n * k)
    packed, scales = be.quantizeLinearWeight(w.reshape(n, k), group)
    op, os_ = orc.quantize_linear_weight(w.reshape(n, k), group)
    assert np.array_equal(packed, op) and np.array_equal(scales, os_)
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int8-grouped", group, "f16"))
    wt = be.createQuantizedWeight(packed, scales, n, k, fmt)
    assert np.array_equal(be.unpackInt8(wt, n, k), orc.unpack_int8(packed, k))
    before = be.getDequantI8DispatchCount()
    out = be.ops.empty([n, k], "f32")
    be.dispatchDequantizeInt8Grouped(wt, wt.scales, out, n, k, group)
    assert be.getDequantI8DispatchCount() == before + 1
    ref = orc.dequantize_to_f32(packed, scales, k, group)
    assert np.array_equal(be.ops.read(out).view(np.uint32), ref.view(np.uint32))
    for dt in ("f16", "bf16"):
        o2 = be.ops.empty([n, k], dt)
        be.dispatchDequantizeInt8Grouped(wt, wt.scales, o2, n, k, group)
        got = be.ops.read(o2)
        if dt == "f16":
            assert np.array_equal(got.view(np.uint16), ref.astype(np.float16).view(np.uint16))
        else:
            assert np.array_equal(got, orc.bf16_bits_rne(ref))
        o2.destroy()
    for t in (out, wt.scales, wt):
        t.destroy()


def test_unpack_every_byte_value_every_lane(backend):
    be = backend
    q = np.zeros((4, 1024), dtype=np.int8)
    for lane in range(4):
        q[lane, lane::4] = np.arange(-128, 128, dtype=np.int8)
    packed = cases.pack_int8(q)
    s = np.full((4, 1), 0.5, dtype=np.float32)
    wt = be.createQuantizedWeight(packed, s, 4, 1024, tb.perChannelFormat(1024))
    assert np.array_equal(be.unpackInt8(wt, 4, 1024), q)
    out = be.ops.empty([4, 1024], "f32")
    be.dispatchDequantizeInt8Grouped(wt, wt.scales, out, 4, 1024, 1024, packing=wt.format.packing)
    assert np.array_equal(be.ops.read(out), q.astype(np.float32) * 0.5)  # -128 is not clamped
    for t in (out, wt.scales, wt):
        t.destroy()


def test_dequant_direct_bit_exact_config0(backend):
    be = backend
    cs = cases.per_channel_case(2048, 2048, 1, seed=0)
    wt = be.createQuantizedWeight(cs["packed"], cs["scales"], 2048, 2048, tb.perChannelFormat(2048))
    out = be.ops.empty([2048, 2048], "f32")
    be.dispatchDequantizeInt8Grouped(wt, wt.scales, out, 2048, 2048, 2048, packing=wt.format.packing)
    ref = orc.dequantize_direct_f32(cs["packed"], cs["scales"], 2048, 2048)
    assert np.array_equal(be.ops.read(out).view(np.uint32), ref.view(np.uint32))
    for t in (out, wt.scales, wt):
        t.destroy()


# ---------------------------------------------------------------------------
# config 0: f32 activations, per-channel scales, every applicable variant
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("variant", [None] + GEMV_VARIANTS_F32)
def test_config0_gemv_f32(backend, variant):
    cs = cases.per_channel_case(2048, 2048, 1, seed=0)
    got, ref = _run_direct(backend, cs, 1, 2048, 2048, "f32", "f32", variant)
    assert cases.rel_err(got, ref) <= TOL_F32


def test_config0_matches_committed_golden_rows(backend):
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "config0_rows0_63.npz"))
    cs = cases.per_channel_case(2048, 2048, 1, seed=0)
    got, _ = _run_direct(backend, cs, 1, 2048, 2048, "f32", "f32")
    assert cases.rel_err(got[:, :64], g["y"]) <= TOL_F32


def test_config0_reference_native_format_g64(backend):
    """The same int8 values in the reference's own layout: f16 group scales
    holding 127*s (so that (q/127)*scale = q*s up to the f16 rounding)."""
    be = backend
    cs = cases.per_channel_case(512, 2048, 1, seed=0)
    s16 = np.repeat((cs["scales"] * 127.0).astype(np.float16), 2048 // 64, axis=1)
    wt = be.createQuantizedWeight(cs["packed"], s16.view(np.uint16), 512, 2048, tb.resolveWeightFormat("int8-64"))
    x = be.ops.tensorFromArray(cs["x"], [1, 2048], "f32")
    y = be.linear(x, wt)
    wref = orc.dequantize_to_f32(cs["packed"], s16.view(np.uint16), 2048, 64)
    assert cases.rel_err(be.ops.read(y), orc.matmul_nt(cs["x"], wref)) <= TOL_F32
    for t in (x, y, wt.scales, wt):
        t.destroy()


# ---------------------------------------------------------------------------
# the reference probes' gate shapes (probe-quant-gemv.ts:34-42, 166-187)
# ---------------------------------------------------------------------------

def _probe_gemv_case(be, n, k, group, state, act_dtype="f32"):
    w, state = orc.lcg_fill(state, n * k)
    a, state = orc.lcg_fill(state, k)
    packed, scales = be.quantizeLinearWeight(w.reshape(n, k), group)
    del w
    fmt = tb.resolveWeightFormat("int8-64" if group == 64 else "int8-128")
    wt = be.createQuantizedWeight(packed, scales, n, k, fmt)
    if act_dtype == "f16":
        a = a.astype(np.float16).astype(np.float32)
        xt = be.ops.tensorFromArray(a.astype(np.float16), [1, k], "f16")
    else:
        xt = be.ops.tensorFromArray(a, [1, k], "f32")
    out = be.ops.empty([1, n], "f32")
    q0 = be.getQuantGemvDispatchCount()
    be.dispatchQuantizedGemvNT(xt, wt, wt.scales, out, n, k, group)
    assert be.getQuantGemvDispatchCount() == q0 + 1  # qHits === 1 (:188)
    got = be.ops.read(out)[0]
    deq = orc.dequantize_to_f32(packed, scales, k, group)
    control = orc.matmul_nt(a.reshape(1, k), deq)[0]
    ref64 = deq.astype(np.float64) @ a.astype(np.float64)
    for t in (out, xt, wt.scales, wt):
        t.destroy()
    return got, control, ref64, state


@pytest.mark.parametrize("act_dtype", ["f32", "f16"])
def test_probe_quant_gemv_shapes(backend, act_dtype):
    state = 0x51A7EE
    for group in (64, 128):
        for n, k in [(128, 128), (512, 1024), (1024, 2048), (2048, 6144)]:
            got, control, ref64, state = _probe_gemv_case(backend, n, k, group, state, act_dtype)
            assert cases.rel_err(got, control) <= 5e-4, (n, k, group)
            assert cases.rel_err(got, ref64) <= 5e-4, (n, k, group)
    assert backend.getGpuUncapturedErrorCount() == 0


def test_probe_quant_gemv_lm_head_scale(backend):
    """N = 151936 (the probe's 2-D-grid case), one group size to bound host time."""
    got, control, ref64, _ = _probe_gemv_case(backend, 151936, 2048, 64, 0x51A7EE)
    assert cases.rel_err(got, control) <= 5e-4
    assert cases.rel_err(got, ref64) <= 5e-4


@pytest.mark.parametrize("m", [1, 4])
def test_probe_quant_operand(backend, m):
    """probe-quant-operand.ts: linear(x, qWeight) vs the f32 control, drift <= 5e-3,
    and the route: no explicit dequant on any M (the reference dequantizes for M=4)."""
    be = backend
    for n, k in [(128, 128), (512, 1024), (2048, 6144)]:
        for group in (64, 128):
            st = (0x51 ^ n ^ (k << 3) ^ (group << 7)) & 0xFFFFFFFF
            w, st = orc.lcg_fill(st, n * k, 0.1)
            x, st = orc.lcg_fill(st, m * k)
            packed, scales = be.quantizeLinearWeight(w.reshape(n, k), group)
            wt = be.createQuantizedWeight(packed, scales, n, k, tb.resolveWeightFormat(f"int8-{group}"))
            xt = be.ops.tensorFromArray(x, [m, k], "f32")
            q0, d0 = be.getQuantGemvDispatchCount(), be.getDequantI8DispatchCount()
            y = be.linear(xt, wt)
            assert be.getQuantGemvDispatchCount() == q0 + 1 and be.getDequantI8DispatchCount() == d0
            ref = orc.matmul_nt(x.reshape(m, k), orc.dequantize_to_f32(packed, scales, k, group))
            assert cases.drift(be.ops.read(y), ref) <= 5e-3, (n, k, group)
            assert cases.rel_err(be.ops.read(y), ref) <= TOL_F32
            for t in (y, xt, wt.scales, wt):
                t.destroy()


# ---------------------------------------------------------------------------
# config 1: Qwen3-0.6B decode projections, f16 activations, M = 1
# ---------------------------------------------------------------------------

CONFIG1 = [(1024, 2048), (1024, 1024), (1024, 1024), (1024, 3072), (1024, 3072), (2048, 1024), (3072, 1024)]


@pytest.mark.parametrize("variant", [None] + GEMV_VARIANTS_HALF[1:])
def test_config1_projections_f16(backend, variant):
    for seed, (k, n) in enumerate(CONFIG1):
        cs = cases.per_channel_case(n, k, 1, seed=seed, act_dtype="f16")
        got, ref = _run_direct(backend, cs, 1, n, k, "f16", "f32", variant)
        assert cases.rel_err(got, ref) <= TOL_F32, (k, n)
        got16, _ = _run_direct(backend, cs, 1, n, k, "f16", "f16", variant)
        assert cases.rel_err(got16, ref) <= TOL_HALF, (k, n)


# ---------------------------------------------------------------------------
# config 2: small batch with fused bias + activation, f16 in / f16 out
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("m", [1, 4, 8, 16])
def test_config2_fused_epilogue_small_batch(backend, m):
    n, k = 14336, 4096
    cs = cases.per_channel_case(n, k, m, seed=100 + m, act_dtype="f16", bias=True)
    for act in (None, "relu", "gelu", "silu"):
        got, ref = _run_direct(backend, cs, m, n, k, "f16", "f16", None, bias=True, act=act)
        assert cases.rel_err(got, ref) <= TOL_HALF, (m, act)
    got32, ref = _run_direct(backend, cs, m, n, k, "f16", "f32", None, bias=True, act="gelu")
    assert cases.rel_err(got32, ref) <= TOL_F32


@pytest.mark.parametrize("m", [2, 3, 5, 9, 13, 16])
@pytest.mark.parametrize("act_dtype", ["f16", "bf16", "f32"])
def test_small_batch_every_variant_and_dtype(backend, m, act_dtype):
    n, k = 272, 512  # n is not a multiple of 16*warps; exercises tail tiles
    cs = cases.per_channel_case(n, k, m, seed=m, act_dtype=act_dtype, bias=True)
    variants = GEMV_VARIANTS_F32 if act_dtype == "f32" else GEMV_VARIANTS_HALF
    for v in [None] + variants:
        got, ref = _run_direct(backend, cs, m, n, k, act_dtype, "f32", v, bias=True, act="silu")
        assert cases.rel_err(got, ref) <= TOL_F32, (v, m, act_dtype)


def test_bf16_output_and_activations(backend):
    cs = cases.per_channel_case(1024, 1024, 8, seed=77, act_dtype="bf16", bias=True)
    got, ref = _run_direct(backend, cs, 8, 1024, 1024, "bf16", "bf16", None, bias=True, act="gelu")
    assert cases.rel_err(got, ref) <= TOL_HALF


# ---------------------------------------------------------------------------
# grouped scales on the fast kernels, odd shapes, fallbacks
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("n,k,group,m", [
    (130, 1024, 64, 1), (130, 1024, 128, 3), (1, 64, 64, 1), (17, 192, 64, 16), (33, 128, 32, 2),
    (50, 80, 16, 1), (9, 68, 4, 1), (9, 68, 68, 5), (5, 8, 2, 1), (300, 4096, 4096, 7),
])
@pytest.mark.parametrize("act_dtype", ["f32", "f16"])
def test_grouped_and_ragged_shapes(backend, n, k, group, m, act_dtype):
    be = backend
    rng = np.random.default_rng(n * 1000 + k + group)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if act_dtype == "f16":
        x = x.astype(np.float16).astype(np.float32)
    packed, scales = be.quantizeLinearWeight(w, group)
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int8-grouped", group, "f16"))
    wt = be.createQuantizedWeight(packed, scales, n, k, fmt)
    xt = be.ops.tensorFromArray(x.astype(np.float16) if act_dtype == "f16" else x, [m, k], act_dtype)
    y = be.linear(xt, wt)
    ref = orc.matmul_nt(x, orc.dequantize_to_f32(packed, scales, k, group))
    assert cases.rel_err(be.ops.read(y), ref) <= TOL_F32
    plan = be.planQuantizedMatmul(m, n, k, act_dtype, "f32", fmt.packing)
    if k % 16 or group % 16:
        assert ".scalar" in plan["variant"]
    elif act_dtype == "f32" or k % 64 or group % 64:
        assert ".simt" in plan["variant"]
    else:
        assert ".ring" in plan["variant"]
    for t in (y, xt, wt.scales, wt):
        t.destroy()


def test_f32_scales_grouped_direct(backend):
    be = backend
    n, k, group, m = 96, 512, 128, 4
    rng = np.random.default_rng(11)
    q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = rng.uniform(0.001, 0.01, size=(n, k // group)).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float16)
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int8-grouped", group, "f32", "direct"))
    wt = be.createQuantizedWeight(cases.pack_int8(q), s, n, k, fmt)
    xt = be.ops.tensorFromArray(x, [m, k], "f16")
    y = be.linear(xt, wt)
    ref = orc.matmul_nt(x.astype(np.float32), orc.dequantize_direct_f32(cases.pack_int8(q), s, k, group))
    assert cases.rel_err(be.ops.read(y), ref) <= TOL_F32
    for t in (y, xt, wt.scales, wt):
        t.destroy()


def test_empty_shapes_launch_nothing(backend):
    be = backend
    lib, ctx = be._lib, be._ctx
    q = B.QuantDesc(1, 64, B.TL_F16, 0)
    buf = be._alloc(1024)
    launches = be.getKernelLaunchCount()
    for m, n in [(0, 64), (1, 0)]:
        rc = lib.tl_qmatmul_nt(ctx, buf, B.TL_F32, buf, buf, buf, B.TL_F32, m, n, 64, C.byref(q), 1.0, None)
        assert rc == B.TL_OK
    assert be.getKernelLaunchCount() == launches
    be._free(buf)


# ---------------------------------------------------------------------------
# epilogue battery (examples/qwen3/probe-gemv.ts:170-235; matmul-epilogue.spec.ts)
# ---------------------------------------------------------------------------

def _epilogue_case(be, ops, m=3, n=70, k=64, out_dtype="f32", act_dtype="f32"):
    rng = np.random.default_rng(len(ops) * 7 + m)
    cs = cases.per_channel_case(n, k, m, seed=5, act_dtype=act_dtype, bias=True)
    extra = rng.standard_normal((m, n)).astype(np.float32)
    wt = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    xt = _upload_act(be, cs, m, k, act_dtype)
    bias_t = be.ops.tensorFromArray(cs["bias"], [n], "f32")
    extra_t = be.ops.tensorFromArray(extra, [m, n], "f32")
    chain, ref = [], orc.matmul_nt(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k))
    for op in ops:
        if op == "bias":
            chain.append(("add", bias_t))
            ref = orc.add_bias(ref, cs["bias"])
        elif op in ("add2d", "sub2d", "mul2d"):
            chain.append((op[:3], extra_t))
            r64 = ref.astype(np.float64)
            e64 = extra.astype(np.float64)
            ref = {"add": r64 + e64, "sub": r64 - e64, "mul": r64 * e64}[op[:3]].astype(np.float32)
        elif op.startswith("cast:"):
            chain.append(("cast", op[5:]))
            ref = ref.astype(np.float16).astype(np.float32) if op[5:] == "f16" else orc.bf16_bits_to_f32(orc.bf16_bits_rne(ref))
        else:
            chain.append((op, None))
            ref = orc.unary(op, ref)
    cfg, inputs, consumed = tb.detectMatmulEpilogue(chain)
    assert consumed == len(ops)
    cfg.outputDtype = out_dtype
    e0 = be.getGemvEpilogueDispatchCount()
    y = be.ops.matmul(xt, be.ops.transpose(wt), {"epilogue": cfg, "epilogueInputs": inputs})
    assert be.getGemvEpilogueDispatchCount() == e0 + 1
    got = _out_to_f32(be.ops.read(y), out_dtype)
    for t in (y, xt, bias_t, extra_t, wt.scales, wt):
        t.destroy()
    return got, ref


@pytest.mark.parametrize("ops", [
    ["bias"], ["relu"], ["gelu"], ["silu"], ["sigmoid"], ["tanh"], ["gelu_erf"], ["bias", "relu"], ["bias", "gelu"],
    ["bias", "silu"], ["add2d"], ["bias", "mul2d", "relu"], ["sub2d", "tanh"], ["cast:f16", "bias"],
    ["bias", "gelu", "cast:f16", "add2d"],
])
def test_epilogue_battery(backend, ops):
    got, ref = _epilogue_case(backend, ops)
    tol = 1e-2 if any(o.startswith("gelu") for o in ops) else 1e-3  # the reference's own tolerances
    assert np.allclose(got, ref, rtol=tol, atol=tol), ops
    assert cases.rel_err(got, ref) <= TOL_F32


def test_epilogue_f16_output_mma_path(backend):
    got, ref = _epilogue_case(backend, ["bias", "gelu"], m=8, n=200, k=256, out_dtype="f16", act_dtype="f16")
    assert cases.rel_err(got, ref) <= TOL_HALF


def test_alpha_scales_before_epilogue(backend):
    be = backend
    cs = cases.per_channel_case(64, 128, 2, seed=4, act_dtype="f16", bias=True)
    wt = be.createQuantizedWeight(cs["packed"], cs["scales"], 64, 128, tb.perChannelFormat(128))
    xt = be.ops.tensorFromArray(cs["x_bits"], [2, 128], "f16")
    bt = be.ops.tensorFromArray(cs["bias"], [64], "f32")
    cfg, inputs, _ = tb.detectMatmulEpilogue([("add", bt), ("relu", None)])
    y = be.ops.matmul(xt, be.ops.transpose(wt), {"epilogue": cfg, "epilogueInputs": inputs, "alpha": 0.25})
    ref = orc.linear_reference(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], 128, 128), cs["bias"],
                               "relu", alpha=0.25)
    assert cases.rel_err(be.ops.read(y), ref) <= TOL_F32
    for t in (y, xt, bt, wt.scales, wt):
        t.destroy()


# ---------------------------------------------------------------------------
# errors: reported by status + message, nothing launched
# ---------------------------------------------------------------------------

def test_argument_errors(backend):
    be = backend
    lib, ctx = be._lib, be._ctx
    buf = be._alloc(4096)
    q = B.QuantDesc(1, 64, B.TL_F16, 0)
    launches = be.getKernelLaunchCount()

    def call(fn=lib.tl_qgemv_nt, a=buf, packed=buf, scales=buf, out=buf, m=1, n=8, k=64, qd=q, epi=None, adt=B.TL_F32):
        return fn(ctx, a, adt, packed, scales, out, B.TL_F32, m, n, k, C.byref(qd) if qd else None, 1.0, epi)

    assert call(m=17) == B.TL_ERR_INVALID_ARG and b"[1,16]" in lib.tl_last_error(ctx)
    assert call(k=66) == B.TL_ERR_INVALID_ARG and b"divisible by 4" in lib.tl_last_error(ctx)
    assert call(k=96) == B.TL_ERR_INVALID_ARG and b"groupSize=64" in lib.tl_last_error(ctx)
    assert call(scales=None) == B.TL_ERR_INVALID_ARG and b"scales" in lib.tl_last_error(ctx)
    assert call(packed=None) == B.TL_ERR_INVALID_ARG
    assert call(out=None) == B.TL_ERR_INVALID_ARG
    assert call(qd=None) == B.TL_ERR_INVALID_ARG and b"packing" in lib.tl_last_error(ctx)
    assert call(qd=B.QuantDesc(7, 64, B.TL_F16, 0)) == B.TL_ERR_UNSUPPORTED and b"scheme" in lib.tl_last_error(ctx)
    assert call(adt=9) == B.TL_ERR_INVALID_ARG
    assert call(a=buf + 2, adt=B.TL_F32) == B.TL_ERR_INVALID_ARG and b"misaligned" in lib.tl_last_error(ctx)
    e = B.Epilogue()
    e.n_ops = 1
    e.ops[0] = B.EpilogueOp(B.TL_EPI_BIAS, 0, 0, 0)
    e.n_inputs = 0
    assert call(epi=C.byref(e)) == B.TL_ERR_INVALID_ARG and b"input" in lib.tl_last_error(ctx)
    e.ops[0] = B.EpilogueOp(B.TL_EPI_UNARY, 99, 0, 0)
    assert call(epi=C.byref(e)) == B.TL_ERR_UNSUPPORTED
    assert be.getKernelLaunchCount() == launches
    assert lib.tl_qgemv_nt(None, buf, 0, buf, buf, buf, 0, 1, 8, 64, C.byref(q), 1.0, None) == B.TL_ERR_INVALID_ARG
    be._free(buf)
    with pytest.raises(tb.TlError, match="packed length"):
        be.createQuantizedWeight(np.zeros(10, np.uint32), np.zeros(4, np.uint16), 4, 64, tb.resolveWeightFormat("int8-64"))
    with pytest.raises(tb.TlError, match="scales length"):
        be.createQuantizedWeight(np.zeros(64, np.uint32), np.zeros(3, np.uint16), 4, 64, tb.resolveWeightFormat("int8-64"))
    with pytest.raises(tb.TlError, match="packing is required"):
        be.createQuantizedWeight(np.zeros(64, np.uint32), np.zeros(4, np.uint16), 4, 64, tb.StorageFormat("f16"))


def test_forced_variant_must_be_applicable(backend):
    be = backend
    cs = cases.per_channel_case(32, 80, 1, seed=1)  # K % 64 != 0: the mma kernel cannot run it
    wt = be.createQuantizedWeight(cs["packed"], cs["scales"], 32, 80, tb.perChannelFormat(80))
    xt = be.ops.tensorFromArray(cs["x"].astype(np.float16), [1, 80], "f16")
    be.forceVariant((1, 3, 4, 4, 0, 0))
    try:
        with pytest.raises(tb.TlError, match="forced variant"):
            be.linear(xt, wt)
    finally:
        be.forceVariant(None)
    for t in (xt, wt.scales, wt):
        t.destroy()


# ---------------------------------------------------------------------------
# replay (captured graph) and counters
# ---------------------------------------------------------------------------

def test_captured_graph_survives_scratch_growth():
    """A graph captured on a kernel that uses library scratch (the TMA-fed GEMV's partial-sum
    meeting point) must stay valid when a later, larger call makes the scratch grow: the old buffer
    is retired, not freed, while the graph lives."""
    be = tb.CudaBackend(0)  # its own context: the scratch starts at its minimum size
    try:
        tma = (1, 5, 6, 0, 0, 0)
        pc = lambda kk: tb.QuantPacking("int8-grouped", kk, "f32", "direct")  # noqa: E731
        n, k, m = 512, 1024, 4
        cs = cases.per_channel_case(n, k, m, seed=21, act_dtype="f16")
        w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
        x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "f16")
        out = be.ops.empty([m, n], "f32")
        be.forceVariant(tma)
        be.dispatchQuantizedGemvNT(x, w, w.scales, out, n, k, k, m=m, packing=pc(k))  # eager: sizes the scratch (1 MiB minimum)
        first = np.array(be.ops.read(out), dtype=np.float32)
        ref = orc.linear_reference(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k), None, None)
        assert cases.rel_err(first, ref) <= TOL_F32
        be.beginCapture()
        be.dispatchQuantizedGemvNT(x, w, w.scales, out, n, k, k, m=m, packing=pc(k))
        graph = be.endCapture()
        # a larger problem on the same variant: m*n*4 bytes of partial sums exceed 1 MiB -> the scratch grows
        n_big, kb = 80_000, 128
        cb = cases.per_channel_case(n_big, kb, 4, seed=22, act_dtype="f16")
        wb = be.createQuantizedWeight(cb["packed"], cb["scales"], n_big, kb, tb.perChannelFormat(kb))
        xb = be.ops.tensorFromArray(cb["x_bits"], [4, kb], "f16")
        outb = be.ops.empty([4, n_big], "f32")
        be.dispatchQuantizedGemvNT(xb, wb, wb.scales, outb, n_big, kb, kb, m=4, packing=pc(kb))
        refb = orc.linear_reference(cb["x"], orc.dequantize_direct_f32(cb["packed"], cb["scales"], kb, kb), None, None)
        assert cases.rel_err(be.ops.read(outb), refb) <= TOL_F32
        # the earlier graph still runs on its own (retired) scratch (this variant sums partial tiles
        # with atomics, so replays agree to rounding, not bit for bit)
        for _ in range(2):
            be._upload(out.buffer, np.zeros((m, n), dtype=np.float32))
            be.replay(graph)
            again = np.array(be.ops.read(out), dtype=np.float32)
            assert cases.rel_err(again, ref) <= TOL_F32 and cases.rel_err(again, first) <= 1e-5
        be.forceVariant(None)
        be.destroyGraph(graph)
        for t in (outb, xb, wb.scales, wb, out, x, w.scales, w):
            t.destroy()
        assert be.getGpuUncapturedErrorCount() == 0
    finally:
        be.destroy()


def test_graph_replay_matches_eager_and_counts(backend):
    """The reference's compiled plans engage on the 2nd+ run (probe-quant-compiled.ts
    loops 12 iterations at N=2048, K=2304, G=64, seed 0x93, w = rng()*0.05, drift <= 5e-3)."""
    be = backend
    n, k, group = 2048, 2304, 64
    w, st = orc.lcg_fill(0x93, n * k, 0.05)
    packed, scales = be.quantizeLinearWeight(w.reshape(n, k), group)
    wt = be.createQuantizedWeight(packed, scales, n, k, tb.resolveWeightFormat("int8-64"))
    deq = orc.dequantize_to_f32(packed, scales, k, group)
    xt = be.ops.empty([1, k], "f32")
    out = be.ops.empty([1, n], "f32")
    x0, st = orc.lcg_fill(st, k)
    be._upload(xt.buffer, x0)
    be.dispatchQuantizedGemvNT(xt, wt, wt.scales, out, n, k, group)  # eager run first
    be.beginCapture()
    be.dispatchQuantizedGemvNT(xt, wt, wt.scales, out, n, k, group)
    graph = be.endCapture()
    total_hits = 0
    for _ in range(12):
        x, st = orc.lcg_fill(st, k)
        be._upload(xt.buffer, x)
        q0 = be.getQuantGemvDispatchCount()
        be.replay(graph)
        total_hits += be.getQuantGemvDispatchCount() - q0
        ref = orc.matmul_nt(x.reshape(1, k), deq)
        assert cases.drift(be.ops.read(out), ref) <= 5e-3
    assert total_hits == 12
    be.destroyGraph(graph)
    for t in (out, xt, wt.scales, wt):
        t.destroy()


# ---------------------------------------------------------------------------
# autotune surface (test/webgpu/matmul-autotune.spec.ts:310-464, 518-764)
# ---------------------------------------------------------------------------

def test_autotune_cache_semantics(backend):
    be = backend
    pk = tb.perChannelFormat(1024).packing
    be.clearPerShapeMatmulChoices()
    assert be.getPerShapeMatmulChoice(1, 2048, 1024, "f16", pk) is None
    default = be.planQuantizedMatmul(1, 2048, 1024, "f16", "f32", pk)
    assert default["family"] == "gemv" and not default["fromTuningCache"]
    runs = be.getAutotuneRunCount()
    # pretune is a no-op until autotuning is switched on (dispatch.ts:557-562)
    assert not be.isAutotuneEnabled()
    be.pretuneMatmulShapes([(1, 2048, 1024)], "f16", "f32", pk)
    assert be.getAutotuneRunCount() == runs and be.getPerShapeMatmulChoice(1, 2048, 1024, "f16", pk) is None
    be.setAutotuneEnabled(True)
    be.pretuneMatmulShapes([(1, 2048, 1024)], "f16", "f32", pk)
    assert be.getAutotuneRunCount() == runs + 1
    won = be.getPerShapeMatmulChoice(1, 2048, 1024, "f16", pk)
    assert won is not None and won[0] == B.TL_FAMILY_QGEMV
    be.pretuneMatmulShapes([(1, 2048, 1024)], "f16", "f32", pk)  # cache hit: no new search
    assert be.getAutotuneRunCount() == runs + 1
    assert be.planQuantizedMatmul(1, 2048, 1024, "f16", "f32", pk)["fromTuningCache"]
    # per-dtype separation
    assert be.getPerShapeMatmulChoice(1, 2048, 1024, "f32", pk) is None
    # a seeded winner short-circuits planning and changes the launch geometry
    be.seedPerShapeMatmulChoice(1, 2048, 1024, "f16", pk, (1, 1, 4, 2, 1, 0))
    seeded = be.planQuantizedMatmul(1, 2048, 1024, "f16", "f32", pk)
    assert ".simt" in seeded["variant"] and seeded["grid"][0] == 2048 // 8 and seeded["block"] == 128
    # a seeded winner is re-gated on applicability: f32 activations cannot use the mma kernel
    be.seedPerShapeMatmulChoice(1, 2048, 1024, "f32", pk, (1, 2, 8, 4, 1, 0))
    assert ".simt" in be.planQuantizedMatmul(1, 2048, 1024, "f32", "f32", pk)["variant"]
    # export / import round trip, invalid JSON rejected without touching the cache
    text = be.exportTuningCache()
    be.clearPerShapeMatmulChoices()
    assert be.getPerShapeMatmulChoice(1, 2048, 1024, "f16", pk) is None
    with pytest.raises(tb.TlError, match="invalid"):
        be.importTuningCache("{not json")
    assert be.getPerShapeMatmulChoice(1, 2048, 1024, "f16", pk) is None
    be.importTuningCache(text)
    assert be.getPerShapeMatmulChoice(1, 2048, 1024, "f16", pk) == (1, 1, 4, 2, 1, 0)
    be.clearPerShapeMatmulChoices()
    assert be.isAutotuneEnabled()
    be.setAutotuneEnabled(False)
    assert not be.isAutotuneEnabled()


def test_tuned_winner_still_matches_oracle(backend):
    be = backend
    n, k = 3072, 1024
    pk = tb.perChannelFormat(k).packing
    be.setAutotuneEnabled(True)
    be.pretuneMatmulShapes([(1, n, k), (8, n, k)], "f16", "f32", pk)
    be.setAutotuneEnabled(False)
    assert be.getPerShapeMatmulChoice(1, n, k, "f16", pk) is not None
    for m in (1, 8):
        cs = cases.per_channel_case(n, k, m, seed=31 + m, act_dtype="f16")
        got, ref = _run_direct(be, cs, m, n, k, "f16", "f32")
        assert cases.rel_err(got, ref) <= TOL_F32
    be.clearPerShapeMatmulChoices()


# ---------------------------------------------------------------------------
# horizontal fusion: several projections over the same activations in one launch
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("m,k,ns,act_dtype", [(1, 1024, (2048, 1024, 1024), "f16"), (8, 512, (304, 48), "bf16"),
                                             (16, 256, (64, 64, 64, 64), "f16"), (3, 80, (32, 16), "f16")])
def test_batched_gemv_matches_separate_calls_and_oracle(backend, m, k, ns, act_dtype):
    be = backend
    lib, ctx = be._lib, be._ctx
    cs0 = cases.per_channel_case(8, k, m, seed=99, act_dtype=act_dtype)
    x = be.ops.tensorFromArray(cs0["x_bits"], [m, k], act_dtype)
    q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, k, B.TL_F32, B.TL_SCALE_DIRECT)
    items = (B.QGemvItem * len(ns))()
    held, refs, outs = [], [], []
    for i, n in enumerate(ns):
        cs = cases.per_channel_case(n, k, m, seed=200 + i, bias=True)
        w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
        bias = be.ops.tensorFromArray(cs["bias"], [n], "f32")
        out = be.ops.empty([m, n], "f32")
        e = None
        if i % 2 == 0:  # every other item carries its own epilogue
            e = B.Epilogue()
            e.n_ops, e.n_inputs = 2, 1
            e.ops[0] = B.EpilogueOp(B.TL_EPI_BIAS, 0, 0, 0)
            e.ops[1] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY["silu"], 0, 0)
            e.inputs[0] = bias.buffer
        alpha = 0.5 + 0.25 * i
        items[i] = B.QGemvItem(w.buffer, w.scales.buffer, out.buffer, n, alpha, C.pointer(e) if e is not None else None)
        held += [w, bias, e]
        outs.append(out)
        wref = orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k)
        refs.append(orc.linear_reference(cs0["x"], wref, cs["bias"] if e is not None else None, "silu" if e is not None else None, alpha))
    q0, l0 = be.getQuantGemvDispatchCount(), be.getKernelLaunchCount()
    B.check(ctx, lib.tl_qgemv_nt_batched(ctx, x.buffer, B.DTYPE_ID[act_dtype], items, len(ns), B.TL_F32, m, k, C.byref(q)))
    assert be.getQuantGemvDispatchCount() == q0 + len(ns)
    if k % 64 == 0:
        assert be.getKernelLaunchCount() == l0 + 1  # one launch for all items
    for out, ref in zip(outs, refs):
        assert cases.rel_err(be.ops.read(out), ref) <= TOL_F32
    with pytest.raises(tb.TlError, match="items"):
        B.check(ctx, lib.tl_qgemv_nt_batched(ctx, x.buffer, B.DTYPE_ID[act_dtype], items, 5, B.TL_F32, m, k, C.byref(q)))
    for t in outs + [h for h in held if isinstance(h, tb.CudaTensor)] + [x]:
        if t.scales is not None:
            t.scales.destroy()
        t.destroy()


@pytest.mark.parametrize("variant", [(1, 3, 4, 4, 0, 0), (1, 5, 6, 0, 0, 0), (1, 6, 16, 32, 0, 0), (1, 4, 4, 6, 0, 0), (1, 2, 8, 4, 1, 0)])
@pytest.mark.parametrize("group", [64, 128])
def test_grouped_scales_on_every_fast_variant(backend, variant, group):
    """Reference-native format (f16 group scales) forced through each tensor-core GEMV variant."""
    be = backend
    n, k, m = 520, 1024, 5
    rng = np.random.default_rng(group + variant[1])
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scales = be.quantizeLinearWeight(w, group)
    fmt = tb.resolveWeightFormat(f"int8-{group}")
    wt = be.createQuantizedWeight(packed, scales, n, k, fmt)
    xt = be.ops.tensorFromArray(x, [m, k], "f16")
    ref = orc.matmul_nt(x.astype(np.float32), orc.dequantize_to_f32(packed, scales, k, group))
    be.forceVariant(variant)
    try:
        if variant[1] == 3 and group == 64:
            with pytest.raises(tb.TlError, match="forced variant"):  # its MMAs span 128 k: not applicable
                be.linear(xt, wt)
        else:
            y = be.linear(xt, wt)
            assert cases.rel_err(be.ops.read(y), ref) <= TOL_F32
            y.destroy()
    finally:
        be.forceVariant(None)
    for t in (xt, wt.scales, wt):
        t.destroy()


def test_ring_launch_shape_fits_one_wave_when_it_can(backend):
    """The default ring shape comes from the occupancy calculator: if any of the 16-, 8- or
    4-warp shapes lets the whole launch be resident at once, the launch is a single wave
    (grid <= resident CTAs), and few-tile matrices get the widest CTA."""
    be = backend
    sms = be.smCount()
    for (n, k) in [(4096, 4096), (4096, 12288), (6144, 4096), (14336, 4096), (1024, 4096)]:
        plan = be.planQuantizedMatmul(8, n, k, "f16", "f16", tb.perChannelFormat(k).packing)
        assert ".ring" in plan["variant"]
        warps, depth = plan["choice"][2], plan["choice"][3]
        assert warps in (4, 8, 16) and depth in (2, 4, 6, 8)
        assert plan["grid"][0] == (n + 15) // 16 and plan["block"] == warps * 32
        # one wave: at most 2048 threads and 64K registers per SM bound the resident CTAs
        assert plan["grid"][0] <= sms * (2048 // plan["block"])
    assert be.planQuantizedMatmul(8, 1024, 4096, "f16", "f16", tb.perChannelFormat(4096).packing)["choice"][2] == 16
    # far more tiles than one wave holds: 4-warp CTAs
    assert be.planQuantizedMatmul(8, 151936, 4096, "f16", "f16", tb.perChannelFormat(4096).packing)["choice"][2] == 4


@pytest.mark.parametrize("m,act_dtype", [(1, "f16"), (8, "f16"), (8, "bf16"), (13, "f16"), (16, "bf16")])
@pytest.mark.parametrize("warps,depth", [(4, 2), (8, 4), (16, 2)])
def test_wide_ring_tiles_give_the_same_bits(backend, m, act_dtype, warps, depth):
    """32-row ring tiles (variant p2 = 2: one activation fragment feeds two MMA row tiles) against the
    16-row tiles of the same warp count: same summation order, so the same bits; ragged N and K."""
    be = backend
    n, k = 1000, 832   # 31 full 32-row tiles + 8 rows; 13 k blocks over 4 / 8 / 16 warps
    cs = cases.per_channel_case(n, k, m, seed=50 + m, act_dtype=act_dtype, bias=True)
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], act_dtype)
    b = be.ops.tensorFromArray(cs["bias"], [n], "f32")
    outs = []
    for wide in (0, 2):
        be.forceVariant((1, 4, warps, depth, wide, 0))
        try:
            y = be.linear(x, w, b, "silu", "f32")
        finally:
            be.forceVariant(None)
        outs.append(be.ops.read(y).copy())
        y.destroy()
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    wref = orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k)
    ref = orc.linear_reference(cs["x"], wref, cs["bias"], "silu")
    assert cases.rel_err(outs[1], ref) <= TOL_F32
    for t in (x, b, w.scales, w):
        t.destroy()


def test_wide_ring_tiles_grouped_scales_and_batched_launch(backend):
    be = backend
    lib, ctx = be._lib, be._ctx
    m, k, group = 6, 512, 64
    rng = np.random.default_rng(61)
    x = rng.standard_normal((m, k)).astype(np.float16)
    xt = be.ops.tensorFromArray(x, [m, k], "f16")
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int8-grouped", group, "f16"))
    ws, outs, refs = [], [], []
    for n in (200, 72, 33):
        wf = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
        packed, scales = be.quantizeLinearWeight(wf, group)
        ws.append(be.createQuantizedWeight(packed, scales, n, k, fmt))
        outs.append(be.ops.empty([m, n], "f32"))
        refs.append(orc.matmul_nt(x.astype(np.float32), orc.dequantize_to_f32(packed, scales, k, group)))
    items = (B.QGemvItem * 3)()
    for i, (w, o) in enumerate(zip(ws, outs)):
        items[i] = B.QGemvItem(w.buffer, w.scales.buffer, o.buffer, w.shape[0], 1.0, None)
    q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, group, B.TL_F16, B.TL_SCALE_SNORM127)
    be.forceVariant((1, 4, 4, 4, 2, 0))
    try:
        B.check(ctx, lib.tl_qgemv_nt_batched(ctx, xt.buffer, B.TL_F16, items, 3, B.TL_F32, m, k, C.byref(q)))
    finally:
        be.forceVariant(None)
    for o, ref in zip(outs, refs):
        assert cases.rel_err(be.ops.read(o).reshape(ref.shape), ref) <= TOL_F32
    for t in [xt] + outs + [w.scales for w in ws] + ws:
        t.destroy()
    assert be.getGpuUncapturedErrorCount() == 0


# ---------------------------------------------------------------------------
# How each KERNEL unpacks: every byte value (-128 included: the dequantizer does not clamp,
# quantize.ts:138-156) in every byte lane, read back through the product with one-hot activations.
# One non-zero term per output and a power-of-two scale: the result is exact in every kernel.
# ---------------------------------------------------------------------------
def _lane_matrix(n, k):
    q = ((np.arange(n)[:, None] + 37 * np.arange(k)[None, :]) % 256 - 128).astype(np.int8)
    for lane in range(4):
        assert len(np.unique(q[:, lane::4])) == 256
    return q


def _one_hot_products(be, fn_name, variant, n, k, act_dtype):
    lib, ctx = be._lib, be._ctx
    q = _lane_matrix(n, k)
    packed = np.ascontiguousarray(q).view(np.uint32).reshape(n, k // 4)
    scales = np.full((n,), 0.5, np.float32)
    w = be.createQuantizedWeight(packed, scales, n, k, tb.perChannelFormat(k))
    qd = be._qdesc(w.format.packing)
    out = be.ops.empty([16, n], "f32")
    be.forceVariant(variant)
    try:
        for k0 in range(0, k, 16):
            x = np.zeros((16, k), np.float32)
            x[np.arange(16), k0 + np.arange(16)] = 1.0
            xt = be.ops.tensorFromArray(x.astype(np.float16) if act_dtype == "f16" else orc.bf16_bits_rne(x.reshape(-1)), [16, k], act_dtype)
            rc = getattr(lib, fn_name)(ctx, xt.buffer, B.DTYPE_ID[act_dtype], w.buffer, w.scales.buffer, out.buffer, B.TL_F32, 16, n, k,
                                       C.byref(qd), 1.0, None)
            if rc == B.TL_ERR_UNSUPPORTED:
                xt.destroy()
                pytest.skip(f"variant {variant} does not run m=16 n={n} k={k}: {lib.tl_last_error(ctx).decode()}")
            B.check(ctx, rc)
            got = be.ops.read(out)
            expect = q[:, k0:k0 + 16].T.astype(np.float32) * 0.5
            assert np.array_equal(got, expect), (variant, k0)
            xt.destroy()
    finally:
        be.forceVariant(None)
        for t in (out, w.scales, w):
            t.destroy()


@pytest.mark.parametrize("act_dtype", ["f16", "bf16"])
@pytest.mark.parametrize("variant", [None] + GEMV_VARIANTS_HALF)
def test_gemv_kernels_unpack_every_byte_in_every_lane(backend, variant, act_dtype):
    _one_hot_products(backend, "tl_qgemv_nt", variant, 256, 128, act_dtype)


@pytest.mark.parametrize("act_dtype", ["f16", "bf16"])
@pytest.mark.parametrize("variant", [None, (2, 0, 16, 128, 8, 8), (2, 0, 128, 64, 8, 4), (2, 0, 192, 128, 3, 8)])
def test_tcgen05_converter_unpacks_every_byte_in_every_lane(backend, variant, act_dtype):
    _one_hot_products(backend, "tl_qgemm_nt", variant, 256, 128, act_dtype)


@pytest.mark.parametrize("m", [1, 8, 64])
def test_gated_mlp_first_half_rides_in_the_epilogue(backend, m):
    """silu(x Wg^T) * (x Wu^T) with the multiply fused into the gate projection's epilogue
    (packages/qwen3-browser/src/model.ts:360-364) against the oracle's unfused sequence."""
    be = backend
    n, k = 768, 512
    cg = cases.per_channel_case(n, k, m, seed=61, act_dtype="f16")
    cu = cases.per_channel_case(n, k, m, seed=62, act_dtype="f16")
    wg = be.createQuantizedWeight(cg["packed"], cg["scales"], n, k, tb.perChannelFormat(k))
    wu = be.createQuantizedWeight(cu["packed"], cu["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cg["x_bits"], [m, k], "f16")
    be.resetCounters()
    h = be.swiglu(x, wg, wu, "f32")
    launches = be.getKernelLaunchCount()
    assert launches == 2, launches  # two products, no element-wise kernel
    g_ref = orc.linear_reference(cg["x"], orc.dequantize_direct_f32(cg["packed"], cg["scales"], k, k), None, "silu")
    u_ref = orc.linear_reference(cg["x"], orc.dequantize_direct_f32(cu["packed"], cu["scales"], k, k))
    ref = (g_ref.astype(np.float64) * u_ref.astype(np.float64)).astype(np.float32)
    assert cases.rel_err(be.ops.read(h), ref) <= 1e-3
    for t in (h, x, wg.scales, wg, wu.scales, wu):
        t.destroy()
