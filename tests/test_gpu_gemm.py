"""GPU parity tests of the tensor-core (tcgen05 / TMEM) quantized GEMM against the
CPU oracle, through the C ABI.

Tolerances: f32 outputs of per-channel weights within 1e-3 (the int8 values enter
the tensor core exactly and the per-channel scale is applied to the f32
accumulator); f16/bf16 outputs, and grouped scales (which are multiplied into the
16-bit operand), within 1e-2.  Metric: |x - ref| / max(1, |ref|).
"""
import numpy as np
import pytest

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B

pytestmark = pytest.mark.gpu

TC_CONFIGS = [(2, 0, 192, 64, 6, 4), (2, 0, 192, 64, 6, 8), (2, 0, 128, 64, 8, 4), (2, 0, 128, 64, 8, 8),
              (2, 0, 64, 128, 6, 8), (2, 0, 32, 128, 8, 8), (2, 0, 16, 128, 8, 8), (2, 0, 128, 128, 4, 8),
              (2, 0, 192, 128, 3, 8), (2, 0, 128, 128, 4, 16), (2, 0, 192, 128, 3, 16)]


def _gemm_case(be, m, n, k, act_dtype, out_dtype, variant=None, bias=False, act=None, seed=0, rows=None):
    cs = cases.per_channel_case(n, k, m, seed=seed, act_dtype=act_dtype, bias=bias)
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], act_dtype)
    bt = be.ops.tensorFromArray(cs["bias"], [n], "f32") if bias else None
    be.forceVariant(variant)
    g0 = be.getQuantGemmDispatchCount()
    try:
        y = be.linear(x, w, bt, act, out_dtype)
    finally:
        be.forceVariant(None)
    assert be.getQuantGemmDispatchCount() == g0 + 1 and be.getDequantI8DispatchCount() >= 0
    got = be.ops.read(y)
    got = orc.bf16_bits_to_f32(got) if out_dtype == "bf16" else np.asarray(got, dtype=np.float32)
    wref = orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k)
    sel = np.arange(m) if rows is None else np.asarray(rows)
    ref = orc.linear_reference(cs["x"][sel], wref, cs["bias"] if bias else None, act)
    for t in (w.scales, w, x, y) + ((bt,) if bt else ()):
        t.destroy()
    be.sync()
    return got[sel], ref


@pytest.mark.parametrize("variant", TC_CONFIGS)
@pytest.mark.parametrize("act_dtype", ["bf16", "f16"])
def test_qgemm_every_tile_config(backend, variant, act_dtype):
    # n, m, k all ragged with respect to the 128 x BN x KSTEP tiles
    got, ref = _gemm_case(backend, 200, 300, 448, act_dtype, "f32", variant, bias=True, act="gelu", seed=3)
    assert cases.rel_err(got, ref) <= 1e-3, variant
    assert backend.getGpuUncapturedErrorCount() == 0


@pytest.mark.parametrize("m,n,k", [(17, 128, 64), (33, 130, 80), (64, 256, 1024), (257, 1000, 2048), (500, 384, 4096)])
def test_qgemm_default_selection_shapes(backend, m, n, k):
    got, ref = _gemm_case(backend, m, n, k, "bf16", "bf16", None, bias=True, act="silu", seed=m)
    assert cases.rel_err(got, ref) <= 1e-2
    got, ref = _gemm_case(backend, m, n, k, "f16", "f16", None, seed=m + 1)
    assert cases.rel_err(got, ref) <= 1e-2


def test_qgemm_many_tiles_per_cta_exercises_both_accumulators(backend):
    # 8 x 40 = 320 tiles of 128 x 128 on 148 CTAs: every CTA walks several tiles and both TMEM buffers
    got, ref = _gemm_case(backend, 1024, 5120, 256, "bf16", "f32", (2, 0, 128, 64, 8, 4), bias=True, seed=11,
                          rows=[0, 1, 127, 128, 129, 511, 512, 1023])
    assert cases.rel_err(got, ref) <= 1e-3


def test_qgemm_partial_wave_is_cut_along_k_and_is_repeatable(backend):
    """Tiles beyond the last whole wave are split along K; partials are summed in part order,
    so two runs agree bit for bit, and the election counters are left clear for the next launch."""
    sms = backend.smCount()
    fmt = tb.perChannelFormat(1024).packing
    # a whole number of waves: nothing to cut
    plan = backend.planQuantizedMatmul(512, sms * 32, 1024, "bf16", "bf16", fmt)
    assert plan["family"] == "gemm" and plan["splitK"] == 1
    # 8 tiles on a machine of `sms` CTAs: cut four ways
    plan = backend.planQuantizedMatmul(256, 512, 1024, "bf16", "bf16", fmt)
    assert plan["splitK"] == 4 and plan["grid"][0] == 32
    runs = []
    for _ in range(3):
        got, ref = _gemm_case(backend, 256, 512, 1024, "bf16", "f32", None, bias=True, act="gelu", seed=21)
        assert cases.rel_err(got, ref) <= 1e-3
        runs.append(got.copy())
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    # whole waves followed by a cut remainder (2 * sms + 4 tiles of 128 x 128)
    n = 128 * (sms + 2)
    got, ref = _gemm_case(backend, 256, n, 256, "f16", "f32", (2, 0, 128, 128, 4, 8), seed=22,
                          rows=[0, 127, 128, 255])
    assert cases.rel_err(got, ref) <= 1e-3
    assert backend.getGpuUncapturedErrorCount() == 0


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("act_dtype", ["f16", "bf16"])
def test_qgemm_grouped_reference_native_format(backend, group, act_dtype):
    be = backend
    m, n, k = 96, 260, 512
    rng = np.random.default_rng(group)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if act_dtype == "f16":
        xb = x.astype(np.float16)
        x = xb.astype(np.float32)
    else:
        xb = orc.bf16_bits_rne(x)
        x = orc.bf16_bits_to_f32(xb)
    packed, scales = be.quantizeLinearWeight(w, group)
    wt = be.createQuantizedWeight(packed, scales, n, k, tb.resolveWeightFormat(f"int8-{group}", act_dtype))
    xt = be.ops.tensorFromArray(xb, [m, k], act_dtype)
    d0 = be.getDequantI8DispatchCount()
    y = be.linear(xt, wt)
    assert be.getDequantI8DispatchCount() == d0  # no explicit dequant on this route
    # the tensor-core operand is the dequantized weight rounded to the activation dtype
    w32 = orc.dequantize_to_f32(packed, scales, k, group)
    w16 = w32.astype(np.float16).astype(np.float32) if act_dtype == "f16" else orc.bf16_bits_to_f32(orc.bf16_bits_rne(w32))
    got = be.ops.read(y)
    assert cases.rel_err(got, orc.matmul_nt(x, w16)) <= 1e-2
    # and it stays close to the unrounded f32 control (the weight rounding itself is ~2^-9 per element in bf16)
    assert cases.rel_err(got, orc.matmul_nt(x, w32)) <= (2e-2 if act_dtype == "bf16" else 2e-3)
    for t in (y, xt, wt.scales, wt):
        t.destroy()


def test_qgemm_f32_activations_fall_back_to_row_slices(backend):
    be = backend
    m, n, k = 40, 96, 128
    cs = cases.per_channel_case(n, k, m, seed=2, bias=True)
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x"], [m, k], "f32")
    extra = np.random.default_rng(0).standard_normal((m, n)).astype(np.float32)
    et = be.ops.tensorFromArray(extra, [m, n], "f32")
    plan = be.planQuantizedMatmul(m, n, k, "f32", "f32", w.format.packing)
    assert plan["family"] == "gemm" and ".sliced" in plan["variant"]
    cfg, inputs, _ = tb.detectMatmulEpilogue([("add", et), ("relu", None)])
    y = be.ops.matmul(x, be.ops.transpose(w), {"epilogue": cfg, "epilogueInputs": inputs})
    ref = orc.matmul_nt(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k))
    ref = orc.unary("relu", (ref.astype(np.float64) + extra).astype(np.float32))
    assert cases.rel_err(be.ops.read(y), ref) <= 1e-3
    for t in (y, x, et, w.scales, w):
        t.destroy()


@pytest.mark.parametrize("k,n", [(4096, 14336), (14336, 4096)])
def test_config3_prefill_sampled(backend, k, n):
    """Benchmark config 3 at full size (M = 2048, bf16, gelu, bf16 out).  The oracle is
    run on a sample of token rows that covers every token-tile edge, over all N."""
    m = 2048
    rows = sorted({0, 1, 2, 127, 128, 191, 192, 193, 383, 384, 1023, 1024, 1919, 1920, 2046, 2047} |
                  set(np.random.default_rng(5).integers(0, m, 16).tolist()))
    got, ref = _gemm_case(backend, m, n, k, "bf16", "bf16", None, act="gelu", seed=33, rows=rows)
    assert cases.rel_err(got, ref) <= 1e-2
    # size-independent property: rows of zeros in, gelu(0) = 0 out; checked on a cheap second call
    be = backend
    w = be.createQuantizedWeight(np.zeros((256, k // 4), np.uint32), np.ones((256, 1), np.float32), 256, k,
                                 tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(orc.bf16_bits_rne(np.random.default_rng(1).standard_normal((64, k)).astype(np.float32)),
                               [64, k], "bf16")
    y = be.linear(x, w, None, "gelu", "bf16")
    assert not be.ops.read(y).any()
    for t in (y, x, w.scales, w):
        t.destroy()


def test_qgemm_graph_replay(backend):
    be = backend
    m, n, k = 128, 512, 512
    cs = cases.per_channel_case(n, k, m, seed=8, act_dtype="bf16")
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "bf16")
    out = be.ops.empty([m, n], "f32")
    wT = be.ops.transpose(w)
    be.ops.matmul(x, wT, {"outBuffer": out})
    be.beginCapture()
    be.ops.matmul(x, wT, {"outBuffer": out})
    graph = be.endCapture()
    be._lib.tl_memset(be._ctx, out.buffer, 0, out.nbytes)
    g0 = be.getQuantGemmDispatchCount()
    be.replay(graph)
    assert be.getQuantGemmDispatchCount() == g0 + 1
    ref = orc.matmul_nt(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k))
    assert cases.rel_err(be.ops.read(out), ref) <= 1e-3
    be.destroyGraph(graph)
    for t in (out, x, w.scales, w):
        t.destroy()


# ---------------------------------------------------------------------------
# "dequant+dense": the weight written once as a 16-bit matrix into library scratch, then the dense
# tensor-core kernel with the per-channel scales applied per output column (the reference's own
# structure for m > 1, matmul-ops.ts:163-181; here the default when tokens per weight byte are many)
# ---------------------------------------------------------------------------
DEQUANT_DENSE = (2, 2, 0, 0, 0, 0)


@pytest.mark.parametrize("act_dtype", ["bf16", "f16"])
@pytest.mark.parametrize("m,n,k", [(200, 300, 448), (33, 64, 64), (300, 1000, 2048)])
def test_qgemm_dequant_dense_per_channel(backend, act_dtype, m, n, k):
    got, ref = _gemm_case(backend, m, n, k, act_dtype, "f32", DEQUANT_DENSE, bias=True, act="gelu", seed=5)
    assert cases.rel_err(got, ref) <= 1e-3  # q enters the tensor core exactly, the scale meets the f32 accumulator
    got, ref = _gemm_case(backend, m, n, k, act_dtype, act_dtype, DEQUANT_DENSE, seed=6)
    assert cases.rel_err(got, ref) <= 1e-2
    assert backend.getGpuUncapturedErrorCount() == 0


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("act_dtype", ["f16", "bf16"])
def test_qgemm_dequant_dense_grouped_matches_the_fused_kernel(backend, group, act_dtype):
    be = backend
    m, n, k = 96, 260, 512
    rng = np.random.default_rng(group + 1)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    xb = x.astype(np.float16) if act_dtype == "f16" else orc.bf16_bits_rne(x)
    xv = xb.astype(np.float32) if act_dtype == "f16" else orc.bf16_bits_to_f32(xb)
    packed, scales = be.quantizeLinearWeight(w, group)
    wt = be.createQuantizedWeight(packed, scales, n, k, tb.resolveWeightFormat(f"int8-{group}", act_dtype))
    xt = be.ops.tensorFromArray(xb, [m, k], act_dtype)
    outs = []
    for variant in (DEQUANT_DENSE, None):
        be.forceVariant(variant)
        try:
            y = be.linear(xt, wt)
        finally:
            be.forceVariant(None)
        outs.append(np.asarray(be.ops.read(y), dtype=np.float32))
        y.destroy()
    w32 = orc.dequantize_to_f32(packed, scales, k, group)
    w16 = w32.astype(np.float16).astype(np.float32) if act_dtype == "f16" else orc.bf16_bits_to_f32(orc.bf16_bits_rne(w32))
    assert cases.rel_err(outs[0], orc.matmul_nt(xv, w16)) <= 1e-2  # the fused kernel's own bound for grouped scales
    assert cases.rel_err(outs[0], outs[1]) <= 1e-4                 # same operand arithmetic as the fused converters: only the summation order differs
    for t in (xt, wt.scales, wt):
        t.destroy()


def test_qgemm_default_goes_dense_only_when_tokens_per_weight_are_many(backend):
    be = backend
    fmt = tb.perChannelFormat(14336).packing
    assert ".dequant+dense" in be.planQuantizedMatmul(2048, 4096, 14336, "bf16", "bf16", fmt)["variant"]
    fmt = tb.perChannelFormat(4096).packing
    assert ".tcgen05" in be.planQuantizedMatmul(2048, 14336, 4096, "bf16", "bf16", fmt)["variant"]
    assert ".tcgen05" in be.planQuantizedMatmul(512, 14336, 4096, "bf16", "bf16", fmt)["variant"]
    assert ".dequant+dense" in be.planQuantizedMatmul(8192, 4096, 4096, "bf16", "bf16", fmt)["variant"]
    g128 = tb.resolveWeightFormat("int8-128", "bf16").packing
    assert ".dequant+dense" in be.planQuantizedMatmul(2048, 14336, 4096, "bf16", "bf16", g128)["variant"]
    assert ".tcgen05" in be.planQuantizedMatmul(128, 14336, 4096, "bf16", "bf16", g128)["variant"]


def test_qgemm_dequant_dense_graph_replay(backend):
    be = backend
    m, n, k = 256, 512, 512
    cs = cases.per_channel_case(n, k, m, seed=9, act_dtype="bf16")
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "bf16")
    out = be.ops.empty([m, n], "f32")
    wT = be.ops.transpose(w)
    be.forceVariant(DEQUANT_DENSE)
    try:
        be.ops.matmul(x, wT, {"outBuffer": out})  # sizes the scratch outside the capture
        be.beginCapture()
        be.ops.matmul(x, wT, {"outBuffer": out})
        graph = be.endCapture()
    finally:
        be.forceVariant(None)
    be._lib.tl_memset(be._ctx, out.buffer, 0, out.nbytes)
    be.replay(graph)
    ref = orc.matmul_nt(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k))
    assert cases.rel_err(be.ops.read(out), ref) <= 1e-3
    be.destroyGraph(graph)
    for t in (out, x, w.scales, w):
        t.destroy()
