"""CPU tests of the oracle: the C restatement against IEEE facts, an independent
numpy restatement, the committed known-answer fixtures and the reference probes'
seeds / shapes / tolerances."""
import os

import numpy as np
import pytest

import cases
from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _ulp_or_abs_close(a, b, ulps=1, atol=1e-12):
    ulp = np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))
    return bool(np.all((ulp <= ulps) | (np.abs(a.astype(np.float64) - b.astype(np.float64)) <= atol)))


def test_f16_bits_to_f32_all_patterns_match_ieee():
    bits = np.arange(65536, dtype=np.uint16)
    ours = orc.f16_bits_to_f32(bits)
    ieee = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(ieee)
    assert np.array_equal(np.isnan(ours), nan)
    assert np.array_equal(ours[~nan].view(np.uint32), ieee[~nan].view(np.uint32))


def test_f32_to_f16_roundtrips_every_f16_value():
    bits = np.arange(65536, dtype=np.uint16)
    vals = bits.view(np.float16).astype(np.float32)
    finite = np.isfinite(vals)
    back = orc.f32_to_f16_bits(vals[finite])
    assert np.array_equal(back, bits[finite])


def test_f32_to_f16_is_rne_on_normals_and_half_up_on_subnormals():
    rng = np.random.default_rng(1)
    v = (rng.standard_normal(20000) * np.exp(rng.uniform(-8, 8, 20000))).astype(np.float32)
    v = v[(np.abs(v) >= 6.2e-5) & (np.abs(v) < 65000)]
    assert np.array_equal(orc.f32_to_f16_bits(v), v.astype(np.float16).view(np.uint16))
    # subnormal branch (quantize.ts:30-37): shifts, then rounds up on bit 12 only.
    # 2^-25 is an exact tie that IEEE rounds to even (0); the reference rounds it up to 1.
    assert int(orc.f32_to_f16_bits(np.float32(2.0 ** -25))) == 1
    assert int(np.float32(2.0 ** -25).astype(np.float16).view(np.uint16)) == 0
    assert int(orc.f32_to_f16_bits(np.float32(2.0 ** -26))) == 0  # exp < -10 flushes
    assert int(orc.f32_to_f16_bits(np.float32(1e6))) == 0x7C00  # overflow -> inf
    assert int(orc.f32_to_f16_bits(np.float32(-1e6))) == 0xFC00


def test_unpack_every_int8_value_in_every_lane():
    q = np.zeros((4, 256 * 4), dtype=np.int8)
    for lane in range(4):
        q[lane, lane::4] = np.arange(-128, 128, dtype=np.int8)
    packed = cases.pack_int8(q)
    assert np.array_equal(orc.unpack_int8(packed, q.shape[1]), q)
    assert np.array_equal(orc.np_unpack_int8(packed, q.shape[1]), q)
    # lane order: lowest k in bits 0-7 (quantize.ts:122-126)
    one = np.array([[1, 2, 3, -1]], dtype=np.int8)
    assert int(cases.pack_int8(one)[0, 0]) == 0xFF030201


@pytest.mark.parametrize("group", [64, 128])
def test_quantizer_properties_and_numpy_crosscheck(group):
    rng = np.random.default_rng(group)
    w = (rng.standard_normal((48, 256)) * 0.05).astype(np.float32)
    w[3, :group] = 0.0  # a zero group: scale 0, all q 0 (quantize.ts:109-115)
    packed, scales = orc.quantize_linear_weight(w, group)
    q = orc.unpack_int8(packed, 256)
    assert q.min() >= -127 and q.max() <= 127
    amax = np.abs(w).reshape(48, -1, group).max(axis=2)
    assert np.array_equal(scales, amax.astype(np.float16).view(np.uint16))
    assert np.all(q[3, :group] == 0) and scales[3, 0] == 0
    # independent restatement of the rounding: floor(x*inv + 0.5)
    s = scales.view(np.float16).astype(np.float64)
    inv = np.where(s > 0, 127.0 / np.where(s > 0, s, 1.0), 0.0)
    expect = np.clip(np.floor(w.astype(np.float64) * np.repeat(inv, group, axis=1) + 0.5), -127, 127)
    assert np.array_equal(q.astype(np.float64), expect)
    deq = orc.dequantize_to_f32(packed, scales, 256, group)
    assert np.array_equal(deq.view(np.uint32), orc.np_dequantize_to_f32(packed, scales, 256, group).view(np.uint32))
    # quantization error is at most half a step (plus the f16 rounding of the abs-max)
    step = np.repeat(s, group, axis=1) / 127.0
    assert np.all(np.abs(deq - w) <= 0.5 * step + np.abs(w) * 2.0 ** -10 + 1e-12)


def test_quantizer_rejects_bad_shapes():
    w = np.zeros((2, 130), dtype=np.float32)
    with pytest.raises(ValueError):
        orc.quantize_linear_weight(w, 64)


def test_math_round_ties_go_up():
    # w*inv = -0.5 rounds to -0 -> 0 ; +0.5 rounds to 1 ; -1.5 -> -1 ; 2.5 -> 3
    w = np.zeros((1, 64), dtype=np.float32)
    w[0, 0] = 127.0  # abs-max 127 -> inv = 1
    w[0, 1:5] = [-0.5, 0.5, -1.5, 2.5]
    packed, _ = orc.quantize_linear_weight(w, 64)
    assert orc.unpack_int8(packed, 64)[0, :5].tolist() == [127, 0, 1, -1, 3]


def test_direct_dequant_is_single_rounding():
    cs = cases.per_channel_case(16, 64, 1, seed=3)
    d = orc.dequantize_direct_f32(cs["packed"], cs["scales"], 64, 64)
    expect = (cs["q"].astype(np.float64) * cs["scales"].astype(np.float64)).astype(np.float32)
    assert np.array_equal(d.view(np.uint32), expect.view(np.uint32))
    assert np.array_equal(d.view(np.uint32), orc.np_dequantize_direct_f32(cs["packed"], cs["scales"], 64, 64).view(np.uint32))


def test_matmul_sequential_f64_and_thread_independent():
    rng = np.random.default_rng(5)
    a = rng.standard_normal((3, 200)).astype(np.float32)
    w = rng.standard_normal((37, 200)).astype(np.float32)
    y1 = orc.matmul_nt(a, w, threads=1)
    assert np.array_equal(y1.view(np.uint32), orc.np_matmul_nt_small(a, w).view(np.uint32))
    assert np.array_equal(y1.view(np.uint32), orc.matmul_nt(a, w, threads=4).view(np.uint32))
    assert np.allclose(y1, a.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("name", ["relu", "silu", "sigmoid", "tanh", "gelu", "gelu_erf"])
def test_unary_matches_numpy_restatement(name):
    x = np.linspace(-12, 12, 4001, dtype=np.float32)
    a, b = orc.unary(name, x), orc.np_unary(name, x)
    # libm and numpy may differ by an ulp in f64: at most 1 f32 ulp after the store, except
    # where 1 + tanh / 1 + erf cancels (large negative x), which gets an absolute bound
    assert _ulp_or_abs_close(a, b)


def test_unary_known_points():
    assert orc.unary("relu", np.array([-1.0, 0.0, 2.5], dtype=np.float32)).tolist() == [0.0, 0.0, 2.5]
    assert orc.unary("gelu", np.zeros(1, np.float32))[0] == 0.0
    assert abs(float(orc.unary("gelu", np.ones(1, np.float32))[0]) - 0.8411919906) < 1e-6
    assert abs(float(orc.unary("gelu_erf", np.ones(1, np.float32))[0]) - 0.8413447) < 2e-6
    assert abs(float(orc.unary("silu", np.ones(1, np.float32))[0]) - 0.7310585786) < 1e-6


def test_lcg_matches_python_and_js_semantics():
    v, s = orc.lcg_fill(0x51A7EE, 1000)
    v2, s2 = orc.np_lcg(0x51A7EE, 1000)
    assert s == s2 and np.array_equal(v.view(np.uint32), v2.view(np.uint32))
    assert v.min() >= -1.0 and v.max() < 1.0
    first = (0x51A7EE * 1664525 + 1013904223) % 2 ** 32
    assert v[0] == np.float32(first / 2 ** 31 - 1)


def test_golden_probe_quant_gemv():
    g = np.load(os.path.join(GOLDEN, "probe_quant_gemv_128x128_g64.npz"))
    w, st = orc.lcg_fill(0x51A7EE, 128 * 128)
    a, st = orc.lcg_fill(st, 128)
    assert st == int(g["next_state"])
    assert np.array_equal(w[:16], g["w_head"]) and np.array_equal(a, g["a"])
    packed, scales = orc.quantize_linear_weight(w.reshape(128, 128), 64)
    assert np.array_equal(packed, g["packed"]) and np.array_equal(scales, g["scales"])
    deq = orc.dequantize_to_f32(packed, scales, 128, 64)
    assert np.array_equal(deq[0], g["deq_row0"]) and np.array_equal(deq[127], g["deq_row127"])
    y = orc.matmul_nt(a.reshape(1, -1), deq, threads=1)
    assert np.array_equal(y, g["y"])
    # the probe's own gate: f32 control vs f64 host dot within 5e-4 (probe-quant-gemv.ts:166-187)
    ref64 = deq.astype(np.float64) @ a.astype(np.float64)
    assert cases.rel_err(y[0], ref64) <= 5e-4


def test_golden_probe_quant_operand_and_config0_and_elementwise():
    g = np.load(os.path.join(GOLDEN, "probe_quant_operand_128x128_g64_m4.npz"))
    deq = orc.dequantize_to_f32(g["packed"], g["scales"], 128, 64)
    assert np.array_equal(orc.matmul_nt(g["x"], deq, threads=2), g["y"])
    g0 = np.load(os.path.join(GOLDEN, "config0_rows0_63.npz"))
    cs = cases.per_channel_case(2048, 2048, 1, seed=0)
    assert np.array_equal(cs["q"][0, :32], g0["q_head"]) and np.array_equal(cs["x"][0, :32], g0["x_head"])
    wdq = orc.dequantize_direct_f32(cs["packed"][:64], cs["scales"][:64], 2048, 2048)
    assert np.array_equal(orc.matmul_nt(cs["x"], wdq), g0["y"])
    ge = np.load(os.path.join(GOLDEN, "elementwise.npz"))
    for name in ("relu", "silu", "sigmoid", "tanh", "gelu", "gelu_erf"):
        assert _ulp_or_abs_close(orc.unary(name, ge["xs"]), ge[name])
    assert np.array_equal(orc.f32_to_f16_bits(ge["f16_in"]), ge["f16_bits"])


def test_unfused_reference_sequence_rounds_between_ops():
    cs = cases.per_channel_case(32, 64, 2, seed=9, bias=True)
    w = orc.dequantize_direct_f32(cs["packed"], cs["scales"], 64, 64)
    y = orc.linear_reference(cs["x"], w, cs["bias"], "gelu")
    step = orc.unary("gelu", orc.add_bias(orc.matmul_nt(cs["x"], w), cs["bias"]))
    assert np.array_equal(y, step)
