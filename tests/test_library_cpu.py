"""CPU tests of the product's host side: the shared library loads and exports
every symbol the header declares, its host quantizer matches the oracle bit for
bit, the epilogue-fusion decision follows the reference, and nothing computes
without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tlcuda.h")).read()
    return sorted(set(re.findall(r"TL_API\s+[\w\s\*]+?\b(tl_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = B.load()
    declared = _declared_symbols()
    assert len(declared) >= 45
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in tlcuda.h but not exported"
    assert set(declared) == set(B.SIGNATURES), "binding.SIGNATURES and tlcuda.h disagree"


def test_struct_layouts_match_header():
    assert C.sizeof(B.QuantDesc) == 16
    assert C.sizeof(B.EpilogueOp) == 16
    assert C.sizeof(B.Epilogue) == 4 + 4 + 8 * 16 + 4 * 8 + 0 or C.sizeof(B.Epilogue) == 176
    assert C.sizeof(B.Variant) == 24
    assert C.sizeof(B.PlanReceipt) == 24 + 12 + 4 * 4


@pytest.mark.parametrize("group", [64, 128, 32])
def test_host_quantizer_bit_exact_vs_oracle(group):
    lib = B.load()
    w, _ = orc.lcg_fill(0x51A7EE, 96 * 384)
    w = w.reshape(96, 384)
    w[5, :group] = 0
    w[7, 3] = 1e-6  # tiny group values exercise the f16 subnormal branch
    w[7, :group] *= 1e-6
    w[9, 2] = np.nan      # Math.min/Math.max propagate NaN and `NaN & 0xff` is 0: the byte is 0
    w[11, 1] = np.inf     # infinite group scale: inv = 0, Inf * 0 = NaN -> 0, everything else 0 as well
    w[13, 0] = -np.inf
    packed = np.zeros((96, 96), dtype=np.uint32)
    scales = np.zeros((96, 384 // group), dtype=np.uint16)
    rc = lib.tl_quantize_linear_weight(w.ctypes.data_as(C.c_void_p), 96, 384, group,
                                       packed.ctypes.data_as(C.c_void_p), scales.ctypes.data_as(C.c_void_p))
    assert rc == 0
    op, os_ = orc.quantize_linear_weight(w, group)
    assert np.array_equal(packed, op) and np.array_equal(scales, os_)
    # known answers read off quantize.ts:100-126 for the non-finite rows
    q = orc.unpack_int8(op, 384)
    assert q[9, 2] == 0 and np.count_nonzero(q[9, :group]) > 0  # NaN is skipped by `a > absMax`, the rest quantizes
    assert os_[11, 0] == 0x7C00 and not q[11, :group].any()
    assert os_[13, 0] == 0x7C00 and not q[13, :group].any()


def test_host_quantizer_large_threaded_matches_oracle():
    lib = B.load()
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((512, 1024)) * 0.1).astype(np.float32)
    packed = np.zeros((512, 256), dtype=np.uint32)
    scales = np.zeros((512, 16), dtype=np.uint16)
    assert lib.tl_quantize_linear_weight(w.ctypes.data_as(C.c_void_p), 512, 1024, 64,
                                         packed.ctypes.data_as(C.c_void_p), scales.ctypes.data_as(C.c_void_p)) == 0
    op, os_ = orc.quantize_linear_weight(w, 64)
    assert np.array_equal(packed, op) and np.array_equal(scales, os_)


def test_host_quantizer_argument_errors():
    lib = B.load()
    w = np.zeros((2, 130), dtype=np.float32)
    out = np.zeros(1000, dtype=np.uint32)
    rc = lib.tl_quantize_linear_weight(w.ctypes.data_as(C.c_void_p), 2, 130, 64, out.ctypes.data_as(C.c_void_p),
                                       out.ctypes.data_as(C.c_void_p))
    assert rc == B.TL_ERR_INVALID_ARG
    assert b"divisible by 4" in lib.tl_last_error(None)
    rc = lib.tl_quantize_linear_weight(w.ctypes.data_as(C.c_void_p), 2, 128, 48, out.ctypes.data_as(C.c_void_p),
                                       out.ctypes.data_as(C.c_void_p))
    assert rc == B.TL_ERR_INVALID_ARG and b"groupSize=48" in lib.tl_last_error(None)
    assert lib.tl_quantize_linear_weight(None, 2, 128, 64, None, None) == B.TL_ERR_INVALID_ARG


def test_f16_converters_match_oracle_everywhere():
    lib = B.load()
    bits = np.arange(65536, dtype=np.uint16)
    ref = orc.f16_bits_to_f32(bits)
    got = np.array([lib.tl_f16_bits_to_f32(int(b)) for b in bits], dtype=np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan) and np.array_equal(got[~nan].view(np.uint32), ref[~nan].view(np.uint32))
    rng = np.random.default_rng(2)
    v = (rng.standard_normal(5000) * np.exp(rng.uniform(-20, 12, 5000))).astype(np.float32)
    v = np.concatenate([v, np.float32([0, -0.0, 2.0 ** -25, 2.0 ** -24, 6e-8, 65504, 65520, 1e9, -1e9])])
    got = np.array([lib.tl_f32_to_f16_bits(float(x)) for x in v], dtype=np.uint16)
    assert np.array_equal(got, orc.f32_to_f16_bits(v))


def test_no_compute_without_a_gpu_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-GPU failure path cannot be observed")
    lib = B.load()
    ctx = C.c_void_p()
    rc = lib.tl_ctx_create(0, C.byref(ctx))
    assert rc == B.TL_ERR_CUDA and not ctx.value
    assert b"CUDA" in lib.tl_last_error(None)
    assert tb.initCuda(0) is False and tb.getCudaInitError()
    with pytest.raises(RuntimeError):
        tb.getBackend()
    # null-context calls are rejected, not crashed
    assert lib.tl_sync(None) == B.TL_ERR_INVALID_ARG
    assert lib.tl_counter_get(None, 0) == -1


def test_weight_format_names():
    f = tb.resolveWeightFormat("int8-64")
    assert f.packing.groupSize == 64 and f.packing.scalesDtype == "f16" and f.elementType == "f16"
    assert tb.resolveWeightFormat("int8-128", "f32").packing.groupSize == 128
    f4 = tb.resolveWeightFormat("int4-32")
    assert f4.packing.scheme == "int4-grouped" and f4.packing.groupSize == 32 and f4.packing.scalesDtype == "f16"
    with pytest.raises(ValueError):
        tb.resolveWeightFormat("int2-32")
    pc = tb.perChannelFormat(4096)
    assert pc.packing.groupSize == 4096 and pc.packing.scaleConvention == "direct"


class _T:
    def __init__(self, shape):
        self.shape = shape


def test_epilogue_fusion_decision_follows_reference_rules():
    # cast then 1-D bias: directive order cast, bias (test/graph-compiler.spec.ts:269-314)
    plan = tb.detectMatmulEpilogue([("cast", "f16"), ("add", _T([64]))], "f32")
    cfg, inputs, consumed = plan
    assert [o["kind"] for o in cfg.ops] == ["cast", "bias"] and consumed == 2 and cfg.outputDtype == "f16"
    assert cfg.additionalInputCount == 1 and len(inputs) == 1
    # a 2-D second operand is a general binary add
    cfg, inputs, _ = tb.detectMatmulEpilogue([("add", _T([4, 64])), ("relu", None)])
    assert cfg.ops[0] == {"kind": "binary", "op": "add", "inputIndex": 0} and cfg.ops[1] == {"kind": "unary", "op": "relu"}
    # gelu approximate:"none" becomes gelu_erf (matmul-epilogue.ts:52-56)
    cfg, _, _ = tb.detectMatmulEpilogue([("gelu", {"approximate": "none"})])
    assert cfg.ops[0]["op"] == "gelu_erf"
    cfg, _, _ = tb.detectMatmulEpilogue([("gelu", None)])
    assert cfg.ops[0]["op"] == "gelu"
    # at most four ops are claimed; an unfusible op ends the chain
    cfg, _, consumed = tb.detectMatmulEpilogue([("relu", None)] * 6)
    assert consumed == 4 and len(cfg.ops) == 4
    cfg, _, consumed = tb.detectMatmulEpilogue([("relu", None), ("softmax", None), ("relu", None)])
    assert consumed == 1
    assert tb.detectMatmulEpilogue([("softmax", None)]) is None
    assert tb.detectMatmulEpilogue([]) is None


def test_case_generator_is_deterministic():
    a = cases.per_channel_case(8, 64, 2, seed=0, act_dtype="f16", bias=True)
    b = cases.per_channel_case(8, 64, 2, seed=0, act_dtype="f16", bias=True)
    for k in a:
        assert np.array_equal(a[k], b[k])
    assert a["q"].min() >= -127 and a["scales"].min() >= 0.001 and a["scales"].max() <= 0.01
    assert np.array_equal(a["x_bits"].view(np.float16).astype(np.float32), a["x"])


def test_int4_host_quantizer_matches_the_oracle_bit_for_bit():
    """tl_quantize_linear_weight_int4 against the oracle's restatement of the planned scheme
    (docs/quantization-design.md:69-75), including NaN / Inf / all-zero groups and ties."""
    from oracle import oracle as orc
    from torchlette_b200 import binding as B
    import ctypes as C
    lib = B.load()
    rng = np.random.default_rng(12)
    for n, k, g in [(3, 64, 32), (17, 256, 128), (5, 40, 8), (2, 32, 32)]:
        w = rng.uniform(-2, 2, (n, k)).astype(np.float32)
        w[0, :g] = 0.0
        w[1, 3] = np.nan
        w[min(2, n - 1), 5] = np.inf
        w[-1, :8] = np.array([0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 3.5, -3.5], np.float32) * (w[-1, :g].max() / 7.0)  # near ties
        packed = np.zeros((n, k // 8), np.uint32)
        scales = np.zeros((n, k // g), np.uint16)
        assert lib.tl_quantize_linear_weight_int4(w.ctypes.data_as(C.c_void_p), n, k, g, packed.ctypes.data_as(C.c_void_p),
                                                  scales.ctypes.data_as(C.c_void_p)) == 0
        op, os_ = orc.quantize_linear_weight_int4(w, g)
        assert np.array_equal(packed, op) and np.array_equal(scales, os_)
        q = orc.unpack_int4(packed, k)
        assert q.min() >= -7 and q.max() <= 7
    assert lib.tl_quantize_linear_weight_int4(w.ctypes.data_as(C.c_void_p), 1, 12, 4, packed.ctypes.data_as(C.c_void_p),
                                              scales.ctypes.data_as(C.c_void_p)) == B.TL_ERR_INVALID_ARG  # K % 8


def test_int4_oracle_round_trips_every_nibble_in_every_lane():
    from oracle import oracle as orc
    for lane in range(8):
        for q in range(-8, 8):
            word = np.array([[(q & 0xF) << (4 * lane)]], dtype=np.uint32)
            un = orc.unpack_int4(word, 8)
            assert un[0, lane] == q and np.count_nonzero(un) == (1 if q else 0)
            scales = np.array([[int(orc.f32_to_f16_bits(np.float32([3.5]))[0])]], dtype=np.uint16)
            d = orc.dequantize_int4_to_f32(word, scales, 8, 8)
            assert d[0, lane] == np.float32((q / 7.0) * 3.5)
