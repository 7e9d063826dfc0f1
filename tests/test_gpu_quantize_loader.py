"""Device-side quantizeLinearWeight and the quantize-at-load path.

The device quantizer must emit the host quantizer's bits (and therefore the oracle's, which
restates src/backend/quantize.ts:77-131) on ordinary weights, on groups that exercise the f16
subnormal branch, on zero groups and on non-finite values; the loader must quantize exactly the
weights the reference's loader would (examples/qwen3/loader.ts:228-253) and give the same linear
results whether a weight was quantized now or read back from the packed-weight cache."""
import numpy as np
import pytest

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import loader

pytestmark = pytest.mark.gpu


def _quantize_on_device(be, w, group):
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int8-grouped", group, "f16"))
    wt = be.ops.tensorFromArray(w, list(w.shape), "f32")
    q = be.quantizeLinearWeightOnDevice(wt, fmt)
    n, k = w.shape
    view = tb.CudaTensor(be, [n, k // 4], "u32", q.buffer, n * (k // 4) * 4, ownsBuffer=False)
    packed, scales = be.ops.read(view).copy(), be.ops.read(q.scales).copy()
    for t in (q.scales, q, wt):
        t.destroy()
    return packed, scales


@pytest.mark.parametrize("n,k,group", [(96, 384, 64), (96, 384, 128), (33, 256, 32), (17, 512, 512), (5, 64, 4), (256, 4096, 64)])
def test_device_quantizer_bit_exact(backend, n, k, group):
    w, _ = orc.lcg_fill(0x51A7EE ^ n ^ k, n * k, 0.1)
    w = w.reshape(n, k).copy()
    w[1, :group] = 0                      # a zero group: scale 0, all q 0
    w[2, :group] *= 1e-6                  # f16-subnormal abs-max: the converter's half-up branch
    w[3, 1] = 3.0e-8                      # below the smallest f16 subnormal
    if n > 4:
        w[4, 2] = np.nan                  # skipped by the abs-max, packs 0
    if n > 6:
        w[5, 0] = np.inf                  # infinite scale: inv = 0, Inf * 0 = NaN -> 0
        w[6, 3] = -np.inf
    w[0, 0] = 70000.0                     # abs-max beyond the f16 range: scale bits 0x7c00
    packed, scales = _quantize_on_device(backend, w, group)
    op, os_ = orc.quantize_linear_weight(w, group)
    assert np.array_equal(scales, os_)
    assert np.array_equal(packed, op)
    hp, hs = backend.quantizeLinearWeight(w, group)
    assert np.array_equal(packed, hp) and np.array_equal(scales, hs)


def test_device_quantizer_argument_errors(backend):
    be = backend
    w = be.ops.tensorFromArray(np.zeros((2, 130), dtype=np.float32), [2, 130], "f32")
    with pytest.raises(tb.TlError, match="divisible by 4"):
        be.quantizeLinearWeightOnDevice(w, tb.resolveWeightFormat("int8-64"))
    w.destroy()
    w = be.ops.tensorFromArray(np.zeros((2, 96), dtype=np.float32), [2, 96], "f32")
    with pytest.raises(tb.TlError, match="groupSize=64"):
        be.quantizeLinearWeightOnDevice(w, tb.resolveWeightFormat("int8-64"))
    with pytest.raises(tb.TlError):
        be.quantizeLinearWeightOnDevice(w, tb.perChannelFormat(96))  # the reference quantizer has f16 scales only
    w.destroy()


def test_loader_quantizes_what_the_reference_loader_would(backend, tmp_path):
    be = backend
    rng = np.random.default_rng(3)
    tensors = {
        "model.layers.0.self_attn.q_proj.weight": (rng.standard_normal((256, 512)) * 0.05).astype(np.float32),
        "model.layers.0.mlp.down_proj.weight": (rng.standard_normal((128, 192)) * 0.05).astype(np.float32),   # 192 % 128 != 0
        "model.layers.0.input_layernorm.weight": rng.standard_normal(512).astype(np.float32),               # not a projection
        "model.embed_tokens.weight": (rng.standard_normal((64, 512)) * 0.05).astype(np.float16),
    }
    x = (rng.standard_normal((3, 512))).astype(np.float16)
    outs = []
    for attempt in range(2):  # second pass reads the packed-weight cache
        before = be.getKernelLaunchCount()
        loaded = loader.load_weights(be, tensors.items(), "int8-128", cache_dir=str(tmp_path), source="unit")
        launches = be.getKernelLaunchCount() - before
        q = loaded["model.layers.0.self_attn.q_proj.weight"]
        assert q.format is not None and q.format.packing.groupSize == 128 and q.scales is not None and q.shape == [256, 512]
        assert loaded["model.layers.0.mlp.down_proj.weight"].format is None       # K % G != 0: stays plain (loader.ts:236-241)
        assert loaded["model.layers.0.input_layernorm.weight"].format is None
        assert loaded["model.embed_tokens.weight"].dtype == "f16"
        assert launches == (1 if attempt == 0 else 0)                             # quantizer ran once, then the cache served
        xt = be.ops.tensorFromArray(x.view(np.uint16), [3, 512], "f16")
        y = be.linear(xt, q, None, None, "f32")
        outs.append(np.array(be.ops.read(y), dtype=np.float32))
        # against the oracle's quantize -> dequantize -> matmul on the same weight
        op, os_ = orc.quantize_linear_weight(tensors["model.layers.0.self_attn.q_proj.weight"], 128)
        ref = orc.matmul_nt(x.astype(np.float32), orc.dequantize_to_f32(op, os_, 512, 128))
        assert cases.rel_err(outs[-1], ref) <= 1e-3
        for t in list(loaded.values()) + [xt, y]:
            if t.scales is not None:
                t.scales.destroy()
            t.destroy()
    assert np.array_equal(outs[0], outs[1])
    assert loader.cache_key("unit", "a.q_proj.weight", tb.resolveWeightFormat("int8-64")) == "unit#a.q_proj.weight#int8g64"
