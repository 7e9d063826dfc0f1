"""GPU tests of the persistent chain (tl_qgemv_chain_*): a sequence of dependent small-batch
quantized products in one cooperative launch, against the same products issued one by one
through tl_qgemv_nt and against the CPU oracle.

The chain uses the ring kernel's tile arithmetic with 8 warps, so against ring launches
forced to that shape the outputs must agree bit for bit; against the oracle the usual
tolerances apply (f32 outputs 1e-3, 16-bit outputs 1e-2; |x-ref| / max(1,|ref|))."""
import numpy as np
import pytest

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B
from torchlette_b200.decode_stack import TINY, DecodeStack

pytestmark = pytest.mark.gpu

RING_8x6 = (1, 4, 8, 6, 0, 0)
RING_8x4 = (1, 4, 8, 4, 0, 0)


def _to_f32(arr, dtype):
    if dtype == "bf16":
        return orc.bf16_bits_to_f32(arr)
    return np.asarray(arr, dtype=np.float32)


def _three_phase_problem(be, m, act_dtype, seed, k0=320):
    """phase 0: x[m,320] -> y0a[m,128] (silu) and y0b[m,60]; phase 1: y0a -> y1[m,192];
    phase 2: y1 -> y2[m,77] f32 with bias + gelu.  K = 320 gives the four warps unequal shares
    of k blocks, N = 60 and 77 end in partial tiles."""
    rng = np.random.Generator(np.random.PCG64(seed))
    dims = {"k0": k0, "n0a": 128, "n0b": 60, "n1": 192, "n2": 77}

    def weight(n, k):
        q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        s = rng.uniform(0.001, 0.01, size=(n, 1)).astype(np.float32)
        return q, s, be.createQuantizedWeight(cases.pack_int8(q), s, n, k, tb.perChannelFormat(k))

    cs = cases.per_channel_case(4, k0, m, seed=seed, act_dtype=act_dtype)
    w0a, w0b = weight(dims["n0a"], k0), weight(dims["n0b"], k0)
    w1 = weight(dims["n1"], dims["n0a"])
    w2 = weight(dims["n2"], dims["n1"])
    bias2 = (rng.standard_normal(dims["n2"]) * 0.02).astype(np.float32)
    return dims, cs, (w0a, w0b, w1, w2), bias2


def _run_both(be, m, act_dtype, seed):
    dims, cs, (w0a, w0b, w1, w2), bias2 = _three_phase_problem(be, m, act_dtype, seed)
    k0 = dims["k0"]
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k0], act_dtype)
    bt = be.ops.tensorFromArray(bias2, [dims["n2"]], "f32")
    alpha0 = 1.0 / (0.43 * np.sqrt(k0))      # keeps the chained activations O(1)
    alpha1 = 1.0 / (0.43 * np.sqrt(dims["n0a"]))
    alpha2 = 1.0 / (0.43 * np.sqrt(dims["n1"]))
    silu = tb.EpilogueConfig([{"kind": "unary", "op": "silu"}], 0)
    bias_gelu = tb.EpilogueConfig([{"kind": "bias", "inputIndex": 0}, {"kind": "unary", "op": "gelu"}], 1)

    def outputs():
        return (be.ops.empty([m, dims["n0a"]], act_dtype), be.ops.empty([m, dims["n0b"]], act_dtype),
                be.ops.empty([m, dims["n1"]], act_dtype), be.ops.empty([m, dims["n2"]], "f32"))

    # -- one launch per product, forced to the ring kernel with 8 warps --
    ya, yb, y1, y2 = outputs()
    be.forceVariant(RING_8x6 if m <= 8 else RING_8x4)
    try:
        for (w, a, o, n, k, al, ep, ei, od) in (
                (w0a, x, ya, dims["n0a"], k0, alpha0, silu, (), act_dtype),
                (w0b, x, yb, dims["n0b"], k0, alpha0, None, (), act_dtype),
                (w1, ya, y1, dims["n1"], dims["n0a"], alpha1, None, (), act_dtype),
                (w2, y1, y2, dims["n2"], dims["n1"], alpha2, bias_gelu, (bt,), "f32")):
            be.dispatchQuantizedGemvNT(a, w[2], w[2].scales, o, n, k, k, od, al, m=m, epilogue=ep, epilogueInputs=ei,
                                       packing=tb.perChannelFormat(k).packing)
    finally:
        be.forceVariant(None)
    single = [be.ops.read(t).copy() for t in (ya, yb, y1, y2)]

    # -- the same three phases as one chain --
    ca, cb, c1, c2 = outputs()
    phases = [
        {"a": x, "k": k0, "groupSize": k0, "outputDtype": act_dtype, "items": [
            {"packed": w0a[2], "scales": w0a[2].scales, "out": ca, "n": dims["n0a"], "alpha": alpha0, "epilogue": silu},
            {"packed": w0b[2], "scales": w0b[2].scales, "out": cb, "n": dims["n0b"], "alpha": alpha0}]},
        {"a": ca, "k": dims["n0a"], "groupSize": dims["n0a"], "outputDtype": act_dtype, "items": [
            {"packed": w1[2], "scales": w1[2].scales, "out": c1, "n": dims["n1"], "alpha": alpha1}]},
        {"a": c1, "k": dims["n1"], "groupSize": dims["n1"], "outputDtype": "f32", "items": [
            {"packed": w2[2], "scales": w2[2].scales, "out": c2, "n": dims["n2"], "alpha": alpha2,
             "epilogue": bias_gelu, "epilogueInputs": (bt,)}]},
    ]
    launches0, gemvs0 = be.getKernelLaunchCount(), be.getQuantGemvDispatchCount()
    chain = be.createQuantizedGemvChain(phases, m)
    chained = []
    for _ in range(3):  # repeated launches: the phase counters are cleared every time
        be.runQuantizedGemvChain(chain)
        chained.append([be.ops.read(t).copy() for t in (ca, cb, c1, c2)])
    be.sync()
    assert be.getKernelLaunchCount() == launches0 + 3 and be.getQuantGemvDispatchCount() == gemvs0 + 12
    be.destroyQuantizedGemvChain(chain)

    for t in (x, bt, ya, yb, y1, y2, ca, cb, c1, c2, w0a[2].scales, w0a[2], w0b[2].scales, w0b[2], w1[2].scales, w1[2],
              w2[2].scales, w2[2]):
        t.destroy()
    return single, chained, dims


@pytest.mark.parametrize("m,act_dtype", [(1, "f16"), (3, "f16"), (8, "bf16"), (16, "f16"), (11, "bf16")])
def test_chain_equals_single_launches_bit_for_bit(backend, m, act_dtype):
    single, chained, _ = _run_both(backend, m, act_dtype, seed=100 + m)
    for rep in chained:
        for got, want in zip(rep, single):
            assert np.array_equal(np.asarray(got).view(np.uint8), np.asarray(want).view(np.uint8))
    assert backend.getGpuUncapturedErrorCount() == 0


@pytest.mark.parametrize("group", [64, 128])
def test_single_phase_chain_against_the_oracle_grouped_scales(backend, group):
    """The reference's native format (f16 scales per group of 64/128, w = q/127*s) through a chain."""
    be = backend
    m, n, k = 5, 300, 512
    rng = np.random.Generator(np.random.PCG64(7 + group))
    wf = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    packed, scales = be.quantizeLinearWeight(wf, group)
    fmt = tb.StorageFormat("f16", tb.QuantPacking("int8-grouped", group, "f16"))
    w = be.createQuantizedWeight(packed, scales, n, k, fmt)
    cs = cases.per_channel_case(4, k, m, seed=group, act_dtype="f16")
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "f16")
    y = be.ops.empty([m, n], "f32")
    chain = be.createQuantizedGemvChain(
        [{"a": x, "k": k, "groupSize": group, "outputDtype": "f32",
          "items": [{"packed": w, "scales": w.scales, "out": y, "n": n}]}], m, scaleConvention="snorm127")
    be.runQuantizedGemvChain(chain)
    got = be.ops.read(y).reshape(m, n)
    be.destroyQuantizedGemvChain(chain)
    wref = orc.dequantize_to_f32(packed, scales, k, group)
    ref = orc.matmul_nt(cs["x"], wref)
    assert cases.rel_err(got, ref) <= 1e-3
    for t in (x, y, w.scales, w):
        t.destroy()


def test_decode_stack_chain_matches_the_graph_of_single_launches(backend):
    """The whole tiny decode stack: one persistent launch against the replayed graph of
    per-projection launches (different warp counts per tile, so equality is up to f16 rounding)."""
    be = backend
    plain = DecodeStack(be, TINY, seed=5)
    chained = DecodeStack(be, TINY, seed=5, chain=True)
    import torch

    x = torch.randn(TINY.batch, TINY.hidden, device=plain.dev).to(plain.tdt)
    plain.x.copy_(x)
    chained.x.copy_(x)
    torch.cuda.synchronize()
    plain.capture()
    plain.step()
    be.sync()
    assert chained.uses_chain() and chained.launches_per_step() == 1
    chained.capture()
    for _ in range(2):
        chained.step()
    be.sync()
    a = plain.logits_local.float().cpu().numpy()
    b = chained.logits_local.float().cpu().numpy()
    assert np.isfinite(b).all() and np.abs(b).max() > 0
    assert cases.rel_err(b, a) <= 1e-2
    plain.destroy()
    chained.destroy()
    assert be.getGpuUncapturedErrorCount() == 0


def test_chain_rejects_what_it_cannot_run(backend):
    be = backend
    k, n, m = 96, 32, 2   # K % 64 != 0
    cs = cases.per_channel_case(n, k, m, seed=1, act_dtype="f16")
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "f16")
    y = be.ops.empty([m, n], "f16")
    phase = {"a": x, "k": k, "groupSize": k, "outputDtype": "f16",
             "items": [{"packed": w, "scales": w.scales, "out": y, "n": n}]}
    with pytest.raises(tb.TlError):
        be.createQuantizedGemvChain([phase], m)
    with pytest.raises(tb.TlError):
        be.createQuantizedGemvChain([dict(phase, k=128, groupSize=128)], 17)  # m outside the GEMV range
    for t in (x, y, w.scales, w):
        t.destroy()
