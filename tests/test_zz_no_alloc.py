"""The allocation-free entry point, tl_qgemv_nt_static_scratch, against tl_qgemv_nt.

Some hosts cannot let a library allocate device memory when they call it: a serving
process that has handed all device memory to its own pool (a cudaMalloc from a
library can only fail there), or a latency-critical loop in which the device-wide
synchronisation hidden in cudaMalloc/cudaFree would stall every other stream.  For
them the library carries one entry point whose scratch is a fixed array inside the
library image.  This file checks, through the C ABI, that it computes what the
ordinary entry point computes and what the CPU oracle computes -- on two calls in a
row, because the fixed array keeps the previous call's contents and the second call
must not see them -- and that it refuses problems whose scratch would not fit.  It is collected last so that a run
that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B

pytestmark = pytest.mark.gpu


def _call(be, fn, x, w, s, out, m, n, k, q, epi):
    B.check(be._ctx, fn(be._ctx, x.buffer, B.TL_F16, w.buffer, s.buffer, out.buffer, B.TL_F32, m, n, k, C.byref(q), 1.0,
                        C.byref(epi) if epi is not None else None))
    return be.ops.read(out).copy()


def test_static_scratch_entry_point_matches_tl_qgemv_nt_twice(backend):
    be = backend
    lib = be._lib
    launches0 = be.getKernelLaunchCount()
    # two different problems back to back: the second reuses (and must clear) what the first left
    for (m, n, k, seed) in [(8, 2000, 1024, 1), (3, 4096, 512, 2)]:
        cs = cases.per_channel_case(n, k, m, seed=seed, act_dtype="f16", bias=True)
        w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
        x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "f16")
        bias = be.ops.tensorFromArray(cs["bias"], [n], "f32")
        q = be._qdesc(w.format.packing)
        epi = B.Epilogue()
        epi.n_ops, epi.n_inputs = 2, 1
        epi.ops[0] = B.EpilogueOp(B.TL_EPI_BIAS, 0, 0, 0)
        epi.ops[1] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY["silu"], 0, 0)
        epi.inputs[0] = bias.buffer
        ref_out = be.ops.empty([m, n], "f32")
        new_out = be.ops.empty([m, n], "f32")
        ref = _call(be, lib.tl_qgemv_nt, x, w, w.scales, ref_out, m, n, k, q, epi)
        oracle = orc.linear_reference(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k), cs["bias"], "silu")
        assert cases.rel_err(ref, oracle) <= 1e-3
        for _ in range(2):  # two calls in a row on the same inputs
            lib.tl_memset(be._ctx, new_out.buffer, 0xFF, new_out.nbytes)
            got = _call(be, lib.tl_qgemv_nt_static_scratch, x, w, w.scales, new_out, m, n, k, q, epi)
            assert np.isfinite(got).all()
            assert cases.rel_err(got, ref) <= 1e-3
            assert cases.rel_err(got, oracle) <= 1e-3
        for t in (ref_out, new_out, bias, x, w.scales, w):
            t.destroy()
    assert be.getKernelLaunchCount() > launches0
    assert be.getGpuUncapturedErrorCount() == 0


def test_static_scratch_entry_point_other_formats_against_the_oracle(backend):
    """Grouped f16 scales (the reference's own format), two token tiles (m = 16), bf16 activations
    and a long k with few rows (several CTAs meet in one band of the array)."""
    be = backend
    lib = be._lib
    # reference-native format: G = 64, f16 abs-max scales, w = (q/127) * s
    n, k, m, group = 300, 8192, 16, 64
    wf, st = orc.lcg_fill(0x51A7EE ^ n, n * k, 0.1)
    packed, scales = be.quantizeLinearWeight(wf.reshape(n, k), group)
    wt = be.createQuantizedWeight(packed, scales, n, k, tb.resolveWeightFormat("int8-64"))
    xs, st = orc.lcg_fill(st, m * k)
    x16 = xs.reshape(m, k).astype(np.float16)
    x = be.ops.tensorFromArray(x16.view(np.uint16), [m, k], "f16")
    out = be.ops.empty([m, n], "f32")
    q = be._qdesc(wt.format.packing)
    oracle = orc.matmul_nt(x16.astype(np.float32), orc.dequantize_to_f32(packed, scales, k, group))
    for _ in range(2):
        lib.tl_memset(be._ctx, out.buffer, 0xFF, out.nbytes)
        B.check(be._ctx, lib.tl_qgemv_nt_static_scratch(be._ctx, x.buffer, B.TL_F16, wt.buffer, wt.scales.buffer, out.buffer,
                                                        B.TL_F32, m, n, k, C.byref(q), 1.0, None))
        assert cases.rel_err(be.ops.read(out), oracle) <= 1e-3
    for t in (out, x, wt.scales, wt):
        t.destroy()
    # bf16 activations, per-channel scales
    n, k, m = 1000, 1024, 5
    cs = cases.per_channel_case(n, k, m, seed=31, act_dtype="bf16")
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "bf16")
    out = be.ops.empty([m, n], "f32")
    q = be._qdesc(w.format.packing)
    oracle = orc.linear_reference(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k), None, None)
    for _ in range(2):
        B.check(be._ctx, lib.tl_qgemv_nt_static_scratch(be._ctx, x.buffer, B.TL_BF16, w.buffer, w.scales.buffer, out.buffer,
                                                        B.TL_F32, m, n, k, C.byref(q), 1.0, None))
        assert cases.rel_err(be.ops.read(out), oracle) <= 1e-3
    for t in (out, x, w.scales, w):
        t.destroy()
    assert be.getGpuUncapturedErrorCount() == 0


def test_static_scratch_entry_point_rejects_what_does_not_fit(backend):
    be = backend
    lib = be._lib
    buf = be._alloc(4096)
    q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, 128, B.TL_F32, B.TL_SCALE_DIRECT)
    launches = be.getKernelLaunchCount()
    # 16 x 151936 f32 partial sums = 9.7 MB > the 4 MiB array
    rc = lib.tl_qgemv_nt_static_scratch(be._ctx, buf, B.TL_F16, buf, buf, buf, B.TL_F32, 16, 151936, 128, C.byref(q), 1.0, None)
    assert rc == B.TL_ERR_UNSUPPORTED and b"bytes of scratch" in lib.tl_last_error(be._ctx)
    rc = lib.tl_qgemv_nt_static_scratch(be._ctx, buf, B.TL_F32, buf, buf, buf, B.TL_F32, 1, 64, 128, C.byref(q), 1.0, None)
    assert rc == B.TL_ERR_UNSUPPORTED and b"f16/bf16" in lib.tl_last_error(be._ctx)
    rc = lib.tl_qgemv_nt_static_scratch(be._ctx, buf, B.TL_F16, buf, buf, buf, B.TL_F32, 17, 64, 128, C.byref(q), 1.0, None)
    assert rc == B.TL_ERR_INVALID_ARG
    assert be.getKernelLaunchCount() == launches
    be._free(buf)
