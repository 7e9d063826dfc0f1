"""The allocation-free entry point, tl_qgemv_nt_static_scratch, against tl_qgemv_nt.

Some hosts cannot let a library allocate device memory when they call it (a stream
capture is open, or they own all device memory through their own pool).  For them
the library carries one entry point whose scratch is a fixed array inside the
library image.  This file checks, through the C ABI, that it computes what the
ordinary entry point computes -- on two calls in a row, because the fixed array keeps
the previous call's contents and the second call must not see them -- and that it
refuses problems whose scratch would not fit.  It is collected last so that a run
that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

import cases
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
        for _ in range(2):  # two calls in a row on the same inputs
            lib.tl_memset(be._ctx, new_out.buffer, 0xFF, new_out.nbytes)
            got = _call(be, lib.tl_qgemv_nt_static_scratch, x, w, w.scales, new_out, m, n, k, q, epi)
            assert np.isfinite(got).all()
            assert cases.rel_err(got, ref) <= 1e-3
        for t in (ref_out, new_out, bias, x, w.scales, w):
            t.destroy()
    assert be.getKernelLaunchCount() > launches0
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
