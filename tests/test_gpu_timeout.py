"""A bounded device-side wait that runs out: error status, no fault, context still usable.

One process, one GPU.  tl_p2p_attach_loopback maps the rank's own exchange buffer in place of
the peer of a two-rank group, so the flag of "rank 1" is never raised; with the wait limit set
to 1024 polls the peer all-reduce kernel gives up by itself, tl_sync reports TL_ERR_TIMEOUT,
tl_p2p_reset clears the exchange, and an ordinary quantized matmul on the same context is
still correct.  Nothing here touches memory outside the context's own buffers."""
import ctypes as C

import pytest
import torch

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B

pytestmark = pytest.mark.gpu


def _qgemv_ok(be):
    n, k, m = 272, 512, 4
    cs = cases.per_channel_case(n, k, m, seed=5, act_dtype="f16", bias=True)
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "f16")
    b = be.ops.tensorFromArray(cs["bias"], [n], "f32")
    y = be.linear(x, w, b, "silu", "f32")
    got = be.ops.read(y)
    ref = orc.linear_reference(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k), cs["bias"], "silu")
    for t in (y, x, b, w.scales, w):
        t.destroy()
    return cases.rel_err(got, ref)


def test_peer_wait_runs_out_and_the_context_survives():
    be = tb.CudaBackend(0)
    lib, ctx = be._lib, be._ctx
    try:
        assert be.getOption("wait_limit_polls") == 1 << 26
        with pytest.raises(tb.TlError):
            be.setOption("no_such_option", 1)
        be.setOption("wait_limit_polls", 1024)
        handle = (C.c_char * 64)()
        B.check(ctx, lib.tl_p2p_create(ctx, 1 << 16, handle))
        B.check(ctx, lib.tl_p2p_attach_loopback(ctx, 2))
        dev = torch.device("cuda", 0)
        src = torch.randn(8 * 1024, device=dev).to(torch.float16)
        dst = torch.full_like(src, 7.0)
        torch.cuda.synchronize(dev)
        errors0 = be.getGpuUncapturedErrorCount()
        # enqueue succeeds; the kernel waits 1024 polls for "rank 1", records the time-out and returns
        B.check(ctx, lib.tl_allreduce_sum_p2p(ctx, src.data_ptr(), dst.data_ptr(), src.numel(), B.TL_F16))
        rc = lib.tl_sync(ctx)
        assert rc == B.TL_ERR_TIMEOUT, rc
        assert b"bounded wait" in lib.tl_last_error(ctx)
        assert be.getGpuUncapturedErrorCount() == errors0 + 1
        # a rank that timed out wrote nothing to dst
        torch.cuda.synchronize(dev)
        assert bool((dst == 7.0).all())
        # the status word is cleared by tl_sync: a second sync is clean
        assert lib.tl_sync(ctx) == B.TL_OK
        # after the reset the context computes as before
        B.check(ctx, lib.tl_p2p_reset(ctx))
        assert lib.tl_sync(ctx) == B.TL_OK
        assert _qgemv_ok(be) <= 1e-3
        assert lib.tl_sync(ctx) == B.TL_OK
    finally:
        be.destroy()


def test_loopback_needs_an_exchange_buffer_and_a_sane_world():
    be = tb.CudaBackend(0)
    lib, ctx = be._lib, be._ctx
    try:
        assert lib.tl_p2p_attach_loopback(ctx, 2) == B.TL_ERR_INVALID_ARG  # no tl_p2p_create yet
        assert lib.tl_p2p_reset(ctx) == B.TL_ERR_INVALID_ARG
        handle = (C.c_char * 64)()
        B.check(ctx, lib.tl_p2p_create(ctx, 4096, handle))
        assert lib.tl_p2p_attach_loopback(ctx, 0) == B.TL_ERR_INVALID_ARG
        assert lib.tl_p2p_attach_loopback(ctx, 9) == B.TL_ERR_INVALID_ARG
        assert lib.tl_sync(ctx) == B.TL_OK
    finally:
        be.destroy()


def test_push_and_reduce_on_read_on_one_gpu():
    """tl_qgemv_nt_push followed by its consumer on a loopback group of one rank: the whole push /
    reduce-on-read path (epoch-tagged words, the summing CTAs, the grid-wide gate) on local memory.
    The sum has one term, so the consumer must see exactly the f16-rounded product, and a consumer
    that does not read the pushed buffer is refused."""
    import numpy as np

    be = tb.CudaBackend(0)
    lib, ctx = be._lib, be._ctx
    try:
        m, n1, k1, n2 = 8, 512, 256, 320
        handle = (C.c_char * 64)()
        B.check(ctx, lib.tl_p2p_create(ctx, m * n1 * 8, handle))
        B.check(ctx, lib.tl_p2p_attach_loopback(ctx, 1))
        c1 = cases.per_channel_case(n1, k1, m, seed=41, act_dtype="f16")
        c2 = cases.per_channel_case(n2, n1, m, seed=42, act_dtype="f16")
        w1 = be.createQuantizedWeight(c1["packed"], c1["scales"], n1, k1, tb.perChannelFormat(k1))
        w2 = be.createQuantizedWeight(c2["packed"], c2["scales"], n2, n1, tb.perChannelFormat(n1))
        x = be.ops.tensorFromArray(c1["x_bits"], [m, k1], "f16")
        h = be.ops.empty([m, n1], "f16")
        y = be.ops.empty([m, n2], "f32")
        other = be.ops.empty([m, n1], "f16")
        q1, q2 = be._qdesc(w1.format.packing), be._qdesc(w2.format.packing)
        alpha = 0.01
        for rep in range(3):  # successive pushes alternate the halves of the exchange buffer
            B.check(ctx, lib.tl_qgemv_nt_push(ctx, x.buffer, B.TL_F16, w1.buffer, w1.scales.buffer, h.buffer, B.TL_F16,
                                              m, n1, k1, C.byref(q1), alpha))
            # a launch that does not read `h` must be refused while the push is pending, and launch nothing
            rc = lib.tl_qgemv_nt(ctx, other.buffer, B.TL_F16, w2.buffer, w2.scales.buffer, y.buffer, B.TL_F32, m, n2, n1,
                                 C.byref(q2), 1.0, None)
            assert rc == B.TL_ERR_INVALID_ARG and b"pending" in lib.tl_last_error(ctx)
            B.check(ctx, lib.tl_qgemv_nt(ctx, h.buffer, B.TL_F16, w2.buffer, w2.scales.buffer, y.buffer, B.TL_F32, m, n2, n1,
                                         C.byref(q2), 1.0, None))
            be.sync()
            ref_h = orc.linear_reference(c1["x"], orc.dequantize_direct_f32(c1["packed"], c1["scales"], k1, k1), None, None, alpha=alpha)
            got_h = np.asarray(be.ops.read(h), dtype=np.float32)
            assert cases.rel_err(got_h, ref_h) <= 1e-2
            ref_y = orc.linear_reference(got_h, orc.dequantize_direct_f32(c2["packed"], c2["scales"], n1, n1), None, None)
            assert cases.rel_err(be.ops.read(y), ref_y) <= 1e-3
        # the stand-alone reduction
        B.check(ctx, lib.tl_qgemv_nt_push(ctx, x.buffer, B.TL_F16, w1.buffer, w1.scales.buffer, h.buffer, B.TL_F16,
                                          m, n1, k1, C.byref(q1), alpha))
        B.check(ctx, lib.tl_reduce_pending(ctx))
        be.sync()
        assert cases.rel_err(np.asarray(be.ops.read(h), dtype=np.float32), ref_h) <= 1e-2
        assert be.getGpuUncapturedErrorCount() == 0
        for t in (other, y, h, x, w2.scales, w2, w1.scales, w1):
            t.destroy()
    finally:
        be.destroy()
