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
        assert lib.tl_p2p_attach_loopback(ctx, 1) == B.TL_ERR_INVALID_ARG
        assert lib.tl_p2p_attach_loopback(ctx, 9) == B.TL_ERR_INVALID_ARG
        assert lib.tl_sync(ctx) == B.TL_OK
    finally:
        be.destroy()
