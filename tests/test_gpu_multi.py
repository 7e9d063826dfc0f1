"""Two-GPU tests of the collectives (skipped on a single-GPU box): the one-shot
peer-memory all-reduce against a locally computed sum, eager and replayed from a
captured graph, and bit-identical across ranks; the row-parallel GEMV fused with its
all-reduce against the unfused pair (bit for bit); NCCL all-gather / all-reduce wrappers.
Ranks are child processes (one per GPU); rendezvous over gloo on 127.0.0.1."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _data(rank, call, count, dtype):
    rng = np.random.default_rng(1000 * call + rank)
    x = rng.standard_normal(count).astype(np.float32)
    if dtype == "f16":
        return x.astype(np.float16)
    return x


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from torchlette_b200 import backend as tb
    from torchlette_b200 import binding as B

    try:
        torch.cuda.set_device(rank)
        B.preload_nccl()
        be = tb.CudaBackend(rank)
        lib, ctx = be._lib, be._ctx
        ident = [None]
        if rank == 0:
            buf = (C.c_char * B.TL_COMM_ID_BYTES)()
            B.check(None, lib.tl_comm_unique_id(buf))
            ident[0] = bytes(buf)
        dist.broadcast_object_list(ident, src=0)
        B.check(ctx, lib.tl_comm_init(ctx, rank, world, (C.c_char * B.TL_COMM_ID_BYTES).from_buffer_copy(ident[0])))
        hbuf = (C.c_char * 64)()
        B.check(ctx, lib.tl_p2p_create(ctx, 1 << 17, hbuf))
        handles = [None] * world
        dist.all_gather_object(handles, bytes(hbuf))
        B.check(ctx, lib.tl_p2p_attach(ctx, (C.c_char * (64 * world)).from_buffer_copy(b"".join(handles))))
        dist.barrier()
        results = {}
        call = 0
        for dtype, count in [("f16", 8 * 4096), ("f32", 1001), ("f16", 4096), ("f32", 8 * 4096)]:
            npdt = np.float16 if dtype == "f16" else np.float32
            t = be.ops.empty([count], dtype)
            for _ in range(4):  # back-to-back calls alternate the staging halves
                mine = _data(rank, call, count, dtype)
                be._upload(t.buffer, mine)
                B.check(ctx, lib.tl_allreduce_sum_p2p(ctx, t.buffer, t.buffer, count, B.DTYPE_ID[dtype]))
                got = be.ops.read(t)
                expect = sum(_data(r, call, count, dtype).astype(np.float32) for r in range(world))
                tol = 2e-3 if dtype == "f16" else 1e-6
                assert np.allclose(got.astype(np.float32), expect, rtol=tol, atol=tol), (dtype, count, call)
                results[call] = got.astype(npdt).tobytes()
                call += 1
            # NCCL wrapper on the same data
            be._upload(t.buffer, _data(rank, call, count, dtype))
            B.check(ctx, lib.tl_allreduce_sum(ctx, t.buffer, count, B.DTYPE_ID[dtype]))
            expect = sum(_data(r, call, count, dtype).astype(np.float32) for r in range(world))
            assert np.allclose(be.ops.read(t).astype(np.float32), expect, rtol=2e-3, atol=2e-3)
            call += 1
            t.destroy()
        # f32 partial sums, 16-bit result: the sum is rounded once (ragged count: scalar tail)
        for dst_dtype, count in [("f16", 8 * 4096), ("bf16", 1003)]:
            src = be.ops.empty([count], "f32")
            dst = be.ops.empty([count], dst_dtype)
            for _ in range(3):
                be._upload(src.buffer, _data(rank, call, count, "f32"))
                B.check(ctx, lib.tl_allreduce_sum_p2p_f32_to(ctx, src.buffer, dst.buffer, B.DTYPE_ID[dst_dtype], count))
                total = np.zeros(count, np.float32)
                for r in range(world):  # rank order, f32, like the kernel
                    total = total + _data(r, call, count, "f32")
                got = be.ops.read(dst)
                if dst_dtype == "f16":
                    assert np.array_equal(got.view(np.uint16), total.astype(np.float16).view(np.uint16)), (dst_dtype, call)
                else:
                    from oracle import oracle as orc
                    assert np.array_equal(got.reshape(-1), orc.bf16_bits_rne(total)), (dst_dtype, call)
                results[call] = np.ascontiguousarray(got).tobytes()
                call += 1
            src.destroy()
            dst.destroy()
        # replay: two all-reduces captured once, replayed three times with fresh inputs
        count = 4096
        a, b = be.ops.empty([count], "f32"), be.ops.empty([count], "f32")
        B.check(ctx, lib.tl_allreduce_sum_p2p(ctx, a.buffer, a.buffer, count, B.TL_F32))  # an odd call first
        be.beginCapture()
        B.check(ctx, lib.tl_allreduce_sum_p2p(ctx, a.buffer, a.buffer, count, B.TL_F32))
        B.check(ctx, lib.tl_allreduce_sum_p2p(ctx, b.buffer, b.buffer, count, B.TL_F32))
        g = be.endCapture()
        for rep in range(3):
            be._upload(a.buffer, _data(rank, 500 + rep, count, "f32"))
            be._upload(b.buffer, _data(rank, 600 + rep, count, "f32"))
            be.replay(g)
            ea = sum(_data(r, 500 + rep, count, "f32") for r in range(world))
            eb = sum(_data(r, 600 + rep, count, "f32") for r in range(world))
            assert np.allclose(be.ops.read(a), ea, atol=1e-6) and np.allclose(be.ops.read(b), eb, atol=1e-6)
        be.destroyGraph(g)
        # fused row-parallel GEMV + all-reduce: same bits as tl_qgemv_nt followed by the peer all-reduce
        m, n, kfull = 5, 300, 256 * world
        rng = np.random.default_rng(77)
        qw = rng.integers(-127, 128, size=(n, kfull), dtype=np.int8)
        sc = rng.uniform(0.001, 0.01, size=(n, 1)).astype(np.float32)
        kr = kfull // world
        wq = np.ascontiguousarray(qw[:, rank * kr:(rank + 1) * kr])
        fmt = tb.perChannelFormat(kr)
        wt = be.createQuantizedWeight(wq.view(np.uint32).reshape(n, kr // 4), sc, n, kr, fmt)
        qd = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, kr, B.TL_F32, B.TL_SCALE_DIRECT)
        y_unfused, y_fused = be.ops.empty([m, n], "f16"), be.ops.empty([m, n], "f16")
        xt = be.ops.empty([m, kr], "f16")
        alpha = 0.37

        def fused_inputs(rep):
            xf = np.random.default_rng(900 + rep).standard_normal((m, kfull)).astype(np.float16)
            be._upload(xt.buffer, np.ascontiguousarray(xf[:, rank * kr:(rank + 1) * kr]))
            return xf

        def run_unfused():
            be.forceVariant((1, 4, 16, 4, 0, 0))  # the fused kernel's tile shape: same summation order
            try:
                B.check(ctx, lib.tl_qgemv_nt(ctx, xt.buffer, B.TL_F16, wt.buffer, wt.scales.buffer, y_unfused.buffer, B.TL_F16,
                                             m, n, kr, C.byref(qd), alpha, None))
            finally:
                be.forceVariant(None)
            B.check(ctx, lib.tl_allreduce_sum_p2p(ctx, y_unfused.buffer, y_unfused.buffer, m * n, B.TL_F16))

        def run_fused():
            B.check(ctx, lib.tl_qgemv_nt_allreduce(ctx, xt.buffer, B.TL_F16, wt.buffer, wt.scales.buffer, y_fused.buffer,
                                                   B.TL_F16, m, n, kr, C.byref(qd), alpha))

        for rep in range(3):  # successive calls alternate the halves of the exchange buffer
            xf = fused_inputs(rep)
            run_unfused()
            run_fused()
            got_u, got_f = be.ops.read(y_unfused).copy(), be.ops.read(y_fused).copy()
            assert np.array_equal(got_u.view(np.uint16), got_f.view(np.uint16)), rep
            ref = alpha * (xf.astype(np.float32) @ (qw.astype(np.float32) * sc).T)
            assert np.allclose(got_f.astype(np.float32).reshape(m, n), ref, rtol=2e-2, atol=2e-2), rep
            results[1000 + rep] = got_f.tobytes()
        be.beginCapture()
        run_fused()
        gf = be.endCapture()
        for rep in range(3, 6):
            xf = fused_inputs(rep)
            be.replay(gf)
            ref = alpha * (xf.astype(np.float32) @ (qw.astype(np.float32) * sc).T)
            got_f = be.ops.read(y_fused).copy()
            assert np.allclose(got_f.astype(np.float32).reshape(m, n), ref, rtol=2e-2, atol=2e-2), rep
            results[1000 + rep] = got_f.tobytes()
        be.destroyGraph(gf)
        # column gather
        m, nl = 3, 40
        loc = be.ops.tensorFromArray(np.full((m, nl), rank + 1, np.float32), [m, nl], "f32")
        full = be.ops.empty([m, nl * world], "f32")
        B.check(ctx, lib.tl_allgather_cols(ctx, loc.buffer, full.buffer, m, nl, B.TL_F32))
        got = be.ops.read(full)
        for r in range(world):
            assert (got[:, r * nl:(r + 1) * nl] == r + 1).all()
        be.sync()
        allres = [None] * world
        dist.all_gather_object(allres, results)
        if rank == 0:
            same = all(allres[0][k] == allres[r][k] for r in range(world) for k in allres[0])
            q.put(("ok", same, be.getGpuUncapturedErrorCount()))
        dist.barrier()
        lib.tl_comm_destroy(ctx)
        be.destroy()
    except Exception as e:  # surfaced to the parent instead of a silent hang
        if rank == 0:
            q.put(("error", repr(e), -1))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_p2p_allreduce_and_nccl_wrappers_two_gpus():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    status, same, errs = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
    assert status == "ok", same
    assert same is True, "ranks disagree bit-wise on an all-reduce result"
    assert errs == 0
    assert all(p.exitcode == 0 for p in procs)


# ---------------------------------------------------------------------------
# The tensor-parallel decode stack against the oracle and against the single-GPU stack
# ---------------------------------------------------------------------------

def _stack_rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc
    from torchlette_b200 import backend as tb
    from torchlette_b200 import binding as B
    from torchlette_b200.decode_stack import TINY, DecodeStack

    def f16(x):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)

    try:
        torch.cuda.set_device(rank)
        B.preload_nccl()
        be = tb.CudaBackend(rank)
        lib, ctx = be._lib, be._ctx
        ident = [None]
        if rank == 0:
            buf = (C.c_char * B.TL_COMM_ID_BYTES)()
            B.check(None, lib.tl_comm_unique_id(buf))
            ident[0] = bytes(buf)
        dist.broadcast_object_list(ident, src=0)
        B.check(ctx, lib.tl_comm_init(ctx, rank, world, (C.c_char * B.TL_COMM_ID_BYTES).from_buffer_copy(ident[0])))
        hbuf = (C.c_char * 64)()
        B.check(ctx, lib.tl_p2p_create(ctx, TINY.batch * TINY.hidden * 8, hbuf))
        handles = [None] * world
        dist.all_gather_object(handles, bytes(hbuf))
        B.check(ctx, lib.tl_p2p_attach(ctx, (C.c_char * (64 * world)).from_buffer_copy(b"".join(handles))))
        dist.barrier()
        dev = torch.device("cuda", rank)
        gen = torch.Generator(device=dev)
        gen.manual_seed(11)
        x = torch.randn(TINY.batch, TINY.hidden, device=dev, generator=gen).to(torch.float16)
        # the oracle and the single-GPU stack: the SAME model (same seed), whole on this GPU
        single = DecodeStack(be, TINY, 0, 1, seed=3)
        single.x.copy_(x)
        torch.cuda.synchronize(dev)
        single.enqueue_step()
        be.sync()
        h = x.float().cpu().numpy()
        for pq, pk, pv, po, pg, pu, pd in single.layers:
            def proj(a, p):
                w = p.w.cpu().numpy().astype(np.float32) * p.s.cpu().numpy().astype(np.float32)[:, None]
                return orc.linear_reference(a, w, None, p.act, alpha=p.alpha)
            h = f16(proj(f16(proj(f16(proj(f16(proj(h, pq)), po)), pg)), pd))
        w = single.lm_head.w.cpu().numpy().astype(np.float32) * single.lm_head.s.cpu().numpy().astype(np.float32)[:, None]
        ref = orc.linear_reference(h, w, None, None, alpha=single.lm_head.alpha)
        one_gpu = single.logits.float().cpu().numpy()
        rel = lambda a, b: float(np.max(np.abs(a - b) / np.maximum(1.0, np.abs(b))))  # noqa: E731
        assert rel(one_gpu, ref) <= 2e-2
        report = {}
        for tp_mode in ("chained", "gather"):
            for allreduce in ("p2p", "fused", "push", "nccl"):
                st = DecodeStack(be, TINY, rank, world, tp_mode, seed=3, allreduce=allreduce)
                st.x.copy_(x)
                torch.cuda.synchronize(dev)
                dist.barrier()
                st.capture()          # an eager step, then the captured one
                for _ in range(2):    # replays
                    st.step()
                be.sync()
                got = st.logits.float().cpu().numpy()
                assert got.shape == ref.shape
                assert rel(got, ref) <= 2e-2, (tp_mode, allreduce, rel(got, ref))
                assert rel(got, one_gpu) <= 2e-2, (tp_mode, allreduce)
                report[(tp_mode, allreduce)] = (st.logits.cpu().numpy().tobytes(), st.h2.cpu().numpy().tobytes())
                dist.barrier()
                st.destroy()
        single.destroy()
        allrep = [None] * world
        dist.all_gather_object(allrep, report)
        if rank == 0:
            same = all(allrep[0][k] == allrep[r][k] for r in range(world) for k in allrep[0])
            q.put(("ok", same, be.getGpuUncapturedErrorCount()))
        dist.barrier()
        lib.tl_comm_destroy(ctx)
        be.destroy()
    except Exception as e:
        if rank == 0:
            q.put(("error", repr(e), -1))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_stack_matches_oracle_and_single_gpu():
    """The tiny stack sharded over two GPUs, both hand-over modes and all three row-parallel sums:
    logits against the CPU oracle and against the unsharded stack with the same seed (<= 2e-2, the
    single-GPU tiny-stack gate), logits and final hidden state bit-identical on both ranks."""
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_stack_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    status, same, errs = q.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
    assert status == "ok", same
    assert same is True, "ranks disagree bit-wise on the sharded stack's outputs"
    assert errs == 0
    assert all(p.exitcode == 0 for p in procs)
