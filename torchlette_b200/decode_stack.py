"""A decoder-shaped stack of quantized projections (q/k/v/o/gate/up/down per
layer plus lm_head) driven through the C ABI, single GPU or tensor-parallel.

This is the matmul skeleton of a Qwen3-style decode step with everything that
is not a weight matmul removed: the o projection consumes the q projection's
output in place of the attention output, the down projection consumes
silu(gate) (fused epilogue).  Per-projection ``alpha`` keeps activations O(1)
through random-init weights.

Tensor parallel (one process per GPU): q/k/v/gate/up/lm_head are column-parallel,
o/down row-parallel.  In "chained" mode the column-parallel outputs feed the
row-parallel projections' K slices directly and each layer costs two all-reduces
(plus one all-gather of the logits); in "gather" mode every column-parallel
output is all-gathered and the row-parallel input re-sliced.

torch supplies device memory, random init and the process group; all compute on
the timed path is this library's kernels plus NCCL.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import binding as B
from .backend import CudaBackend
from .sharding import plan_shard


@dataclass
class StackConfig:
    hidden: int = 4096
    layers: int = 36
    q_out: int = 4096      # 32 heads x 128
    kv_out: int = 1024     # 8 kv heads x 128
    inter: int = 12288
    vocab: int = 151936
    batch: int = 8
    act_dtype: str = "f16"

    def projections(self):
        """(name, K, N, parallel mode) of one layer, in execution order."""
        h = self.hidden
        return [("q", h, self.q_out, "column"), ("k", h, self.kv_out, "column"), ("v", h, self.kv_out, "column"),
                ("o", self.q_out, h, "row"), ("gate", h, self.inter, "column"), ("up", h, self.inter, "column"),
                ("down", self.inter, h, "row")]

    def weight_bytes_per_step(self) -> int:
        per_layer = sum(k * n for _, k, n, _ in self.projections())
        return per_layer * self.layers + self.hidden * self.vocab

    def algorithmic_bytes_per_step(self) -> int:
        """int8 weights + f32 per-channel scales + activations in + outputs."""
        m, a = self.batch, 2
        total = 0
        for _, k, n, _ in self.projections():
            total += n * k + n * 4 + m * k * a + m * n * a
        total *= self.layers
        total += self.vocab * self.hidden + self.vocab * 4 + m * self.hidden * a + m * self.vocab * 4
        return total

    def flops_per_step(self) -> int:
        return 2 * self.batch * self.weight_bytes_per_step()


QWEN3_8B = StackConfig()
# same layer shapes, two layers and a small vocabulary: smoke tests and CPU-side checks
TINY = StackConfig(hidden=256, layers=2, q_out=256, kv_out=64, inter=512, vocab=1024, batch=2)


class _Proj:
    __slots__ = ("name", "k", "n", "mode", "w", "s", "alpha", "act", "out_dtype")


class DecodeStack:
    def __init__(self, be: CudaBackend, cfg: StackConfig, rank: int = 0, world: int = 1, tp_mode: str = "chained",
                 seed: int = 0, allreduce: str = "nccl", fuse: bool = True, chain: bool = False,
                 loopback_push: bool = False):
        assert tp_mode in ("chained", "gather") and allreduce in ("nccl", "p2p", "fused", "push")
        # chain: the whole step as ONE persistent cooperative launch (tl_qgemv_chain_*); single rank,
        # batch <= 16 only -- elsewhere the step stays a graph of per-projection launches
        self.chain_requested = chain
        # one rank with a loopback exchange attached (tl_p2p_attach_loopback(ctx, 1)): the row-parallel
        # projections still go through tl_qgemv_nt_push and its reduce-on-read consumer
        self.loopback_push = loopback_push
        self._partials = {}
        self._chain = None
        self._chain_keep = []
        self.be, self.cfg, self.rank, self.world, self.tp_mode = be, cfg, rank, world, tp_mode
        self.fuse = fuse  # q/k/v and gate/up as one launch each
        # "p2p": the library's one-shot peer-memory all-reduce (peers must be attached);
        # "fused": the row-parallel projections do their own all-reduce (tl_qgemv_nt_allreduce);
        # "push": they push their partials and the next launch sums them (tl_qgemv_nt_push)
        self.allreduce = allreduce
        self.dev = torch.device("cuda", be.device)
        self.lib, self.ctx = be._lib, be._ctx
        self.tdt = torch.float16 if cfg.act_dtype == "f16" else torch.bfloat16
        self.adt = B.DTYPE_ID[cfg.act_dtype]
        gen = torch.Generator(device=self.dev)
        self.layers = []
        sigma_w = 73.32 * math.sqrt((1e-6 + 1e-5 + 1e-4) / 3.0)  # std of q*s for q~U[-127,127], s~U[.001,.01]
        for li in range(cfg.layers):
            projs = []
            for pi, (name, k, n, mode) in enumerate(cfg.projections()):
                projs.append(self._make_proj(gen, seed + 1000 * li + pi, name, k, n, mode, sigma_w))
            self.layers.append(projs)
        self.lm_head = self._make_proj(gen, seed + 999_983, "lm_head", cfg.hidden, cfg.vocab, "column", sigma_w)
        self.lm_head.out_dtype = "f32"
        m, h = cfg.batch, cfg.hidden
        w = world
        z = lambda *shape, dt=self.tdt: torch.zeros(*shape, dtype=dt, device=self.dev)  # noqa: E731
        self.x = z(m, h)
        self.q, self.kk, self.v = z(m, cfg.q_out // w), z(m, cfg.kv_out // w), z(m, cfg.kv_out // w)
        self.h1 = z(m, h)
        self.g, self.u = z(m, cfg.inter // w), z(m, cfg.inter // w)
        self.h2 = z(m, h)
        self.logits_local = z(m, cfg.vocab // w, dt=torch.float32)
        self.logits = z(m, cfg.vocab, dt=torch.float32) if w > 1 else self.logits_local
        if tp_mode == "gather" and w > 1:
            self.q_full, self.g_full = z(m, cfg.q_out), z(m, cfg.inter)
            self.q_slice, self.g_slice = z(m, cfg.q_out // w), z(m, cfg.inter // w)
        torch.cuda.synchronize(self.dev)
        self.graph: Optional[int] = None

    def _make_proj(self, gen, seed, name, k, n, mode, sigma_w) -> _Proj:
        sh = plan_shard(mode, n, k, k, self.rank, self.world)
        p = _Proj()
        p.name, p.k, p.n, p.mode = name, sh.k, sh.n, mode
        # Every rank draws the FULL [N, K] matrix and its scales from the projection's seed (the
        # device generator gives the same stream on every GPU) and keeps its own slice, so a stack
        # sharded over g ranks is the same model as the single-GPU stack with that seed.
        gen.manual_seed(seed)
        full = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=self.dev, generator=gen)
        scales = torch.empty(n, dtype=torch.float32, device=self.dev).uniform_(0.001, 0.01, generator=gen)
        p.w = full[sh.n_offset:sh.n_offset + sh.n, sh.k_offset:sh.k_offset + sh.k].contiguous()
        p.s = scales[sh.n_offset:sh.n_offset + sh.n].contiguous()
        del full, scales
        # silu(gate) roughly halves the rms at unit amplitude but is linear at large amplitude, and the
        # stack has no normalisation between layers: 1.6 keeps the hidden state inside the f16 range
        # over 36 layers (1.8 let it grow to ~3e4, half of the f16 maximum)
        p.alpha = (1.6 if name == "down" else 1.0) / (sigma_w * math.sqrt(k))
        p.act = "silu" if name == "gate" else None
        p.out_dtype = self.cfg.act_dtype
        return p

    # -- one projection through the C ABI ------------------------------------
    def _run(self, p: _Proj, x: torch.Tensor, out: torch.Tensor, out_dtype: Optional[str] = None):
        q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, p.k, B.TL_F32, B.TL_SCALE_DIRECT)
        e = None
        if p.act:
            e = B.Epilogue()
            e.n_ops = 1
            e.ops[0] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY[p.act], 0, 0)
        B.check(self.ctx, self.lib.tl_qmatmul_nt(
            self.ctx, x.data_ptr(), self.adt, p.w.data_ptr(), p.s.data_ptr(), out.data_ptr(),
            B.DTYPE_ID[out_dtype or p.out_dtype], self.cfg.batch, p.n, p.k, C.byref(q), p.alpha,
            C.byref(e) if e is not None else None))

    def _run_batched(self, projs, x: torch.Tensor, outs):
        """Projections that read the same activations in one launch (tl_qgemv_nt_batched)."""
        if self.cfg.batch > 16 or not self.fuse:
            for p, o in zip(projs, outs):
                self._run(p, x, o)
            return
        items = (B.QGemvItem * len(projs))()
        keep = []
        for i, (p, o) in enumerate(zip(projs, outs)):
            e = None
            if p.act:
                e = B.Epilogue()
                e.n_ops = 1
                e.ops[0] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY[p.act], 0, 0)
                keep.append(e)
            items[i] = B.QGemvItem(p.w.data_ptr(), p.s.data_ptr(), o.data_ptr(), p.n, p.alpha,
                                   C.pointer(e) if e is not None else None)
        q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, projs[0].k, B.TL_F32, B.TL_SCALE_DIRECT)
        B.check(self.ctx, self.lib.tl_qgemv_nt_batched(self.ctx, x.data_ptr(), self.adt, items, len(projs),
                                                       B.DTYPE_ID[projs[0].out_dtype], self.cfg.batch, projs[0].k,
                                                       C.byref(q)))

    def _run_row_parallel(self, p: _Proj, x: torch.Tensor, out: torch.Tensor):
        """o / down: the partial product and its sum over ranks."""
        if self.world > 1 and self.allreduce == "fused" and self.cfg.batch <= 16 and not p.act:
            q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, p.k, B.TL_F32, B.TL_SCALE_DIRECT)
            B.check(self.ctx, self.lib.tl_qgemv_nt_allreduce(
                self.ctx, x.data_ptr(), self.adt, p.w.data_ptr(), p.s.data_ptr(), out.data_ptr(),
                B.DTYPE_ID[p.out_dtype], self.cfg.batch, p.n, p.k, C.byref(q), p.alpha))
            return
        if (self.world > 1 or self.loopback_push) and self.allreduce == "push" and self.cfg.batch <= 16 and not p.act \
                and self.tp_mode == "chained":
            # the partial goes to every rank's exchange buffer; the NEXT launch (q+k+v, gate+up or lm_head,
            # which reads `out`) sums the ranks' partials in its prologue: no collective launch at all
            q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, p.k, B.TL_F32, B.TL_SCALE_DIRECT)
            B.check(self.ctx, self.lib.tl_qgemv_nt_push(
                self.ctx, x.data_ptr(), self.adt, p.w.data_ptr(), p.s.data_ptr(), out.data_ptr(),
                B.DTYPE_ID[p.out_dtype], self.cfg.batch, p.n, p.k, C.byref(q), p.alpha))
            return
        if self.world == 1:
            self._run(p, x, out)
            return
        # The partial products are exchanged in f32 and their sum is rounded ONCE to the activation
        # type: 16-bit partials lose up to half an ulp of a partial that can be far larger than the
        # total, and at 8 ranks that alone reaches the 1e-2 parity bound.
        part = self._partial_f32(out)
        self._run(p, x, part, out_dtype="f32")
        if self.allreduce in ("p2p", "fused", "push"):
            B.check(self.ctx, self.lib.tl_allreduce_sum_p2p_f32_to(self.ctx, part.data_ptr(), out.data_ptr(), self.adt, part.numel()))
        else:
            B.check(self.ctx, self.lib.tl_allreduce_sum(self.ctx, part.data_ptr(), part.numel(), B.TL_F32))
            B.check(self.ctx, self.lib.tl_unary_op(self.ctx, 0, part.data_ptr(), B.TL_F32, out.data_ptr(), self.adt, part.numel()))

    def _partial_f32(self, like: torch.Tensor) -> torch.Tensor:
        """One f32 buffer per output shape for the row-parallel partial products."""
        key = tuple(like.shape)
        if key not in self._partials:
            self._partials[key] = torch.empty(like.shape, dtype=torch.float32, device=like.device)
        return self._partials[key]

    def _allgather(self, local: torch.Tensor, full: torch.Tensor, dtype_id: int):
        B.check(self.ctx, self.lib.tl_allgather_cols(self.ctx, local.data_ptr(), full.data_ptr(), local.shape[0],
                                                     local.shape[1], dtype_id))

    def _slice_cols(self, full: torch.Tensor, out: torch.Tensor):
        w, esz = out.shape[1], full.element_size()
        # strided device-to-device copy of this rank's K slice, on the library's stream
        B.check(self.ctx, self.lib.tl_copy2d(self.ctx, out.data_ptr(), w * esz, full.data_ptr() + self.rank * w * esz,
                                             full.shape[1] * esz, w * esz, out.shape[0]))

    # -- the whole step as one persistent launch --------------------------------
    def _phase(self, x: torch.Tensor, projs, outs) -> "B.ChainPhase":
        ph = B.ChainPhase()
        ph.a, ph.k, ph.group_size = x.data_ptr(), projs[0].k, projs[0].k
        ph.out_dtype, ph.n_items = B.DTYPE_ID[projs[0].out_dtype], len(projs)
        for i, (p, o) in enumerate(zip(projs, outs)):
            e = None
            if p.act:
                e = B.Epilogue()
                e.n_ops = 1
                e.ops[0] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY[p.act], 0, 0)
                self._chain_keep.append(e)
            ph.items[i] = B.QGemvItem(p.w.data_ptr(), p.s.data_ptr(), o.data_ptr(), p.n, p.alpha,
                                      C.pointer(e) if e is not None else None)
        return ph

    def uses_chain(self) -> bool:
        return self.chain_requested and self.world == 1 and self.cfg.batch <= 16

    def build_chain(self):
        """Describe the step to the library once: 4 phases per layer (q+k+v, o, gate+up, down) + lm_head."""
        phases = []
        x = self.x
        for pq, pk, pv, po, pg, pu, pd in self.layers:
            phases.append(self._phase(x, (pq, pk, pv), (self.q, self.kk, self.v)))
            phases.append(self._phase(self.q, (po,), (self.h1,)))
            phases.append(self._phase(self.h1, (pg, pu), (self.g, self.u)))
            phases.append(self._phase(self.g, (pd,), (self.h2,)))
            x = self.h2
        phases.append(self._phase(x, (self.lm_head,), (self.logits_local,)))
        arr = (B.ChainPhase * len(phases))(*phases)
        handle = C.c_void_p()
        B.check(self.ctx, self.lib.tl_qgemv_chain_create(self.ctx, arr, len(phases), self.adt, self.cfg.batch,
                                                         B.TL_F32, B.TL_SCALE_DIRECT, C.byref(handle)))
        self._chain = handle
        return handle

    def enqueue_step(self):
        """Enqueue one pass over the whole stack on the library's stream."""
        if self.uses_chain():
            if self._chain is None:
                self.build_chain()
            B.check(self.ctx, self.lib.tl_qgemv_chain_launch(self.ctx, self._chain))
            return
        x = self.x
        for projs in self.layers:
            x = self._enqueue_layer(projs, x)
        self._run(self.lm_head, x, self.logits_local)
        if self.world > 1:
            self._allgather(self.logits_local, self.logits, B.TL_F32)

    def _enqueue_layer(self, projs, x: torch.Tensor) -> torch.Tensor:
        gather = self.tp_mode == "gather" and self.world > 1
        pq, pk, pv, po, pg, pu, pd = projs
        self._run_batched((pq, pk, pv), x, (self.q, self.kk, self.v))
        o_in = self.q
        if gather:
            self._allgather(self.q, self.q_full, self.adt)
            self._slice_cols(self.q_full, self.q_slice)
            o_in = self.q_slice
        self._run_row_parallel(po, o_in, self.h1)
        self._run_batched((pg, pu), self.h1, (self.g, self.u))
        d_in = self.g
        if gather:
            self._allgather(self.g, self.g_full, self.adt)
            self._slice_cols(self.g_full, self.g_slice)
            d_in = self.g_slice
        self._run_row_parallel(pd, d_in, self.h2)
        return self.h2

    def run_layer(self, li: int):
        """Enqueue layer ``li`` alone (input self.x for layer 0, else the current self.h2): the buffers
        q/kk/v/h1/g/u/h2 then hold that layer's results, which a test checks projection by projection."""
        self._enqueue_layer(self.layers[li], self.x if li == 0 else self.h2)

    def capture(self):
        """Run once eagerly (sizes scratch, warms caches), then capture the step
        as a replayable graph — the analogue of the reference's compiled plans."""
        self.enqueue_step()
        self.be.sync()
        if self.uses_chain():
            return None  # already a single launch: nothing for a graph to save
        self.be.beginCapture()
        try:
            self.enqueue_step()
        finally:
            self.graph = self.be.endCapture()
        return self.graph

    def step(self):
        if self.graph is not None:
            self.be.replay(self.graph)
        else:
            self.enqueue_step()

    def launches_per_step(self) -> int:
        if self.uses_chain():
            return 1
        fused = self.fuse and self.cfg.batch <= 16
        return (4 if fused else 7) * self.cfg.layers + 1

    def destroy(self):
        if self._chain is not None:
            self.lib.tl_qgemv_chain_destroy(self.ctx, self._chain)
            self._chain = None
        if self.graph is not None:
            self.be.destroyGraph(self.graph)
            self.graph = None
