"""GPU tests of the decode matmul stack (the benchmark's workload) through the C ABI.

The tiny stack is checked end to end against the CPU oracle, projection by projection with
the f16 hand-over between them.  The full Qwen3-8B-shaped stack (7.6 GB of int8 weights) is
too large for the oracle, so it is checked through size-independent properties: sampled
lm_head rows against the oracle on the stack's own last hidden state, bit-identical replays,
and batch-row independence (row i of a batch-8 step has the bits of a batch-1 step on that
row: every batch row is its own MMA column and the tile shape does not depend on m <= 8)."""
import numpy as np
import pytest
import torch

import cases
from oracle import oracle as orc
from torchlette_b200.decode_stack import QWEN3_8B, TINY, DecodeStack, StackConfig

pytestmark = pytest.mark.gpu


def _f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def _oracle_proj(x, p, out_f16=True):
    w = p.w.cpu().numpy().astype(np.float32) * p.s.cpu().numpy().astype(np.float32)[:, None]
    y = orc.linear_reference(x, w, None, p.act, alpha=p.alpha)
    return _f16(y) if out_f16 else y


def test_tiny_stack_matches_the_oracle_end_to_end(backend):
    st = DecodeStack(backend, TINY, seed=3)
    gen = torch.Generator(device=st.dev)
    gen.manual_seed(11)
    x = torch.randn(TINY.batch, TINY.hidden, device=st.dev, generator=gen).to(st.tdt)
    st.x.copy_(x)
    torch.cuda.synchronize()
    st.capture()
    st.step()
    backend.sync()
    h = x.float().cpu().numpy()
    for pq, pk, pv, po, pg, pu, pd in st.layers:
        q = _oracle_proj(h, pq)
        h1 = _oracle_proj(q, po)
        g = _oracle_proj(h1, pg)
        h = _oracle_proj(g, pd)
    ref = _oracle_proj(h, st.lm_head, out_f16=False)
    got = st.logits_local.float().cpu().numpy()
    assert cases.rel_err(got, ref) <= 2e-2
    st.destroy()
    assert backend.getGpuUncapturedErrorCount() == 0


def test_full_size_stack_properties(backend):
    cfg8 = StackConfig(**{**QWEN3_8B.__dict__, "batch": 8})
    cfg1 = StackConfig(**{**QWEN3_8B.__dict__, "batch": 1})
    s8 = DecodeStack(backend, cfg8, seed=0)
    gen = torch.Generator(device=s8.dev)
    gen.manual_seed(12)  # seeded: the inputs, like the weights, are the same in every run
    x8 = torch.randn(8, cfg8.hidden, device=s8.dev, generator=gen).to(s8.tdt)
    s8.x.copy_(x8)
    torch.cuda.synchronize()
    s8.capture()
    s8.step()
    backend.sync()
    first = s8.logits_local.clone()
    assert torch.isfinite(first).all() and float(first.abs().max()) > 0
    # replays are bit-identical
    s8.step()
    s8.step()
    backend.sync()
    assert torch.equal(first, s8.logits_local)
    # sampled lm_head rows against the oracle, on the stack's own last hidden state
    rows = np.unique(np.concatenate([np.arange(0, 16), np.arange(75_000, 75_016), np.arange(cfg8.vocab - 16, cfg8.vocab)]))
    h = s8.h2.float().cpu().numpy()
    w = s8.lm_head.w[torch.as_tensor(rows, device=s8.dev)].cpu().numpy().astype(np.float32)
    w *= s8.lm_head.s[torch.as_tensor(rows, device=s8.dev)].cpu().numpy().astype(np.float32)[:, None]
    ref = orc.linear_reference(h, w, None, None, alpha=s8.lm_head.alpha)
    got = first[:, torch.as_tensor(rows, device=s8.dev)].cpu().numpy()
    err = cases.rel_err(got, ref)
    print(f"lm_head sampled rows: rel err {err:.3e}")
    assert err <= 1e-3
    # batch-row independence: the same weights (same seed), batch 1, activation row 5
    s1 = DecodeStack(backend, cfg1, seed=0)
    s1.x.copy_(x8[5:6])
    torch.cuda.synchronize()
    s1.capture()
    s1.step()
    backend.sync()
    assert torch.equal(s1.logits_local[0], first[5])
    s1.destroy()
    s8.destroy()
    assert backend.getGpuUncapturedErrorCount() == 0


@pytest.mark.parametrize("li", [0, 35])
def test_full_size_first_and_last_layer_projections_against_oracle(backend, li):
    """BASELINE config 4 at full size: the seven projections of layer 0 and of the last layer, each
    against the oracle on 48 sampled output columns, computed from the stack's own inputs to that
    projection (so an error cannot hide behind the next one).  f16 outputs: 1e-2."""
    cfg = StackConfig(**{**QWEN3_8B.__dict__, "batch": 8})
    s = DecodeStack(backend, cfg, seed=0)
    try:
        gen = torch.Generator(device=s.dev)
        gen.manual_seed(100 + li)
        xin = torch.randn(8, cfg.hidden, device=s.dev, generator=gen).to(s.tdt)
        (s.x if li == 0 else s.h2).copy_(xin)
        torch.cuda.synchronize()
        s.run_layer(li)
        backend.sync()
        pq, pk, pv, po, pg, pu, pd = s.layers[li]
        checks = [(pq, xin, s.q), (pk, xin, s.kk), (pv, xin, s.v), (po, s.q, s.h1), (pg, s.h1, s.g), (pu, s.h1, s.u), (pd, s.g, s.h2)]
        for p, inp, out in checks:
            rows = np.unique(np.concatenate([np.arange(0, 16), np.arange(p.n // 2, p.n // 2 + 16), np.arange(p.n - 16, p.n)]))
            idx = torch.as_tensor(rows, device=s.dev)
            w = p.w[idx].cpu().numpy().astype(np.float32) * p.s[idx].cpu().numpy().astype(np.float32)[:, None]
            ref = orc.linear_reference(inp.float().cpu().numpy(), w, None, p.act, alpha=p.alpha)
            got = out[:, idx].float().cpu().numpy()
            err = cases.rel_err(got, ref)
            assert err <= 1e-2, (li, p.name, err)
    finally:
        s.destroy()
    assert backend.getGpuUncapturedErrorCount() == 0
