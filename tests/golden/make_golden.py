"""Generates the known-answer fixtures in this directory from the CPU oracle.

The reference ships no golden vectors for the quantized matmul path and cannot
be run where this was written (no node), so these vectors pin the ORACLE against
regressions and travel to machines without the reference; they do not pin it
against the reference (parity unpinned).

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle as orc  # noqa: E402
import cases  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def probe_quant_gemv_case(n, k, group, state):
    """Inputs exactly as examples/qwen3/probe-quant-gemv.ts:80-100 draws them:
    one LCG stream, weights [N,K] first, then activations [K]."""
    w, state = orc.lcg_fill(state, n * k)
    a, state = orc.lcg_fill(state, k)
    w = w.reshape(n, k)
    packed, scales = orc.quantize_linear_weight(w, group)
    deq = orc.dequantize_to_f32(packed, scales, k, group)
    y = orc.matmul_nt(a.reshape(1, k), deq, threads=1)
    return dict(w=w, a=a, packed=packed, scales=scales, deq=deq, y=y), state


def main():
    # 1. first two shapes of the probe-quant-gemv sweep (G=64), seed 0x51a7ee
    state = 0x51A7EE
    c, state = probe_quant_gemv_case(128, 128, 64, state)
    np.savez_compressed(os.path.join(OUT, "probe_quant_gemv_128x128_g64.npz"),
                        packed=c["packed"], scales=c["scales"], a=c["a"], y=c["y"],
                        deq_row0=c["deq"][0], deq_row127=c["deq"][127], w_head=c["w"][0, :16],
                        next_state=np.uint32(state))
    # 2. probe-quant-operand style: seed 0x51 ^ N ^ (K<<3) ^ (G<<7), w = rng()*0.1, M=4
    n, k, g, m = 128, 128, 64, 4
    st = (0x51 ^ n ^ (k << 3) ^ (g << 7)) & 0xFFFFFFFF
    w, st = orc.lcg_fill(st, n * k, 0.1)
    x, st = orc.lcg_fill(st, m * k)
    packed, scales = orc.quantize_linear_weight(w.reshape(n, k), g)
    deq = orc.dequantize_to_f32(packed, scales, k, g)
    y = orc.matmul_nt(x.reshape(m, k), deq, threads=1)
    np.savez_compressed(os.path.join(OUT, "probe_quant_operand_128x128_g64_m4.npz"),
                        packed=packed, scales=scales, x=x.reshape(m, k), y=y)
    # 3. benchmark config 0 slice: per-channel direct scales, f32 activations, first 64 rows
    cs = cases.per_channel_case(2048, 2048, 1, seed=0)
    wdq = orc.dequantize_direct_f32(cs["packed"][:64], cs["scales"][:64], 2048, 2048)
    y = orc.matmul_nt(cs["x"], wdq, threads=1)
    np.savez_compressed(os.path.join(OUT, "config0_rows0_63.npz"), y=y, scales=cs["scales"][:64],
                        q_head=cs["q"][0, :32], x_head=cs["x"][0, :32])
    # 4. activations + f16 converter spot values
    xs = np.array([-6, -3, -1, -0.5, -1e-3, 0, 1e-3, 0.5, 1, 2, 3, 6, 10], dtype=np.float32)
    acts = {name: orc.unary(name, xs) for name in ("relu", "silu", "sigmoid", "tanh", "gelu", "gelu_erf")}
    f16_in = np.array([0, 1, -1, 0.1, 65504, 65520, 1e-5, 6e-8, 3e-8, 2.98e-8, 1e-10, 0.333251953125, 1000.5],
                      dtype=np.float32)
    np.savez_compressed(os.path.join(OUT, "elementwise.npz"), xs=xs, f16_in=f16_in,
                        f16_bits=orc.f32_to_f16_bits(f16_in), **acts)
    print("wrote fixtures to", OUT)


if __name__ == "__main__":
    main()
