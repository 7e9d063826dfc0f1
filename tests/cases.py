"""Seeded synthetic inputs for the benchmark configurations and the reference
probes' own gate shapes.  Shared by the CPU and GPU tests so both sides see the
same bits."""
from __future__ import annotations

import numpy as np


def pack_int8(q: np.ndarray) -> np.ndarray:
    """int8 [N,K] -> u32 [N,K/4], byte lane = k & 3 (little-endian lanes)."""
    q = np.ascontiguousarray(q, dtype=np.int8)
    return q.view(np.uint32).reshape(q.shape[0], q.shape[1] // 4)


def per_channel_case(n, k, m, seed, act_dtype="f32", bias=False):
    """Benchmark-config inputs: draw order q, scales, activations, bias."""
    rng = np.random.Generator(np.random.PCG64(seed))
    q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = rng.uniform(0.001, 0.01, size=(n, 1)).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal(n) * 0.02).astype(np.float32) if bias else None
    if act_dtype == "f16":
        x_bits = x.astype(np.float16).view(np.uint16)
        x = x_bits.view(np.float16).astype(np.float32)
    elif act_dtype == "bf16":
        u = x.view(np.uint32).astype(np.uint64)
        x_bits = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        x = (x_bits.astype(np.uint32) << 16).view(np.float32)
    else:
        x_bits = x
    return {"q": q, "packed": pack_int8(q), "scales": s, "x": x, "x_bits": x_bits, "bias": b}


def rel_err(x: np.ndarray, ref: np.ndarray) -> float:
    """The reference probes' error metric |x-ref| / max(1,|ref|)
    (examples/qwen3/probe-quant-gemv.ts:166-177), maximum over elements."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(x - ref) / np.maximum(1.0, np.abs(ref)))) if ref.size else 0.0


def drift(x: np.ndarray, ref: np.ndarray) -> float:
    """max-abs / RMS(ref) (examples/qwen3/probe-quant-operand.ts:101-109)."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 1.0
    return float(np.max(np.abs(x - ref))) / (rms if rms > 0 else 1.0)
