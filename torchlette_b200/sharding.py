"""Tensor-parallel sharding of packed int8 weights across the GPUs of one node.

The quantized matmul shards naturally: output columns are independent
(column-parallel, results concatenated by an all-gather) and a dot product over
K is a sum of dot products over K slices (row-parallel, partials summed by an
all-reduce).  The reference has no counterpart (its only parallelism is DiLoCo
data parallel over WebSocket, src/distributed/); the packed layout sliced here is
the one src/backend/quantize.ts:62-131 defines: u32 [N, K/4], scales [N, K/G].

Pure host logic (numpy), shared by the benchmark and by CPU tests that run the
collectives over gloo.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Shard:
    mode: str        # "column" | "row"
    rank: int
    world: int
    n: int           # local N
    k: int           # local K
    n_offset: int    # first global output column held
    k_offset: int    # first global k held
    group: int       # local group size (per-channel stays per-channel: == local K)


def plan_shard(mode: str, n: int, k: int, group: int, rank: int, world: int) -> Shard:
    """Geometry of rank's shard, or ValueError when the shape cannot be split."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    per_channel = group == k
    if mode == "column":
        if n % world != 0:
            raise ValueError(f"column-parallel: N={n} must be divisible by world={world}")
        nl = n // world
        return Shard("column", rank, world, nl, k, rank * nl, 0, group)
    if mode == "row":
        if k % world != 0:
            raise ValueError(f"row-parallel: K={k} must be divisible by world={world}")
        kl = k // world
        if kl % 4 != 0:
            raise ValueError(f"row-parallel: K/world={kl} must be divisible by 4 (packing)")
        if not per_channel and kl % group != 0:
            raise ValueError(f"row-parallel: K/world={kl} must be divisible by groupSize={group}")
        return Shard("row", rank, world, n, kl, 0, rank * kl, kl if per_channel else group)
    raise ValueError(f"unknown shard mode {mode}")


def shard_weight(packed: np.ndarray, scales: np.ndarray, n: int, k: int, group: int, s: Shard):
    """Slices of the packed words and the scales for shard ``s``.  Per-channel
    scales are replicated across row-parallel ranks (each partial is scaled by
    the same s[n] before the sum)."""
    packed = np.asarray(packed).reshape(n, k // 4)
    scales = np.asarray(scales).reshape(n, k // group)
    if s.mode == "column":
        rows = slice(s.n_offset, s.n_offset + s.n)
        return np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scales[rows])
    words = slice(s.k_offset // 4, (s.k_offset + s.k) // 4)
    if group == k:
        return np.ascontiguousarray(packed[:, words]), np.ascontiguousarray(scales)
    groups = slice(s.k_offset // group, (s.k_offset + s.k) // group)
    return np.ascontiguousarray(packed[:, words]), np.ascontiguousarray(scales[:, groups])


def shard_activation(x: np.ndarray, s: Shard) -> np.ndarray:
    """Row-parallel ranks take the matching K slice of the activation; column-
    parallel ranks take all of it."""
    if s.mode == "column":
        return x
    return np.ascontiguousarray(x[..., s.k_offset:s.k_offset + s.k])
