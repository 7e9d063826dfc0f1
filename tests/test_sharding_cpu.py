"""Tensor-parallel sharding of packed weights: pure host logic, plus the N > 1
data path run as world_size-2 gloo ranks on CPU with the oracle standing in for
the GPU kernels (column-parallel + all-gather, row-parallel + all-reduce)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from oracle import oracle as orc
from torchlette_b200.sharding import plan_shard, shard_activation, shard_weight


def test_plan_shard_geometry_and_errors():
    s = plan_shard("column", 4096, 1024, 1024, 1, 4)
    assert (s.n, s.k, s.n_offset, s.k_offset, s.group) == (1024, 1024, 1024, 0, 1024)
    s = plan_shard("row", 4096, 12288, 12288, 3, 8)  # per-channel stays per-channel
    assert (s.n, s.k, s.k_offset, s.group) == (4096, 1536, 4608, 1536)
    s = plan_shard("row", 64, 1024, 64, 1, 2)
    assert (s.k, s.k_offset, s.group) == (512, 512, 64)
    with pytest.raises(ValueError):
        plan_shard("column", 10, 64, 64, 0, 4)
    with pytest.raises(ValueError):
        plan_shard("row", 8, 24, 24, 0, 4)      # K/world = 6 not divisible by 4
    with pytest.raises(ValueError):
        plan_shard("row", 8, 256, 64, 0, 8)     # K/world = 32 not divisible by G = 64
    with pytest.raises(ValueError):
        plan_shard("row", 8, 256, 64, 2, 2)
    with pytest.raises(ValueError):
        plan_shard("diagonal", 8, 256, 64, 0, 2)


@pytest.mark.parametrize("group", [64, 256])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_sharded_results_reassemble(group, world):
    """Column shards concatenate, row shards sum, to the unsharded oracle result."""
    n, k, m = 48, 256, 3
    rng = np.random.default_rng(world)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    packed, scales = orc.quantize_linear_weight(w, group)
    full = orc.matmul_nt(x, orc.dequantize_to_f32(packed, scales, k, group))
    cols, partial = [], np.zeros((m, n), dtype=np.float64)
    for r in range(world):
        sc = plan_shard("column", n, k, group, r, world)
        pk, ss = shard_weight(packed, scales, n, k, group, sc)
        cols.append(orc.matmul_nt(shard_activation(x, sc), orc.dequantize_to_f32(pk, ss, sc.k, sc.group)))
        sr = plan_shard("row", n, k, group, r, world)
        pk, ss = shard_weight(packed, scales, n, k, group, sr)
        if group == k:  # per-channel abs-max scale is shared by every K slice of the row
            wr = orc.dequantize_to_f32(pk, np.repeat(ss, 1, axis=1), sr.k, sr.k)
        else:
            wr = orc.dequantize_to_f32(pk, ss, sr.k, sr.group)
        partial += orc.matmul_nt(shard_activation(x, sr), wr)
    assert np.array_equal(np.concatenate(cols, axis=1), full)  # column-parallel is exact
    assert cases.rel_err(partial.astype(np.float32), full) <= 1e-5  # row-parallel only reorders the K sum


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, k, m = 64, 128, 2
        cs = cases.per_channel_case(n, k, m, seed=12, act_dtype="f16")
        # column-parallel q projection -> (chained) row-parallel o projection, as the decode stack does
        sc = plan_shard("column", n, k, k, rank, world)
        pk, ss = shard_weight(cs["packed"], cs["scales"], n, k, k, sc)
        y_local = orc.matmul_nt(cs["x"], orc.dequantize_direct_f32(pk, ss, sc.k, sc.k))
        gathered = [torch.zeros(m, sc.n) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(y_local))
        y = torch.cat(gathered, dim=1).numpy()
        cs2 = cases.per_channel_case(32, n, m, seed=13)
        sr = plan_shard("row", 32, n, n, rank, world)
        pk2, ss2 = shard_weight(cs2["packed"], cs2["scales"], 32, n, n, sr)
        part = orc.matmul_nt(np.ascontiguousarray(y_local), orc.dequantize_direct_f32(pk2, ss2, sr.k, sr.k))
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        if rank == 0:
            q.put((y, t.numpy()))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_single_rank():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    y, z = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    n, k, m = 64, 128, 2
    cs = cases.per_channel_case(n, k, m, seed=12, act_dtype="f16")
    y_ref = orc.matmul_nt(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k))
    assert np.array_equal(y, y_ref)
    cs2 = cases.per_channel_case(32, n, m, seed=13)
    z_ref = orc.matmul_nt(y_ref, orc.dequantize_direct_f32(cs2["packed"], cs2["scales"], n, n))
    assert cases.rel_err(z, z_ref) <= 1e-5
