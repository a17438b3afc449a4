"""Multi-GPU host logic on CPU: world_size-2 gloo process groups exercise the partitioning helpers and the
all-gather of split-KV partials (floneum_b200/sharding.py).  The oracle stands in for the per-rank kernel."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from floneum_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partition_helpers():
    assert [sharding.kv_head_range(8, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert [sharding.q_head_range(32, 8, r, 2) for r in range(2)] == [(0, 16), (16, 32)]
    with pytest.raises(ValueError):
        sharding.kv_head_range(8, 0, 3)
    with pytest.raises(ValueError, match="must be divisible"):
        sharding.q_head_range(30, 8, 0, 2)
    for n, w in [(131072, 8), (1000, 3), (7, 8)]:
        rs = [sharding.kv_chunk_range(n, r, w) for r in range(w)]
        assert rs[0][0] == 0 and rs[-1][1] == n and all(rs[i][1] == rs[i + 1][0] for i in range(w - 1))
        sizes = [b - a for a, b in rs]
        assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        rng = np.random.default_rng(11)  # the same tensors on every rank
        B, Hq, Hkv, Skv, D = 2, 8, 4, 333, 32
        q = rng.standard_normal((B, Hq, 1, D), dtype=np.float32)
        k = rng.standard_normal((B, Hkv, Skv, D), dtype=np.float32)
        v = rng.standard_normal((B, Hkv, Skv, D), dtype=np.float32)
        scale = 0.2
        full = O.flash_attention(q, k, v, scale)
        # (1) KV-sequence chunks: local partial -> all-gather -> log-sum-exp merge on every rank
        lo, hi = sharding.kv_chunk_range(Skv, rank, world)
        part = O.attention_partial(q, k, v, scale, lo, hi)[:, :, 0]           # [B, Hq, D+2]
        gathered = sharding.all_gather_partials(torch.from_numpy(part))       # [world, B, Hq, D+2]
        assert tuple(gathered.shape) == (world, B, Hq, D + 2)
        merged = O.lse_combine(gathered.numpy())
        ok_chunks = float(np.abs(merged - full[:, :, 0]).max())
        # (2) KV-head shards: no collective on the data path; each rank's slice equals the same slice of the full result
        q0, q1 = sharding.q_head_range(Hq, Hkv, rank, world)
        k0, k1 = sharding.kv_head_range(Hkv, rank, world)
        mine = O.flash_attention(q[:, q0:q1], k[:, k0:k1], v[:, k0:k1], scale)
        ok_heads = float(np.abs(mine - full[:, q0:q1]).max())
        # (3) output projection over head shards: partial sums of this rank's heads x weight columns, all-reduced
        N = 24
        w = rng.standard_normal((N, Hq * D), dtype=np.float32)
        bias = rng.standard_normal(N, dtype=np.float32)
        attn_full = rng.standard_normal((B, Hq, 5, D), dtype=np.float32)
        c0, c1 = sharding.out_proj_weight_columns(Hq, Hkv, D, rank, world)
        assert (c0, c1) == (q0 * D, q1 * D)
        part_o = O.out_proj(attn_full[:, q0:q1], np.ascontiguousarray(w[:, c0:c1]), bias if rank == 0 else None)
        summed = sharding.all_reduce_sum(torch.from_numpy(part_o)).numpy()
        ok_proj = float(np.abs(summed - O.out_proj(attn_full, w, bias)).max())
        # max over ranks, as the benchmark does for its timings
        t = torch.tensor([ok_chunks, ok_heads, ok_proj], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ret["chunks"], ret["heads"], ret["proj"] = float(t[0]), float(t[1]), float(t[2])
    finally:
        dist.destroy_process_group()


def test_kv_chunk_allgather_and_head_shards_world2():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert ret["chunks"] < 2e-6, ret
    assert ret["heads"] == 0.0, ret
    assert ret["proj"] < 1e-4, ret  # f32 sums of 256 terms of size ~1 in two different orders
