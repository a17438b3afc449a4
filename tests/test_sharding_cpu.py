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


def test_kv_chunks_of_a_sequence_shorter_than_the_world():
    """Five keys over eight ranks: three ranks hold nothing, their partial record is the empty one {-inf, 0, 0...}, and
    the merge of all eight records is the attention over the five keys (the rule the GPU path follows for empty chunks)."""
    from oracle import oracle as O
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 4, 1, 16)).astype(np.float32)
    k, v = (rng.standard_normal((1, 2, 5, 16)).astype(np.float32) for _ in range(2))
    parts, empty = [], 0
    for r in range(8):
        lo, hi = sharding.kv_chunk_range(5, r, 8)
        p = O.attention_partial(q, k, v, 0.25, lo, hi)[:, :, 0]
        if lo == hi:
            empty += 1
            assert np.all(p[..., 0] == -np.inf) and np.all(p[..., 1:] == 0)
        parts.append(p)
    assert empty == 3
    assert np.abs(O.lse_combine(np.stack(parts)) - O.flash_attention(q, k, v, 0.25)[:, :, 0]).max() < 1e-6


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
        # (4) the library communicator's rendezvous: rank 0 makes the 128-byte id, every rank ends up with the same bytes;
        # without a GPU the initialisation itself must refuse with a status code, not crash or fall back
        box = [sharding.Communicator.make_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ids = [None] * world
        dist.all_gather_object(ids, box[0])
        same_id = float(len(box[0]) == 128 and all(i == ids[0] for i in ids))
        # max over ranks, as the benchmark does for its timings
        t = torch.tensor([ok_chunks, ok_heads, ok_proj, 1.0 - same_id], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ret["chunks"], ret["heads"], ret["proj"], ret["id_mismatch"] = float(t[0]), float(t[1]), float(t[2]), float(t[3])
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
    assert ret["id_mismatch"] == 0.0, ret


def test_llama_cache_layer_rule():
    """LlamaCache::new (models/kalosm-llama/src/raw/cache.rs:23-46): with sliding_window_type t and size w, layer i keeps w
    tokens unless (i + 1) % t == 0; without both settings every layer keeps the context length.  No device is touched
    until a layer's first append."""
    from floneum_b200 import LlamaCache
    assert [b.max_sequence_len for b in LlamaCache(6, 8192, 3, 512).blocks] == [512, 512, 8192, 512, 512, 8192]
    assert [b.max_sequence_len for b in LlamaCache(4, 4096).blocks] == [4096] * 4
    assert [b.max_sequence_len for b in LlamaCache(3, 4096, sliding_window_type=2).blocks] == [4096] * 3  # size missing: no window
    assert [b.max_sequence_len for b in LlamaCache(3, 4096, 1, 128).blocks] == [4096] * 3             # every layer is global
    c = LlamaCache.new(2, 100, 2, 10)
    assert c.start_time == 0 and c.tokens == [] and all(b.concat_dim == 2 and b.current_seq_len() == 0 for b in c.blocks)
    c.clear()


def test_communicator_needs_a_device_and_checks_arguments():
    import ctypes
    import torch
    from floneum_b200 import _lib
    L = _lib.load()
    h = ctypes.c_void_p()
    assert L.fusor_cuda_comm_init(None, b"x" * 128, 0, 1, 1000, ctypes.byref(h)) == _lib.INVALID_ARGUMENT
    assert L.fusor_cuda_comm_unique_id(None) == _lib.INVALID_ARGUMENT
    assert L.fusor_cuda_comm_poll(None) == _lib.INVALID_ARGUMENT
    assert L.fusor_cuda_comm_destroy(None) == _lib.OK
    assert L.fusor_cuda_exchange_disconnect(None) == _lib.OK
    if not torch.cuda.is_available():
        from floneum_b200 import Device, FusorCudaError
        with pytest.raises(FusorCudaError):
            Device.gpu(0)  # no context, hence no communicator: there is no CPU path behind the C ABI
