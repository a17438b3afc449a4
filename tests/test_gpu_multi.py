"""Two-GPU checks (skipped when fewer than two GPUs are visible): the peer-memory exchange of split-KV records, the
KV-chunk decode built on it and the library's communicator with the head-sharded output projection, one process per GPU,
against the oracle on the unsplit problem.  No GPU is made to fault or hang: a peer that never publishes is covered by the
bounded wait (TIMEOUT status) that tests/test_gpu_decode.py exercises on one GPU, and a rank that never joins a
communicator is a host-side deadline (last test, one GPU)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        import floneum_b200 as fb
        from floneum_b200 import sharding
        from oracle import workloads as W
        from oracle import oracle as O
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            dev = fb.Device.gpu(rank, stream.cuda_stream)
            w = W.cfg4(Skv=8192, rank=rank, world=world)  # this rank's chunk of an 8192-token sequence, paged
            B, Hq, _, D = w.q.shape
            cache = fb.PagedKvCache(dev, B, w.k_pages.shape[1], D, w.k_pages.shape[0], w.page_table.shape[1])
            cache.write_pages(0, w.k_pages, w.v_pages)
            cache.set_page_table(w.page_table, w.kv_len)
            ex = sharding.PeerExchange(dev, rank, world, B * Hq * (D + 2))
            q = fb.Tensor.from_slice(dev, w.q.shape, w.q, 1)
            part = torch.empty((B, Hq, D + 2), dtype=torch.float32, device=f"cuda:{rank}")
            out = torch.empty((B, Hq, D), dtype=torch.float32, device=f"cuda:{rank}")
            worst = 0.0
            full = W.cfg4(Skv=8192)
            want = O.flash_attention(full.q, full.k_dense[0][None], full.v_dense[0][None], full.scale)[:, :, 0]
            for step in range(4):  # several steps: both slot parities, epochs 1..4; both producers of the records
                if step % 2 == 0:  # split-KV kernel, then one kernel: merge local records, store on every rank, wait, merge
                    ex.decode(cache, q, w.scale, fb.Tensor.from_torch(dev, out))
                else:              # records the caller holds: push, publish, wait and merge in one launch
                    cache.decode_partial(q, w.scale, fb.Tensor.from_torch(dev, part))
                    ex.lse_combine(fb.Tensor.from_torch(dev, part), fb.Tensor.from_torch(dev, out))
                dev.synchronize()
                worst = max(worst, float(np.abs(out.cpu().numpy() - want).max()))
                out.zero_()
            ex.close()  # collective: unmap, barrier, free
            # the library's communicator: all-reduce of a known tensor, then the head-sharded output projection
            comm = sharding.Communicator(dev, rank, world, timeout_ms=60000)
            t = torch.full((1000,), float(rank + 1), dtype=torch.float32, device=f"cuda:{rank}")
            comm.all_reduce_sum(fb.Tensor.from_torch(dev, t))
            dev.synchronize()
            assert float(t[0]) == world * (world + 1) / 2 and float(t[-1]) == world * (world + 1) / 2
            rng = np.random.default_rng(3)
            Bp, Hq_all, S, Dh, N = 1, 8, 256, 128, 256
            attn = W.bf16_round(rng.standard_normal((Bp, Hq_all, S, Dh)).astype(np.float32))
            wt = W.bf16_round((rng.standard_normal((N, Hq_all * Dh)) / 32).astype(np.float32))
            bias = rng.standard_normal(N).astype(np.float32)
            hq = Hq_all // world
            a_shard = np.ascontiguousarray(attn[:, rank * hq:(rank + 1) * hq])
            w_shard = np.ascontiguousarray(wt[:, rank * hq * Dh:(rank + 1) * hq * Dh])
            o = torch.empty((Bp, S, N), dtype=torch.float32, device=f"cuda:{rank}")
            comm.out_proj(fb.Tensor.from_slice(dev, a_shard.shape, a_shard, 1), fb.Tensor.from_slice(dev, w_shard.shape, w_shard, 1),
                          fb.Tensor.from_slice(dev, bias.shape, bias), fb.Tensor.from_torch(dev, o))
            dev.synchronize()
            comm.poll()
            worst_proj = float(np.abs(o.cpu().numpy() - O.out_proj(attn, wt, bias)).max())
            comm.close()
        t = torch.tensor([worst, worst_proj], dtype=torch.float64, device=f"cuda:{rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ret["err"] = float(t[0].item())
            ret["err_proj"] = float(t[1].item())
    finally:
        dist.destroy_process_group()


def test_kv_chunk_decode_over_peer_exchange_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["err"] <= 2e-3, dict(ret)
    assert ret["err_proj"] <= 4e-4, dict(ret)

