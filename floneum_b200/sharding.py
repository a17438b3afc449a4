"""Multi-GPU partitioning of the attention path: one process per GPU.

Two partitions, both defined by the benchmark configurations (the reference has no multi-GPU code):
  * KV heads (prefill and batched decode): rank r owns kv heads [r*Hkv/N, (r+1)*Hkv/N) and the query
    heads that read them.  Inputs arrive sharded, outputs stay sharded: no collective.
  * KV-sequence chunks (long-context decode): rank r owns keys [r*Skv/N, (r+1)*Skv/N); each rank emits
    a partial {m, l, O} per query head, the partials are all-gathered (NCCL over NVLink on GPUs, gloo in
    the CPU tests) and merged by log-sum-exp on every rank.
The output projection that follows head-sharded attention is the one place the head partition needs a collective: rank r
multiplies its heads by columns [q0*D, q1*D) of the weight and the partial sums are all-reduced (`out_proj_all_reduce`).
"""
from __future__ import annotations

from typing import Tuple


def kv_head_range(num_kv_heads: int, rank: int, world: int) -> Tuple[int, int]:
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} kv heads do not split evenly over {world} ranks")
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per


def q_head_range(num_q_heads: int, num_kv_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """Query heads that read the kv heads of `rank` (query head h reads kv head h // (Hq/Hkv))."""
    if num_q_heads % num_kv_heads != 0:
        raise ValueError(f"Number of Q heads ({num_q_heads}) must be divisible by number of K/V heads ({num_kv_heads})")
    g = num_q_heads // num_kv_heads
    lo, hi = kv_head_range(num_kv_heads, rank, world)
    return lo * g, hi * g


def kv_chunk_range(kv_len: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous key range of `rank`; ranges tile [0, kv_len) and differ in size by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    return rank * kv_len // world, (rank + 1) * kv_len // world


def all_gather_partials(partial, group=None):
    """partial: torch tensor [rows..., D+2] on this rank -> [world, rows..., D+2] on every rank."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(partial.shape), dtype=partial.dtype, device=partial.device)
    if partial.is_cuda:
        dist.all_gather_into_tensor(out, partial.contiguous(), group=group)
    else:
        chunks = list(out.unbind(0))
        dist.all_gather(chunks, partial.contiguous(), group=group)
    return out


class PeerExchange:
    """This rank's end of the peer-memory record exchange (`fusor_cuda_exchange_*`): every rank's buffer is mapped into
    every other rank's address space once (handles travel through torch.distributed), after which a step's records
    move as peer stores inside the library's own kernels, with no collective call."""

    def __init__(self, device, rank: int, world: int, slot_floats: int, group=None):
        import ctypes
        from . import _lib
        self.device, self.rank, self.world = device, rank, world
        self._L = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self._L.fusor_cuda_exchange_create(device.handle, world, rank, (slot_floats + 3) // 4 * 4, ctypes.byref(h)),
                   device.handle)
        self._h = h
        if world > 1:
            import torch
            import torch.distributed as dist
            mine = ctypes.create_string_buffer(64)
            _lib.check(self._L.fusor_cuda_exchange_handle(self._h, mine), device.handle)
            t = torch.frombuffer(bytearray(mine.raw), dtype=torch.uint8).to(f"cuda:{device.ordinal}")
            allh = torch.empty(world * 64, dtype=torch.uint8, device=t.device)
            dist.all_gather_into_tensor(allh, t, group=group)
            blob = bytes(allh.cpu().numpy().tobytes())
            _lib.check(self._L.fusor_cuda_exchange_connect(self._h, blob), device.handle)
            dist.barrier(group=group)  # nobody pushes before everybody has mapped

    def lse_combine(self, records, out):
        """records: Tensor f32 [rows..., D+2] of this rank; out: Tensor f32 [rows..., D].  Collective."""
        from . import _lib
        shape = records.shape()
        d = shape[-1] - 2
        n_rows = 1
        for x in shape[:-1]:
            n_rows *= x
        _lib.check(self._L.fusor_cuda_exchange_lse_combine(self._h, records.ptr, n_rows, d, out.ptr), self.device.handle)
        return out

    def decode(self, cache, q, scale: float, out):
        """KV-chunk decode: `cache` holds this rank's chunk of the keys, `q` [B,Hq,1,D] is the same on every rank,
        out f32 [B,Hq,D] receives the attention over all ranks' keys.  Collective, two launches."""
        import ctypes
        from . import _lib
        cq = q._c4()
        _lib.check(self._L.fusor_cuda_exchange_decode(self._h, cache._h, ctypes.byref(cq), ctypes.c_float(scale), out.ptr),
                   self.device.handle)
        return out

    def close(self, group=None):
        """Collective teardown in two phases: every rank unmaps the other ranks' buffers, the ranks meet, and only then
        does each free its own (freeing an exported buffer that a peer still has mapped is undefined in CUDA)."""
        if getattr(self, "_h", None) and self.device.handle:
            self._L.fusor_cuda_exchange_disconnect(self._h)
            if self.world > 1:
                import torch.distributed as dist
                if dist.is_available() and dist.is_initialized():
                    dist.barrier(group=group)
            self._L.fusor_cuda_exchange_destroy(self._h)
        self._h = None

    def __del__(self):
        # no collective from a finaliser: a rank that forgot close() only unmaps its peers; its own buffer stays
        # allocated until the process ends, when no peer can still be mapped to freed memory
        try:
            if getattr(self, "_h", None) and self.device.handle:
                self._L.fusor_cuda_exchange_disconnect(self._h)
        except Exception:
            pass


def decode_kv_chunks(device, cache, q, scale: float, group=None):
    """Long-context decode over KV chunks: local split-KV partial -> all-gather -> log-sum-exp merge.

    `cache` holds this rank's chunk of the keys, `q` [B,Hq,1,D] is replicated.  Returns a torch tensor
    [B,Hq,D] f32 on this rank's GPU (every rank gets the full result).  The collective runs on torch's current
    stream, which must be the stream the Device was created on."""
    import torch
    from .cache import lse_combine
    from .tensor import F32, Tensor
    B, Hq, _, D = q.shape()
    partial = torch.empty((B, Hq, D + 2), dtype=torch.float32, device=f"cuda:{device.ordinal}")
    cache.decode_partial(q, scale, Tensor.from_torch(device, partial))
    gathered = all_gather_partials(partial, group)
    out = torch.empty((B, Hq, D), dtype=torch.float32, device=partial.device)
    lse_combine(device, Tensor.from_torch(device, gathered), Tensor.from_torch(device, out))
    return out


def out_proj_weight_columns(num_q_heads: int, num_kv_heads: int, head_dim: int, rank: int, world: int) -> Tuple[int, int]:
    """Columns of the [out_features, Hq*D] projection weight that multiply the query heads of `rank`."""
    q0, q1 = q_head_range(num_q_heads, num_kv_heads, rank, world)
    return q0 * head_dim, q1 * head_dim


class Communicator:
    """The library's own communicator (`fusor_cuda_comm_*`): NCCL behind the C ABI, initialised without blocking and
    polled against a host deadline, so that a rank that never joins ends in a TIMEOUT error instead of a hang.
    The 128-byte id is made on rank 0 and reaches the others through `broadcast_bytes` (default: torch.distributed's
    object broadcast, which works on the gloo backend too)."""

    def __init__(self, device, rank: int, world: int, timeout_ms: int = 30000, unique_id: bytes | None = None, group=None):
        import ctypes
        from . import _lib
        self.device, self.rank, self.world = device, rank, world
        self._L = _lib.load()
        if unique_id is None:
            import torch.distributed as dist
            box = [self.make_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0, group=group)
            unique_id = box[0]
        assert len(unique_id) == 128
        h = ctypes.c_void_p()
        _lib.check(self._L.fusor_cuda_comm_init(device.handle, unique_id, rank, world, int(timeout_ms), ctypes.byref(h)),
                   device.handle)
        self._h = h

    @staticmethod
    def make_unique_id() -> bytes:
        import ctypes
        from . import _lib
        buf = ctypes.create_string_buffer(128)
        _lib.check(_lib.load().fusor_cuda_comm_unique_id(buf), None)
        return bytes(buf.raw)

    def poll(self):
        from . import _lib
        _lib.check(self._L.fusor_cuda_comm_poll(self._h), self.device.handle)

    def all_reduce_sum(self, t):
        """In-place sum over the ranks of a contiguous library Tensor, on the device's stream."""
        from . import _lib
        assert t.is_contiguous()
        _lib.check(self._L.fusor_cuda_comm_all_reduce_sum(self._h, t.ptr, t.numel(), t.dtype), self.device.handle)
        return t

    def out_proj(self, attn, weight_shard, bias, out):
        """This rank's heads x weight columns, then the sum over ranks, in one library call.  attn [B, Hq/N, S, D] bf16,
        weight_shard [out, Hq/N * D] bf16, bias f32 [out] or None (used on rank 0), out [B, S, out] contiguous."""
        import ctypes
        from . import _lib
        from .tensor import Tensor
        B, _, S, _ = attn.shape()
        ws = weight_shard.shape()
        w4 = Tensor(self.device, weight_shard.ptr, (1, 1, ws[0], ws[1]), weight_shard.dtype,
                    (ws[0] * weight_shard.strides[0], ws[0] * weight_shard.strides[0], weight_shard.strides[0], weight_shard.strides[1]),
                    owner=weight_shard)
        o4 = Tensor(self.device, out.ptr, (B, 1, S, ws[0]), out.dtype, (S * ws[0], S * ws[0], ws[0], 1), owner=out)
        ca, cw, co = attn._c4(), w4._c4(), o4._c4()
        _lib.check(self._L.fusor_cuda_attention_out_proj_all_reduce(self.device.handle, self._h, ctypes.byref(ca), ctypes.byref(cw),
                                                                    bias.ptr if bias is not None else None, ctypes.byref(co)),
                   self.device.handle)
        return out

    def abort(self):
        if getattr(self, "_h", None):
            self._L.fusor_cuda_comm_abort(self._h)

    def close(self):
        if getattr(self, "_h", None) and self.device.handle:
            self._L.fusor_cuda_comm_destroy(self._h)
        self._h = None


def all_reduce_sum(t, group=None):
    """In-place sum over ranks of a torch tensor (NCCL on GPUs, gloo in the CPU tests)."""
    import torch.distributed as dist
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def out_proj_all_reduce(device, attn, weight_shard, bias, rank: int, group=None):
    """Tensor-parallel output projection: attn [B, Hq/N, S, D] (this rank's heads, bf16), weight_shard [out, Hq/N * D]
    (this rank's columns), bias f32 [out] or None (added on rank 0 only) -> torch f32 [B, S, out], summed over ranks.
    The collective runs on torch's current stream, which must be the stream the Device was created on."""
    import torch
    from .tensor import Tensor
    B, _, S, _ = attn.shape()
    n_out = weight_shard.shape()[0]
    out = torch.empty((B, S, n_out), dtype=torch.float32, device=f"cuda:{device.ordinal}")
    attn.out_proj(weight_shard, bias if rank == 0 else None, out=Tensor.from_torch(device, out))
    return all_reduce_sum(out, group)
