"""Rotary position embedding behind fusor's names: `RopeCache` and the `Tensor` rope ops.

Reference: fusor-ml/fusor/src/composite/rope.rs — `Tensor::rope` (:38-68), `rope_interleaved` (:70-118),
`RopeCache::new / from_parts / forward / forward_interleaved` (:186-265) — and the llama call site
models/kalosm-llama/src/raw/rope.rs:86-111.  `RopeCache.forward_append` is the fused form of
"rope(q, k) then KvCache.append(k, v)": one kernel rotates q, rotates k into the bf16 pages and copies v there.
All arithmetic runs in libfusor_cuda.so.
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import numpy as np

from . import _lib
from .device import Device
from .tensor import F32, Tensor


def base_inverse_frequency(dim: int, rope_theta: float) -> np.ndarray:
    """`1 / theta^(i/dim)` for i = 0, 2, .. dim-2 in f32 (rope.rs:189-194)."""
    theta = np.float32(rope_theta)
    return np.array([np.float32(1.0) / theta ** (np.float32(i) / np.float32(dim)) for i in range(0, dim, 2)],
                    dtype=np.float32)


def rope(x: Tensor, cos: Tensor, sin: Tensor, start_pos: int = 0, interleaved: bool = False,
         out_dtype: int | None = None) -> Tensor:
    """x [B,H,n,D] rotated with rows start_pos .. start_pos+n of cos/sin [context, D/2] (f32 device tensors)."""
    shape = x.shape()
    assert len(shape) == 4, "rope expects [batch, heads, sequence, head_dim]"
    assert shape[3] % 2 == 0, "head_dim must be even"
    cs, ss = cos.shape(), sin.shape()
    assert tuple(cs) == tuple(ss) and len(cs) == 2 and cs[1] == shape[3] // 2, (
        f"cos/sin shape {list(cs)} / {list(ss)} does not match [context, {shape[3] // 2}]")
    assert cos.dtype == F32 and sin.dtype == F32 and cos.is_contiguous() and sin.is_contiguous()
    dev = x.device
    out = Tensor.empty(dev, shape, x.dtype if out_dtype is None else out_dtype)
    cx, co = x._c4(), out._c4()
    _lib.check(_lib.load().fusor_cuda_rope(dev.handle, ctypes.byref(cx), cos.ptr, sin.ptr, cs[0], int(start_pos),
                                           int(bool(interleaved)), ctypes.byref(co)), dev.handle)
    return out


class RopeCache:
    """cos / sin tables [context_length, head_dim/2] on the device (rope.rs:180-265)."""

    def __init__(self, cos: Tensor, sin: Tensor):
        assert tuple(cos.shape()) == tuple(sin.shape()) and len(cos.shape()) == 2
        self.cos, self.sin = cos, sin

    @classmethod
    def new(cls, head_dim: int, context_length: int, rope_theta: float, device: Device) -> "RopeCache":
        inv = base_inverse_frequency(head_dim, rope_theta)
        outer = np.arange(context_length, dtype=np.float32)[:, None] * inv[None, :]
        shape = (context_length, head_dim // 2)
        return cls(Tensor.from_slice(device, shape, np.cos(outer).astype(np.float32)),
                   Tensor.from_slice(device, shape, np.sin(outer).astype(np.float32)))

    @classmethod
    def from_parts(cls, cos: Tensor, sin: Tensor) -> "RopeCache":
        return cls(cos, sin)

    def forward(self, q: Tensor, k: Tensor, start_pos: int) -> Tuple[Tensor, Tensor]:
        return (rope(q, self.cos, self.sin, start_pos, False), rope(k, self.cos, self.sin, start_pos, False))

    def forward_interleaved(self, q: Tensor, k: Tensor, start_pos: int) -> Tuple[Tensor, Tensor]:
        return (rope(q, self.cos, self.sin, start_pos, True), rope(k, self.cos, self.sin, start_pos, True))

    def forward_append(self, q: Tensor, k: Tensor, v: Tensor, cache, start_pos: int = -1, interleaved: bool = False,
                       out_dtype: int | None = None):
        """Rotates q, rotates k into `cache` and appends v, in one launch.

        `cache` is a `KvCache` (returns `(q_rotated, cached_k, cached_v)`) or a `PagedKvCache` (returns q_rotated).
        start_pos < 0 positions every sequence at its own cache length."""
        from .cache import KvCache

        if isinstance(cache, KvCache):
            return cache._append_rotated(self, q, k, v, start_pos, interleaved, out_dtype)
        return cache.rope_append(q, k, v, self.cos, self.sin, start_pos, interleaved, out_dtype)
