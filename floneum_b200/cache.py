"""KV cache and mask cache mirrors of fusor::cache for the attention path.

Reference: `AttentionMask` (fusor-ml/fusor/src/cache/attention_mask.rs:10-81), `MaskCache`
(mask_cache.rs:10-116), `KvCache` (kv_cache.rs:12-68) on `TensorCache` (tensor_cache.rs:9-124).
The reference keeps dense f32 K/V tensors and copies the whole valid cache on every append;
here `KvCache` sits on the paged bf16 cache of libfusor_cuda.so and `append` hands back views
that `Tensor.flash_attention` recognises, so a decode step reads the pages in place.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional, Tuple

import numpy as np

from . import _lib
from .device import Device
from .tensor import BF16, F32, MaskKind, Tensor

PAGE_TOKENS = 16
NEG_INF = float("-inf")


# ======================================================================================= masks
class AttentionMask:
    """Additive 0 / -inf mask.  Built by `causal` or by `MaskCache.get_mask` it also remembers its
    structure, so the attention kernels can apply it analytically instead of reading [Sq,Skv] floats."""

    def __init__(self, mask: Optional[Tensor] = None, *, device: Optional[Device] = None, structure=None):
        self._mask = mask
        self._device = device if device is not None else (mask.device if mask is not None else None)
        self._structure = structure  # ("causal", seq_len, offset) | ("sliding", seq_len, window, offset)

    @classmethod
    def new(cls, mask: Tensor) -> "AttentionMask":
        return cls(mask)

    @classmethod
    def causal(cls, device: Device, seq_len: int) -> "AttentionMask":
        """mask[i, j] = -inf if j > i else 0 (attention_mask.rs:26-46)."""
        return cls(device=device, structure=("causal", seq_len, 0))

    def host_values(self) -> np.ndarray:
        """The dense values this mask stands for (what the reference would have uploaded)."""
        if self._structure is None:
            return self._mask.as_slice()
        kind, seq_len = self._structure[0], self._structure[1]
        offset = self._structure[-1]
        i = np.arange(seq_len)[:, None]
        j = np.arange(seq_len)[None, :]
        if kind == "causal":
            bad = j > i
        else:
            w = self._structure[2]
            bad = (i < j) | (j + w <= i)
        base = np.where(bad, np.float32(NEG_INF), np.float32(0.0)).astype(np.float32)
        if offset > 0:  # left-pad with zero columns (mask_cache.rs:73-82)
            base = np.concatenate([np.zeros((seq_len, offset), np.float32), base], axis=1)
        return base

    def mask(self) -> Tensor:
        if self._mask is None:
            v = self.host_values()
            self._mask = Tensor.from_slice(self._device, v.shape, v)
        return self._mask

    def shape(self) -> Tuple[int, int]:
        if self._structure is not None:
            return (self._structure[1], self._structure[1] + self._structure[-1])
        return tuple(self._mask.shape())

    def analytic_kind(self, q_len: int, kv_len: int):
        """(mask_kind, window) of the C ABI when this mask equals an analytic one for [q_len, kv_len]."""
        s = self._structure
        if s is None or s[1] != q_len or s[1] + s[-1] != kv_len:
            return None
        if s[0] == "causal":
            return (_lib.MASK_CAUSAL, 0)
        return (_lib.MASK_SLIDING, s[2])


class MaskCache:
    """Memoised causal / sliding-window masks (mask_cache.rs:10-116)."""

    def __init__(self):
        self._masks = {}
        self._lock = threading.RLock()

    def get_mask(self, seq_len: int, seqlen_offset: int, sliding_window_size: Optional[int], device: Device) -> AttentionMask:
        if sliding_window_size is not None:
            seqlen_offset = min(seqlen_offset, max(sliding_window_size - seq_len, 0))
        key = (seq_len, sliding_window_size)
        with self._lock:
            base = self._masks.get(key)
            if base is None:
                if sliding_window_size is not None:
                    base = AttentionMask(device=device, structure=("sliding", seq_len, sliding_window_size, 0))
                else:
                    base = AttentionMask.causal(device, seq_len)
                self._masks[key] = base
        if seqlen_offset > 0:
            s = base._structure
            return AttentionMask(device=device, structure=s[:-1] + (seqlen_offset,))
        return base


# ======================================================================================= paged cache
class PagedKvCache:
    """Handle of a `fusor_cuda_kvcache`: bf16 pools [num_pages][Hkv][16][D] + page table + lengths."""

    def __init__(self, device: Device, max_batch: int, num_kv_heads: int, head_dim: int, num_pages: int,
                 max_pages_per_seq: int, page_tokens: int = PAGE_TOKENS):
        self.device = device
        self.max_batch, self.num_kv_heads, self.head_dim = max_batch, num_kv_heads, head_dim
        self.num_pages, self.max_pages_per_seq, self.page_tokens = num_pages, max_pages_per_seq, page_tokens
        self._L = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self._L.fusor_cuda_kvcache_create(device.handle, max_batch, num_kv_heads, head_dim, page_tokens,
                                                     num_pages, max_pages_per_seq, ctypes.byref(h)), device.handle)
        self._h = h

    def close(self):
        if getattr(self, "_h", None) and self.device.handle:
            self._L.fusor_cuda_kvcache_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc):
        _lib.check(rc, self.device.handle)

    def reset(self):
        self._ck(self._L.fusor_cuda_kvcache_reset(self._h))

    def append(self, k_new: Tensor, v_new: Tensor):
        ck, cv = k_new._c4(), v_new._c4()
        self._ck(self._L.fusor_cuda_kvcache_append(self._h, ctypes.byref(ck), ctypes.byref(cv)))

    def rope_append(self, q: Tensor, k_new: Tensor, v_new: Tensor, cos: Tensor, sin: Tensor, start_pos: int = -1,
                    interleaved: bool = False, out_dtype: Optional[int] = None) -> Tensor:
        """RoPE of q and k_new plus the append of (rotated k, v) in one kernel; returns rotated q.

        cos, sin: f32 device tensors [context, D/2].  start_pos < 0: each sequence's own length."""
        assert tuple(cos.shape()) == tuple(sin.shape()) and cos.shape()[1] == self.head_dim // 2
        assert cos.dtype == F32 and sin.dtype == F32 and cos.is_contiguous() and sin.is_contiguous()
        q_out = Tensor.empty(self.device, q.shape(), q.dtype if out_dtype is None else out_dtype)
        cq, ck, cv, co = q._c4(), k_new._c4(), v_new._c4(), q_out._c4()
        self._ck(self._L.fusor_cuda_kvcache_rope_append(self._h, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv),
                                                        cos.ptr, sin.ptr, cos.shape()[0], int(start_pos),
                                                        int(bool(interleaved)), ctypes.byref(co)))
        return q_out

    def truncate_front(self, b: int, keep: int):
        self._ck(self._L.fusor_cuda_kvcache_truncate_front(self._h, b, keep))

    def seq_len(self, b: int = 0) -> int:
        n = ctypes.c_int32()
        self._ck(self._L.fusor_cuda_kvcache_seq_len(self._h, b, ctypes.byref(n)))
        return n.value

    def set_page_table(self, page_table: np.ndarray, kv_len: np.ndarray):
        pt = np.ascontiguousarray(page_table, dtype=np.int32)
        kl = np.ascontiguousarray(kv_len, dtype=np.int32)
        assert pt.ndim == 2 and pt.shape[1] == self.max_pages_per_seq and kl.shape == (pt.shape[0],)
        i32p = ctypes.POINTER(ctypes.c_int32)
        self._ck(self._L.fusor_cuda_kvcache_set_page_table(self._h, pt.ctypes.data_as(i32p), kl.ctypes.data_as(i32p),
                                                           pt.shape[0]))

    def write_pages(self, first_page: int, k_bits: np.ndarray, v_bits: np.ndarray):
        """k_bits, v_bits: uint16 bf16 bit patterns [n_pages, Hkv, page_tokens, D]."""
        k_bits = np.ascontiguousarray(k_bits, dtype=np.uint16)
        v_bits = np.ascontiguousarray(v_bits, dtype=np.uint16)
        assert k_bits.shape[1:] == (self.num_kv_heads, self.page_tokens, self.head_dim) and v_bits.shape == k_bits.shape
        self._ck(self._L.fusor_cuda_kvcache_write_pages(self._h, first_page, k_bits.shape[0],
                                                        k_bits.ctypes.data_as(ctypes.c_void_p),
                                                        v_bits.ctypes.data_as(ctypes.c_void_p)))
        self.device.synchronize()

    def read_pages(self, first_page: int, n_pages: int):
        shape = (n_pages, self.num_kv_heads, self.page_tokens, self.head_dim)
        k, v = np.empty(shape, np.uint16), np.empty(shape, np.uint16)
        self._ck(self._L.fusor_cuda_kvcache_read_pages(self._h, first_page, n_pages, k.ctypes.data_as(ctypes.c_void_p),
                                                       v.ctypes.data_as(ctypes.c_void_p)))
        return k, v

    def pools(self) -> Tuple[int, int]:
        k, v = ctypes.c_void_p(), ctypes.c_void_p()
        self._ck(self._L.fusor_cuda_kvcache_pools(self._h, ctypes.byref(k), ctypes.byref(v)))
        return k.value, v.value

    def gather(self, batch: int, length: int, dtype: int = F32) -> Tuple[Tensor, Tensor]:
        shape = (batch, self.num_kv_heads, length, self.head_dim)
        k, v = Tensor.empty(self.device, shape, dtype), Tensor.empty(self.device, shape, dtype)
        ck, cv = k._c4(), v._c4()
        self._ck(self._L.fusor_cuda_kvcache_gather(self._h, ctypes.byref(ck), ctypes.byref(cv)))
        return k, v

    def set_decode_ctas(self, ctas: int):
        """Grid size of the decode kernel: 0 = automatic (from the number of cached pages), n > 0 = exactly n CTAs."""
        self._ck(self._L.fusor_cuda_kvcache_set_decode_ctas(self._h, int(ctas)))

    def decode(self, q: Tensor, scale: float, out: Optional[Tensor] = None, out_dtype: int = F32) -> Tensor:
        """q [B,Hq,1,D] -> out [B,Hq,1,D]."""
        if out is None:
            out = Tensor.empty(self.device, q.shape(), out_dtype)
        cq, co = q._c4(), out._c4()
        self._ck(self._L.fusor_cuda_flash_attention_decode(self.device.handle, self._h, ctypes.byref(cq),
                                                           ctypes.c_float(scale), ctypes.byref(co)))
        return out

    def decode_partial(self, q: Tensor, scale: float, partial: Optional[Tensor] = None) -> Tensor:
        """q [B,Hq,1,D] -> partial f32 [B,Hq,D+2] = {m, l, O[D]} over the keys this cache holds."""
        B, Hq, _, D = q.shape()
        if partial is None:
            partial = Tensor.empty(self.device, (B, Hq, D + 2), F32)
        cq = q._c4()
        self._ck(self._L.fusor_cuda_flash_attention_decode_partial(self.device.handle, self._h, ctypes.byref(cq),
                                                                   ctypes.c_float(scale), ctypes.c_void_p(partial.ptr)))
        return partial

    def decode_host(self, q: np.ndarray, scale: float, q_dtype: int = F32) -> np.ndarray:
        """Host-memory decode: q f32 numpy [B,Hq,1,D] (or bf16 bits when q_dtype is BF16) -> f32 numpy."""
        q = np.ascontiguousarray(q)
        out = np.empty(q.shape, np.float32)
        tq, to = _lib.Tensor4(), _lib.Tensor4()
        for t, a, dt in ((tq, q, q_dtype), (to, out, F32)):
            t.data = a.ctypes.data
            t.dtype = dt
            acc = 1
            for i in range(3, -1, -1):
                t.shape[i] = a.shape[i]
                t.stride[i] = acc
                acc *= a.shape[i]
        self._ck(self._L.fusor_cuda_flash_attention_decode_host(self.device.handle, self._h, ctypes.byref(tq),
                                                                ctypes.c_float(scale), ctypes.byref(to)))
        return out


def lse_combine(device: Device, parts: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """parts f32 [n_parts, rows..., D+2] -> out f32 [rows..., D] (log-sum-exp merge)."""
    shp = parts.shape()
    n_parts, D = shp[0], shp[-1] - 2
    n_rows = int(np.prod(shp[1:-1]))
    if out is None:
        out = Tensor.empty(device, tuple(shp[1:-1]) + (D,), F32)
    _lib.check(_lib.load().fusor_cuda_lse_combine(device.handle, ctypes.c_void_p(parts.ptr), n_parts, n_rows, D,
                                                  ctypes.c_void_p(out.ptr)), device.handle)
    return out


# ======================================================================================= KvCache mirror
class CachedKv:
    """What `KvCache.append` returns in place of the reference's dense K (or V) tensor."""

    def __init__(self, cache: "KvCache", which: str):
        self.cache, self.which = cache, which

    def shape(self):
        c = self.cache
        return (c._batch, c._num_kv_heads, c.current_seq_len(), c._head_dim)

    def to_tensor(self, dtype: int = F32) -> Tensor:
        k, v = self.cache._dense(dtype)
        return k if self.which == "k" else v

    def as_slice(self) -> np.ndarray:
        return self.to_tensor(F32).as_slice()


class KvCache:
    """Growable KV cache with the reference's interface (kv_cache.rs:24-67).

    `concat_dim` must be 2 (the sequence axis of [B, Hkv, S, D]), the value kalosm-llama uses
    (models/kalosm-llama/src/raw/cache.rs:26-39).  Past `max_sequence_len` the oldest rows are
    dropped, like TensorCache::append (tensor_cache.rs:55-78)."""

    def __init__(self, concat_dim: int, max_sequence_len: int):
        if concat_dim != 2:
            raise _lib.FusorCudaError(_lib.UNSUPPORTED, "KvCache concatenates along axis 2 of [B, Hkv, S, D] only")
        self.concat_dim = concat_dim
        self.max_sequence_len = max_sequence_len
        self._paged: Optional[PagedKvCache] = None
        self._batch = self._num_kv_heads = self._head_dim = 0

    @classmethod
    def new(cls, concat_dim: int, max_sequence_len: int) -> "KvCache":
        return cls(concat_dim, max_sequence_len)

    def current_seq_len(self) -> int:
        return self._paged.seq_len(0) if self._paged is not None and self._batch else 0

    def reset(self):
        if self._paged is not None:
            self._paged.reset()
        self._batch = 0

    def k(self) -> Optional[CachedKv]:
        return CachedKv(self, "k") if self.current_seq_len() else None

    def v(self) -> Optional[CachedKv]:
        return CachedKv(self, "v") if self.current_seq_len() else None

    def _make_room(self, device: Device, k: Tensor, v: Tensor):
        """Allocation on first use and the eviction rule of TensorCache::append; returns (k, v, rows dropped from the
        front of the new tensors)."""
        B, Hkv, n, D = k.shape()
        assert tuple(v.shape()) == (B, Hkv, n, D), "k and v shapes differ"
        if self._paged is None or B > self._paged.max_batch or (self._num_kv_heads, self._head_dim) != (Hkv, D):
            pages_per_seq = (self.max_sequence_len + PAGE_TOKENS - 1) // PAGE_TOKENS + 1
            self._paged = PagedKvCache(device, B, Hkv, D, B * pages_per_seq, pages_per_seq)
            self._num_kv_heads, self._head_dim = Hkv, D
        mx = self.max_sequence_len
        skip = 0
        if n >= mx:  # only the newest max_sequence_len rows survive
            self._paged.reset()
            skip = n - mx
            k = Tensor(device, k.ptr + skip * k.strides[2] * (4 if k.dtype == F32 else 2), (B, Hkv, mx, D), k.dtype, k.strides, owner=k)
            v = Tensor(device, v.ptr + skip * v.strides[2] * (4 if v.dtype == F32 else 2), (B, Hkv, mx, D), v.dtype, v.strides, owner=v)
        elif self.current_seq_len() + n > mx:
            for b in range(B):
                self._paged.truncate_front(b, mx - n)
        return k, v, skip

    def append(self, device: Device, k: Tensor, v: Tensor) -> Tuple[CachedKv, CachedKv]:
        k, v, _ = self._make_room(device, k, v)
        self._paged.append(k, v)
        self._batch = k.shape()[0]
        return CachedKv(self, "k"), CachedKv(self, "v")

    def _append_rotated(self, rope_cache, q: Tensor, k: Tensor, v: Tensor, start_pos: int, interleaved: bool, out_dtype):
        """`RopeCache.forward(q, k, start_pos)` then `append(k, v)` in one launch (see RopeCache.forward_append)."""
        if start_pos < 0:
            start_pos = self.current_seq_len()
        n = k.shape()[2]
        k2, v2, skip = self._make_room(q.device, k, v)
        if skip:  # the rows that do not survive still rotate q; do that with the plain op and append the rest
            from .rope import rope
            q_rot = rope(q, rope_cache.cos, rope_cache.sin, start_pos, interleaved, out_dtype)
            dummy = Tensor(q.device, q.ptr + skip * q.strides[2] * (4 if q.dtype == F32 else 2),
                           (q.shape()[0], q.shape()[1], n - skip, q.shape()[3]), q.dtype, q.strides, owner=q)
            self._paged.rope_append(dummy, k2, v2, rope_cache.cos, rope_cache.sin, start_pos + skip, interleaved, out_dtype)
        else:
            q_rot = self._paged.rope_append(q, k2, v2, rope_cache.cos, rope_cache.sin, start_pos, interleaved, out_dtype)
        self._batch = k.shape()[0]
        return q_rot, CachedKv(self, "k"), CachedKv(self, "v")

    # ------------------------------------------------------------------ session export / import
    def export_session(self) -> dict:
        """The cache as host arrays: {"k", "v": f32 [B, Hkv, len, D], "max_sequence_len"} (what the reference's session
        save would hold, models/kalosm-llama/src/session.rs:51-69, where it is stubbed out).  Values are the bf16-rounded
        rows the pages hold; an empty cache exports zero-length arrays."""
        n = self.current_seq_len()
        if n == 0:
            z = np.zeros((self._batch, self._num_kv_heads, 0, self._head_dim), np.float32)
            return {"k": z, "v": z.copy(), "max_sequence_len": self.max_sequence_len}
        k, v = self._dense(F32)
        return {"k": k.as_slice(), "v": v.as_slice(), "max_sequence_len": self.max_sequence_len}

    @classmethod
    def import_session(cls, device: Device, session: dict) -> "KvCache":
        """Rebuilds a cache from `export_session`'s dictionary (dense rows go back into pages through `append`)."""
        cache = cls(2, int(session["max_sequence_len"]))
        k, v = np.asarray(session["k"], np.float32), np.asarray(session["v"], np.float32)
        assert k.shape == v.shape and k.ndim == 4, "session k and v must be [B, Hkv, len, D] arrays of one shape"
        if k.shape[2] > 0:
            cache.append(device, Tensor.from_slice(device, k.shape, k), Tensor.from_slice(device, v.shape, v))
        return cache

    def _dense(self, dtype: int) -> Tuple[Tensor, Tensor]:
        return self._paged.gather(self._batch, self.current_seq_len(), dtype)

    def _attend(self, q: Tensor, scale: float, mask, out_dtype: int) -> Tensor:
        B, Hq, Sq, D = q.shape()
        kv_len = self.current_seq_len()
        zero_mask = mask is None
        if mask is not None:
            m, mk = mask
            if isinstance(m, AttentionMask) and mk is MaskKind.QKMask:
                a = m.analytic_kind(Sq, kv_len)
                zero_mask = Sq == 1 and a is not None and a[0] == _lib.MASK_CAUSAL
        if Sq == 1 and zero_mask:
            return self._paged.decode(q, scale, out_dtype=out_dtype)
        kd, vd = self._dense(BF16)
        return q.to_bf16().flash_attention(kd, vd, scale, mask, out_dtype)


class LlamaCache:
    """One `KvCache` per layer (models/kalosm-llama/src/raw/cache.rs:14-54), concatenating along axis 2.

    With a sliding-window model (`sliding_window_type` and `sliding_window_size` both given) layer i keeps
    `sliding_window_size` tokens unless (i + 1) % sliding_window_type == 0; those layers, and every layer of a model
    without a window, keep `context_length` tokens.  The layer loop hands `blocks[i]` to layer i
    (models/kalosm-llama/src/raw/mod.rs:614-627)."""

    CONCAT_DIMENSION = 2

    def __init__(self, n_layer: int, context_length: int, sliding_window_type: Optional[int] = None,
                 sliding_window_size: Optional[int] = None):
        self.start_time = 0
        self.tokens: list = []
        self.blocks = [KvCache(self.CONCAT_DIMENSION, self.layer_max_seq_len(i, context_length, sliding_window_type,
                                                                             sliding_window_size))
                       for i in range(n_layer)]

    new = classmethod(lambda cls, *a, **kw: cls(*a, **kw))

    @staticmethod
    def layer_max_seq_len(layer_idx: int, context_length: int, sliding_window_type: Optional[int],
                          sliding_window_size: Optional[int]) -> int:
        if sliding_window_type is not None and sliding_window_size is not None:
            if (layer_idx + 1) % sliding_window_type != 0:
                return sliding_window_size
        return context_length

    def clear(self):
        for block in self.blocks:
            block.reset()
