"""Device tensors and `Tensor.flash_attention`, mirroring fusor's API for the attention path.

Reference: `fusor::Tensor` (fusor-ml/fusor/src/lib.rs:125-129), construction from host
data (fusor-ml/fusor/src/composite/construction.rs:100-122), readback `as_slice`
(fusor-ml/fusor/src/lib.rs:391-403) and
`Tensor::<4>::flash_attention(&self, k, v, scale, mask)`
(fusor-ml/fusor/src/composite/flash_attention.rs:52-73).  Misuse the reference answers
with assert!/panic! raises here (AssertionError for shape asserts, FusorCudaError for the
rest).  All arithmetic happens in libfusor_cuda.so.
"""
from __future__ import annotations

import ctypes
import enum
from typing import Optional, Sequence, Tuple

import numpy as np

from . import _lib
from .device import Device

F32, BF16, F16 = _lib.F32, _lib.BF16, _lib.F16
_ITEMSIZE = {F32: 4, BF16: 2, F16: 2}


class MaskKind(enum.Enum):
    """How a 2-D mask is laid out (fusor-ml/fusor/src/composite/flash_attention.rs:10-19)."""
    QKMask = 1        # [q_seq_len, kv_seq_len], same for every (batch, head)
    BatchKeyMask = 2  # [batch, kv_seq_len], broadcast over heads and queries


def _to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def _from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def _host_bits(a: np.ndarray, dtype: int) -> np.ndarray:
    """f32 host values -> the array that is uploaded for `dtype` (f16: numpy's own round-to-nearest-even)."""
    if dtype == F32:
        return a
    return _to_bf16_bits(a) if dtype == BF16 else np.ascontiguousarray(a.astype(np.float16)).view(np.uint16)


class Tensor:
    """A strided view of device memory: shape, element strides, dtype (f32, bf16 or f16)."""

    def __init__(self, device: Device, ptr: int, shape: Sequence[int], dtype: int = F32,
                 strides: Optional[Sequence[int]] = None, owner=None, owns: bool = False):
        self.device = device
        self.ptr = int(ptr)
        self._shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        if strides is None:
            strides, acc = [], 1
            for s in reversed(self._shape):
                strides.append(acc)
                acc *= s
            strides = tuple(reversed(strides))
        self.strides = tuple(int(s) for s in strides)
        self._owner = owner  # keeps a borrowed allocation (e.g. a torch tensor) alive
        self._owns = owns

    # ------------------------------------------------------------------ construction / readback
    @classmethod
    def empty(cls, device: Device, shape: Sequence[int], dtype: int = F32) -> "Tensor":
        n = int(np.prod(shape)) if len(shape) else 1
        ptr = device.alloc(max(n, 1) * _ITEMSIZE[dtype])
        return cls(device, ptr, shape, dtype, owns=True)

    @classmethod
    def from_slice(cls, device: Device, shape: Sequence[int], data, dtype: int = F32) -> "Tensor":
        """Upload host data (any array-like of floats) as a contiguous tensor of `shape`."""
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(shape))
        host = _host_bits(a, dtype)
        t = cls.empty(device, shape, dtype)
        L = _lib.load()
        _lib.check(L.fusor_cuda_buffer_upload(device.handle, ctypes.c_void_p(t.ptr), host.ctypes.data_as(ctypes.c_void_p),
                                              host.nbytes), device.handle)
        device.synchronize()  # `host` may be a temporary
        return t

    new = from_slice

    @classmethod
    def from_torch(cls, device: Device, t) -> "Tensor":
        """Borrow a CUDA torch tensor (float32, bfloat16 or float16) without copying."""
        import torch
        dt = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}[t.dtype]
        return cls(device, t.data_ptr(), tuple(t.shape), dt, tuple(t.stride()), owner=t)

    @classmethod
    def zeros(cls, device: Device, shape: Sequence[int], dtype: int = F32) -> "Tensor":
        return cls.from_slice(device, shape, np.zeros(shape, np.float32), dtype)

    def shape(self) -> Tuple[int, ...]:
        return self._shape

    def is_contiguous(self) -> bool:
        acc = 1
        for s, st in zip(reversed(self._shape), reversed(self.strides)):
            if s != 1 and st != acc:
                return False
            acc *= s
        return True

    def numel(self) -> int:
        return int(np.prod(self._shape)) if self._shape else 1

    def as_slice(self) -> np.ndarray:
        """Read back as a float32 numpy array indexable like the reference's TensorSlice."""
        assert self.is_contiguous(), "as_slice needs a contiguous tensor"
        host = np.empty(self._shape, np.float32 if self.dtype == F32 else np.uint16)
        L = _lib.load()
        _lib.check(L.fusor_cuda_buffer_download(self.device.handle, host.ctypes.data_as(ctypes.c_void_p),
                                                ctypes.c_void_p(self.ptr), host.nbytes), self.device.handle)
        self.device.synchronize()
        if self.dtype == F32:
            return host
        if self.dtype == F16:
            return host.view(np.float16).astype(np.float32)
        return _from_bf16_bits(host).reshape(self._shape)

    def cast(self, dtype: int) -> "Tensor":
        assert self.is_contiguous()
        out = Tensor.empty(self.device, self._shape, dtype)
        _lib.check(_lib.load().fusor_cuda_cast(self.device.handle, ctypes.c_void_p(out.ptr), dtype, ctypes.c_void_p(self.ptr),
                                               self.dtype, self.numel()), self.device.handle)
        return out

    def to_bf16(self) -> "Tensor":
        return self if self.dtype == BF16 else self.cast(BF16)

    def to_f32(self) -> "Tensor":
        return self if self.dtype == F32 else self.cast(F32)

    def __del__(self):
        try:
            if self._owns and self.ptr and self.device is not None and self.device.handle:
                self.device.free(self.ptr)
        except Exception:
            pass

    # ------------------------------------------------------------------ C views
    def _c4(self) -> _lib.Tensor4:
        assert len(self._shape) == 4, f"expected a rank-4 tensor, got shape {self._shape}"
        t = _lib.Tensor4()
        t.data = self.ptr
        t.dtype = self.dtype
        for i in range(4):
            t.shape[i] = self._shape[i]
            t.stride[i] = self.strides[i]
        return t

    def _c2(self) -> _lib.Tensor2:
        assert len(self._shape) == 2 and self.dtype == F32, "masks are rank-2 f32 tensors"
        t = _lib.Tensor2()
        t.data = self.ptr
        for i in range(2):
            t.shape[i] = self._shape[i]
            t.stride[i] = self.strides[i]
        return t

    # ------------------------------------------------------------------ output projection
    def out_proj(self, weight: "Tensor", bias: Optional["Tensor"] = None, out_dtype: int = F32,
                 out: Optional["Tensor"] = None) -> "Tensor":
        """self = attention output [B,Hq,S,D] (bf16) -> [B,S,N]: the layer's `transpose(1, 2).reshape(..)` followed by
        `Linear::forward` with a dense bf16 weight [N, Hq*D] and an optional f32 bias [N]
        (models/kalosm-llama/src/raw/attention_layer.rs:450-454; fusor-ml/fusor/src/layers/linear.rs:72-115)."""
        B, Hq, S, D = self._shape
        ws = weight.shape()
        assert len(ws) == 2 and ws[1] == Hq * D, f"weight shape {list(ws)} does not match [out_features, {Hq * D}]"
        if bias is not None:
            assert tuple(bias.shape()) == (ws[0],) and bias.dtype == F32, "bias must be f32 [out_features]"
        if out is None:
            out = Tensor.empty(self.device, (B, S, ws[0]), out_dtype)
        assert tuple(out.shape()) == (B, S, ws[0]) and out.is_contiguous(), "out must be a contiguous [B, S, out_features]"
        out_dtype = out.dtype
        w4 = Tensor(self.device, weight.ptr, (1, 1, ws[0], ws[1]), weight.dtype,
                    (ws[0] * weight.strides[0], ws[0] * weight.strides[0], weight.strides[0], weight.strides[1]), owner=weight)
        o4 = Tensor(self.device, out.ptr, (B, 1, S, ws[0]), out_dtype, (S * ws[0], S * ws[0], ws[0], 1), owner=out)
        ca, cw, co = self._c4(), w4._c4(), o4._c4()
        _lib.check(_lib.load().fusor_cuda_attention_out_proj(self.device.handle, ctypes.byref(ca), ctypes.byref(cw),
                                                             bias.ptr if bias is not None else None, ctypes.byref(co)),
                   self.device.handle)
        return out

    # ------------------------------------------------------------------ rotary embedding
    def rope(self, cos: "Tensor", sin: "Tensor") -> "Tensor":
        """Tensor::rope (fusor-ml/fusor/src/composite/rope.rs:38-68): halves (i, i + D/2); cos/sin [seq, D/2]."""
        from .rope import rope
        return rope(self, cos, sin, 0, False)

    def rope_interleaved(self, cos: "Tensor", sin: "Tensor") -> "Tensor":
        """Tensor::rope_interleaved (rope.rs:70-118): adjacent pairs (2i, 2i+1)."""
        from .rope import rope
        return rope(self, cos, sin, 0, True)

    rope_normal_fused = rope          # rope.rs:158-175
    rope_fused = rope_interleaved     # rope.rs:140-156

    # ------------------------------------------------------------------ the operator
    def flash_attention(self, k, v, scale: float, mask=None, out_dtype: int = F32) -> "Tensor":
        """softmax(q k^T * scale + mask) v with GQA; self is q [B,Hq,Sq,D].

        `k`, `v`: tensors [B,Hkv,Skv,D], or the views a `KvCache.append` returned.
        `mask`: None, or `(mask, MaskKind)` where mask is a rank-2 Tensor or an `AttentionMask`
        (an AttentionMask that knows it is causal / sliding-window is applied analytically).
        """
        from .cache import AttentionMask, CachedKv  # circular

        L = _lib.load()
        dev = self.device
        if isinstance(k, CachedKv) or isinstance(v, CachedKv):
            assert isinstance(k, CachedKv) and isinstance(v, CachedKv) and k.cache is v.cache, \
                "k and v must come from the same KvCache"
            return k.cache._attend(self, scale, mask, out_dtype)

        q_shape, k_shape = self._shape, k.shape()
        assert len(q_shape) == 4 and len(k_shape) == 4
        num_heads, num_kv_heads = q_shape[1], k_shape[1]
        assert num_heads % num_kv_heads == 0, (
            f"Number of Q heads ({num_heads}) must be divisible by number of K/V heads ({num_kv_heads})")
        kind, window, mask_t = _lib.MASK_NONE, 0, None
        if mask is not None:
            m, mk = mask
            if isinstance(m, AttentionMask):
                analytic = m.analytic_kind(q_shape[2], k_shape[2]) if mk is MaskKind.QKMask else None
                if analytic is not None:
                    kind, window = analytic
                else:
                    mask_t = m.mask()
            else:
                mask_t = m
            if mask_t is not None:
                if mask_t.device is not dev:
                    raise _lib.FusorCudaError(_lib.INVALID_ARGUMENT, "Mask must be on the same device as other tensors")
                kind = _lib.MASK_QK if mk is MaskKind.QKMask else _lib.MASK_BATCH_KEY
                exp = [q_shape[2], k_shape[2]] if mk is MaskKind.QKMask else [q_shape[0], k_shape[2]]
                assert list(mask_t.shape()) == exp, (
                    f"{mk.name} shape {list(mask_t.shape())} does not match expected {exp}")
        out = Tensor.empty(dev, q_shape, out_dtype)
        cq, ck, cv, co = self._c4(), k._c4(), v._c4(), out._c4()
        cm = mask_t._c2() if mask_t is not None else None
        rc = L.fusor_cuda_flash_attention(dev.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv),
                                          ctypes.c_float(scale), ctypes.byref(cm) if cm is not None else None, kind,
                                          window, ctypes.byref(co))
        _lib.check(rc, dev.handle)
        return out
