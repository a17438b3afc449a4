"""Device handle: one CUDA context object of libfusor_cuda.so per GPU.

Mirrors fusor::Device (fusor-ml/fusor/src/device.rs:7-13).  Only the Gpu variant exists here:
this package is the GPU arm of the attention path and has no CPU implementation.
"""
from __future__ import annotations

import ctypes

from . import _lib


class Device:
    def __init__(self, ordinal: int = 0, stream: int | None = None):
        L = _lib.load()
        h = ctypes.c_void_p()
        rc = L.fusor_cuda_ctx_create(ordinal, ctypes.c_void_p(stream) if stream else None, ctypes.byref(h))
        _lib.check(rc, None)
        self._h = h
        self.ordinal = ordinal
        self._L = L

    @classmethod
    def gpu(cls, ordinal: int = 0, stream: int | None = None) -> "Device":
        return cls(ordinal, stream)

    @classmethod
    def cpu(cls):
        raise _lib.FusorCudaError(_lib.NO_DEVICE, "floneum_b200 has no CPU device: it is the CUDA arm of the attention path")

    @staticmethod
    def count() -> int:
        n = ctypes.c_int32(0)
        _lib.load().fusor_cuda_device_count(ctypes.byref(n))
        return n.value

    @property
    def handle(self):
        return self._h

    def set_stream(self, stream: int):
        _lib.check(self._L.fusor_cuda_ctx_set_stream(self._h, ctypes.c_void_p(stream)), self._h)

    def stream(self) -> int:
        return self._L.fusor_cuda_ctx_stream(self._h) or 0

    def synchronize(self):
        _lib.check(self._L.fusor_cuda_stream_sync(self._h), self._h)

    def launch_count(self) -> int:
        return int(self._L.fusor_cuda_launch_count(self._h))

    def alloc(self, nbytes: int) -> int:
        p = ctypes.c_void_p()
        _lib.check(self._L.fusor_cuda_buffer_alloc(self._h, nbytes, ctypes.byref(p)), self._h)
        return p.value

    def free(self, ptr: int):
        self._L.fusor_cuda_buffer_free(self._h, ctypes.c_void_p(ptr))

    def close(self):
        if getattr(self, "_h", None):
            self._L.fusor_cuda_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
