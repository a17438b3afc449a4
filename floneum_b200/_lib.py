"""ctypes binding of libfusor_cuda.so (the C ABI in include/fusor_cuda.h).

The library is the product; this module only declares its entry points.  It raises when
the shared object is missing: there is no Python or CPU fallback for any compute call.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

from . import build as _build

OK, INVALID_ARGUMENT, SHAPE_MISMATCH, UNSUPPORTED, CUDA_ERROR, NO_DEVICE, TIMEOUT, OUT_OF_PAGES, INTERNAL, NCCL_ERROR = range(10)
F32, BF16, F16 = 0, 1, 2
MASK_NONE, MASK_QK, MASK_BATCH_KEY, MASK_CAUSAL, MASK_SLIDING = range(5)

STATUS_NAMES = ["OK", "INVALID_ARGUMENT", "SHAPE_MISMATCH", "UNSUPPORTED", "CUDA_ERROR", "NO_DEVICE", "TIMEOUT",
                "OUT_OF_PAGES", "INTERNAL", "NCCL_ERROR"]


class Tensor4(ctypes.Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int32), ("_pad", c_int32), ("shape", c_int64 * 4),
                ("stride", c_int64 * 4)]


class Tensor2(ctypes.Structure):
    _fields_ = [("data", c_void_p), ("shape", c_int64 * 2), ("stride", c_int64 * 2)]


class FusorCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{STATUS_NAMES[code] if 0 <= code < len(STATUS_NAMES) else code}] {message}")
        self.code = code
        self.message = message


_T4 = POINTER(Tensor4)
_T2 = POINTER(Tensor2)

# name -> (restype, argtypes); every symbol include/fusor_cuda.h declares
SIGNATURES = {
    "fusor_cuda_device_count": (c_int32, [POINTER(c_int32)]),
    "fusor_cuda_ctx_create": (c_int32, [c_int32, c_void_p, POINTER(c_void_p)]),
    "fusor_cuda_ctx_destroy": (c_int32, [c_void_p]),
    "fusor_cuda_ctx_set_stream": (c_int32, [c_void_p, c_void_p]),
    "fusor_cuda_ctx_stream": (c_void_p, [c_void_p]),
    "fusor_cuda_last_error": (c_char_p, [c_void_p]),
    "fusor_cuda_stream_sync": (c_int32, [c_void_p]),
    "fusor_cuda_launch_count": (c_int64, [c_void_p]),
    "fusor_cuda_buffer_alloc": (c_int32, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "fusor_cuda_buffer_free": (c_int32, [c_void_p, c_void_p]),
    "fusor_cuda_buffer_upload": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "fusor_cuda_buffer_download": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "fusor_cuda_cast": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_int32, c_int64]),
    "fusor_cuda_flash_attention": (c_int32, [c_void_p, _T4, _T4, _T4, c_float, _T2, c_int32, c_int32, _T4]),
    "fusor_cuda_flash_attention_host": (c_int32, [c_void_p, _T4, _T4, _T4, c_float, _T2, c_int32, c_int32, _T4]),
    "fusor_cuda_flash_attention_general": (c_int32, [c_void_p, _T4, _T4, _T4, c_float, _T2, c_int32, c_int32, _T4]),
    "fusor_cuda_flash_attention_noalloc": (c_int32, [c_void_p, _T4, _T4, _T4, c_float, c_int32, _T4]),
    "fusor_cuda_selftest_wait_limit": (c_int32, [c_void_p]),
    "fusor_cuda_kvcache_create": (c_int32, [c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                            POINTER(c_void_p)]),
    "fusor_cuda_kvcache_destroy": (c_int32, [c_void_p]),
    "fusor_cuda_kvcache_reset": (c_int32, [c_void_p]),
    "fusor_cuda_kvcache_append": (c_int32, [c_void_p, _T4, _T4]),
    "fusor_cuda_exchange_create": (c_int32, [c_void_p, c_int32, c_int32, c_int64, POINTER(c_void_p)]),
    "fusor_cuda_exchange_handle": (c_int32, [c_void_p, c_void_p]),
    "fusor_cuda_exchange_connect": (c_int32, [c_void_p, c_void_p]),
    "fusor_cuda_exchange_disconnect": (c_int32, [c_void_p]),
    "fusor_cuda_exchange_destroy": (c_int32, [c_void_p]),
    "fusor_cuda_exchange_decode": (c_int32, [c_void_p, c_void_p, _T4, c_float, c_void_p]),
    "fusor_cuda_kvcache_set_decode_ctas": (c_int32, [c_void_p, c_int32]),
    "fusor_cuda_exchange_lse_combine": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "fusor_cuda_attention_out_proj": (c_int32, [c_void_p, _T4, _T4, c_void_p, _T4]),
    "fusor_cuda_comm_unique_id": (c_int32, [c_void_p]),
    "fusor_cuda_comm_init": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, POINTER(c_void_p)]),
    "fusor_cuda_comm_poll": (c_int32, [c_void_p]),
    "fusor_cuda_comm_abort": (c_int32, [c_void_p]),
    "fusor_cuda_comm_destroy": (c_int32, [c_void_p]),
    "fusor_cuda_comm_all_reduce_sum": (c_int32, [c_void_p, c_void_p, c_int64, c_int32]),
    "fusor_cuda_attention_out_proj_all_reduce": (c_int32, [c_void_p, c_void_p, _T4, _T4, c_void_p, _T4]),
    "fusor_cuda_rope": (c_int32, [c_void_p, _T4, c_void_p, c_void_p, c_int32, c_int32, c_int32, _T4]),
    "fusor_cuda_kvcache_rope_append": (c_int32, [c_void_p, _T4, _T4, _T4, c_void_p, c_void_p, c_int32, c_int32, c_int32, _T4]),
    "fusor_cuda_kvcache_truncate_front": (c_int32, [c_void_p, c_int32, c_int32]),
    "fusor_cuda_kvcache_seq_len": (c_int32, [c_void_p, c_int32, POINTER(c_int32)]),
    "fusor_cuda_kvcache_set_page_table": (c_int32, [c_void_p, POINTER(c_int32), POINTER(c_int32), c_int32]),
    "fusor_cuda_kvcache_write_pages": (c_int32, [c_void_p, c_int32, c_int32, c_void_p, c_void_p]),
    "fusor_cuda_kvcache_read_pages": (c_int32, [c_void_p, c_int32, c_int32, c_void_p, c_void_p]),
    "fusor_cuda_kvcache_pools": (c_int32, [c_void_p, POINTER(c_void_p), POINTER(c_void_p)]),
    "fusor_cuda_kvcache_gather": (c_int32, [c_void_p, _T4, _T4]),
    "fusor_cuda_flash_attention_decode": (c_int32, [c_void_p, c_void_p, _T4, c_float, _T4]),
    "fusor_cuda_flash_attention_decode_partial": (c_int32, [c_void_p, c_void_p, _T4, c_float, c_void_p]),
    "fusor_cuda_flash_attention_decode_host": (c_int32, [c_void_p, c_void_p, _T4, c_float, _T4]),
    "fusor_cuda_decode_plan": (c_int32, [POINTER(c_int32), c_int32, c_int32, c_int32, POINTER(c_int32), c_int32,
                                         POINTER(c_int32), POINTER(c_int32)]),
    "fusor_cuda_lse_combine": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int32, c_void_p]),
}

_lib = None


def load(path: str | None = None):
    """Loads the shared library (building it first when the sources are newer and nvcc exists)."""
    global _lib
    if _lib is not None:
        return _lib
    override = path or os.environ.get("FUSOR_CUDA_LIB")  # a differently tuned build of the same sources
    path = override or _build.LIB_PATH
    if not override and _build.needs_build() and os.path.exists(os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")):
        _build.build()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m floneum_b200.build`. "
            "floneum_b200 has no fallback path without its CUDA library.")
    L = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def check(rc: int, ctx=None):
    if rc != OK:
        msg = load().fusor_cuda_last_error(ctx)
        raise FusorCudaError(rc, msg.decode() if msg else "")
