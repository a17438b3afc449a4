"""fusor_cuda_flash_attention_noalloc: the prefill entry point for callers that cannot let a library allocate
device memory (a server whose own pool already owns all of the GPU, or a loop that cannot take the device-wide
synchronisation of cudaMalloc / cudaFree).  It keeps its f16 copy of V in a fixed array inside the library
instead of a cudaMalloc'ed buffer, so its results must equal those of fusor_cuda_flash_attention.

Collected last on purpose: a failure here cannot hide one in the other tests under `pytest -x`.
The test does not depend on the others: it creates everything it uses."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t4(t):
    return t._c4()


def test_noalloc_matches_the_allocating_entry_point_twice(device):
    import floneum_b200 as fb
    from conftest import assert_close
    from floneum_b200 import _lib, workloads as W
    L = _lib.load()
    rng = np.random.default_rng(424242)
    scale = float(1.0 / np.sqrt(128.0))
    # two calls in a row with different shapes and values: the second one meets the first one's leftovers
    for (B, Hq, Hkv, Sq, Skv, kind) in [(2, 8, 2, 300, 300, _lib.MASK_CAUSAL), (1, 4, 4, 130, 517, _lib.MASK_NONE)]:
        q = W.bf16_round(rng.standard_normal((B, Hq, Sq, 128), dtype=np.float32))
        k = W.bf16_round(rng.standard_normal((B, Hkv, Skv, 128), dtype=np.float32))
        v = W.bf16_round(rng.standard_normal((B, Hkv, Skv, 128), dtype=np.float32))
        tq, tk, tv = (fb.Tensor.from_slice(device, a.shape, a, _lib.BF16) for a in (q, k, v))
        want_t = fb.Tensor.empty(device, q.shape, _lib.F32)
        cq, ck, cv, cw = _t4(tq), _t4(tk), _t4(tv), _t4(want_t)
        _lib.check(L.fusor_cuda_flash_attention(device.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv),
                                                ctypes.c_float(scale), None, kind, 0, ctypes.byref(cw)), device.handle)
        want = want_t.as_slice()
        got_t = fb.Tensor.zeros(device, q.shape, _lib.F32)
        cg = _t4(got_t)
        rc = L.fusor_cuda_flash_attention_noalloc(ctypes.c_void_p(device.stream()), ctypes.byref(cq), ctypes.byref(ck),
                                                  ctypes.byref(cv), ctypes.c_float(scale), kind, ctypes.byref(cg))
        assert rc == _lib.OK, L.fusor_cuda_last_error(None)
        got = got_t.as_slice()
        # same kernels on the same data; held to the tolerance of the path (max 2e-3, mean 2e-4)
        assert_close(got, want, what=f"noalloc vs allocating entry point {B}x{Hq}/{Hkv}x{Sq}/{Skv}")


def test_noalloc_rejects_what_does_not_fit(device):
    import floneum_b200 as fb
    from floneum_b200 import _lib
    L = _lib.load()
    # V with 2 * 8 * 4096 * 128 elements is twice the static scratch: refused before anything is launched
    shape_q, shape_kv = (2, 8, 16, 128), (2, 8, 4096, 128)
    tq = fb.Tensor.zeros(device, shape_q, _lib.BF16)
    tk = fb.Tensor.zeros(device, shape_kv, _lib.BF16)
    out = fb.Tensor.zeros(device, shape_q, _lib.F32)
    cq, ck, co = _t4(tq), _t4(tk), _t4(out)
    rc = L.fusor_cuda_flash_attention_noalloc(ctypes.c_void_p(device.stream()), ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(ck),
                                              ctypes.c_float(0.1), _lib.MASK_CAUSAL, ctypes.byref(co))
    assert rc == _lib.UNSUPPORTED
    assert b"at most 4194304" in L.fusor_cuda_last_error(None)
    # f32 inputs belong to the general kernel, which this entry point does not run
    t32 = fb.Tensor.zeros(device, (1, 1, 16, 128), _lib.F32)
    c32 = _t4(t32)
    rc = L.fusor_cuda_flash_attention_noalloc(ctypes.c_void_p(device.stream()), ctypes.byref(c32), ctypes.byref(c32), ctypes.byref(c32),
                                              ctypes.c_float(0.1), _lib.MASK_NONE, ctypes.byref(c32))
    assert rc == _lib.UNSUPPORTED
