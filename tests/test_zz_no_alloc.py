"""fusor_cuda_flash_attention_noalloc: the prefill entry point for callers that cannot let a library allocate
device memory (a server whose own pool already owns all of the GPU, or a loop that cannot take the device-wide
synchronisation of cudaMalloc / cudaFree).  It keeps its f16 copy of V in a fixed array inside the library
instead of a cudaMalloc'ed buffer, so its results must agree with fusor_cuda_flash_attention and with the oracle.

Collected last on purpose: a failure here cannot hide one in the other tests under `pytest -x`.
The test does not depend on the others: it creates everything it uses."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t4(t):
    return t._c4()


def _both(device, q, k, v, scale, kind, out_dtype):
    """(allocating entry point, allocation-free entry point) on the same device tensors."""
    import floneum_b200 as fb
    from floneum_b200 import _lib
    L = _lib.load()
    tq, tk, tv = (fb.Tensor.from_slice(device, a.shape, a, _lib.BF16) for a in (q, k, v))
    want_t = fb.Tensor.empty(device, q.shape, out_dtype)
    cq, ck, cv, cw = _t4(tq), _t4(tk), _t4(tv), _t4(want_t)
    _lib.check(L.fusor_cuda_flash_attention(device.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv),
                                            ctypes.c_float(scale), None, kind, 0, ctypes.byref(cw)), device.handle)
    got_t = fb.Tensor.zeros(device, q.shape, out_dtype)
    cg = _t4(got_t)
    rc = L.fusor_cuda_flash_attention_noalloc(ctypes.c_void_p(device.stream()), ctypes.byref(cq), ctypes.byref(ck),
                                              ctypes.byref(cv), ctypes.c_float(scale), kind, ctypes.byref(cg))
    assert rc == _lib.OK, L.fusor_cuda_last_error(None)
    return want_t.as_slice(), got_t.as_slice()


def test_noalloc_matches_the_allocating_entry_point_twice(device):
    from conftest import assert_close
    from floneum_b200 import _lib
    from oracle import workloads as W
    from oracle import oracle as O
    rng = np.random.default_rng(424242)
    scale = float(1.0 / np.sqrt(128.0))
    # two calls in a row with different shapes and values: the second one meets the first one's leftovers.  The first
    # shape sends the allocating entry point to the two-tile kernel (Sq >= 256) while this one always runs the 64-key
    # kernel, so the two agree within the tolerance of the path; the second shape runs the same kernel in both and
    # must agree bit for bit.
    for (B, Hq, Hkv, Sq, Skv, kind) in [(2, 8, 2, 300, 300, _lib.MASK_CAUSAL), (1, 4, 4, 130, 517, _lib.MASK_NONE)]:
        q = W.bf16_round(rng.standard_normal((B, Hq, Sq, 128), dtype=np.float32))
        k = W.bf16_round(rng.standard_normal((B, Hkv, Skv, 128), dtype=np.float32))
        v = W.bf16_round(rng.standard_normal((B, Hkv, Skv, 128), dtype=np.float32))
        want, got = _both(device, q, k, v, scale, kind, _lib.F32)
        assert_close(got, want, what=f"noalloc vs allocating entry point {B}x{Hq}/{Hkv}x{Sq}/{Skv}")
        if Sq < 256:
            assert np.array_equal(got, want)
        oracle = O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL if kind == _lib.MASK_CAUSAL else O.MASK_NONE)
        assert_close(got, oracle, what=f"noalloc vs oracle {B}x{Hq}/{Hkv}x{Sq}/{Skv}")


def test_noalloc_overflowing_v_and_bf16_out(device):
    """The two paths through the static header words: a V element outside the f16 range raises the flag that sends every
    CTA to bf16 weights against the original V, and a bf16 output tensor goes through the same staging."""
    from conftest import assert_close
    from floneum_b200 import _lib
    from oracle import workloads as W
    from oracle import oracle as O
    rng = np.random.default_rng(7)
    scale = float(1.0 / np.sqrt(128.0))
    q = W.bf16_round(rng.standard_normal((1, 4, 200, 128), dtype=np.float32))
    k = W.bf16_round(rng.standard_normal((1, 2, 200, 128), dtype=np.float32))
    v = W.bf16_round(rng.standard_normal((1, 2, 200, 128), dtype=np.float32))
    v_big = v.copy()
    v_big[0, 1, 17, 5] = W.bf16_round(np.array([1.0e5], np.float32))[0]
    want, got = _both(device, q, k, v_big, scale, _lib.MASK_CAUSAL, _lib.F32)
    assert np.array_equal(got, want)  # same kernel, same fallback
    oracle = O.flash_attention(q, k, v_big, scale, mask_kind=O.MASK_CAUSAL)
    rel = np.abs(got - oracle) / (1.0 + np.abs(oracle))
    assert rel.max() < 8e-3, rel.max()  # bf16 weights: 8 significant bits
    # the next call, with an in-range V, is back on f16 weights: the flag word was cleared
    want, got = _both(device, q, k, v, scale, _lib.MASK_CAUSAL, _lib.BF16)
    assert np.array_equal(got, want)
    assert_close(got, O.bf16_round(O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL)), max_tol=2e-3 + 2.0 ** -7, mean_tol=2e-3,
                 what="noalloc bf16 out")


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
    # a tensor that is not memory of the current device (here: host memory) is refused, not handed to a tensor map
    host = np.zeros((1, 1, 16, 128), np.uint16)
    small = fb.Tensor.zeros(device, (1, 1, 16, 128), _lib.BF16)
    cs = _t4(small)
    ch = _t4(small)
    ch.data = host.ctypes.data
    o32 = fb.Tensor.zeros(device, (1, 1, 16, 128), _lib.F32)
    co = _t4(o32)
    rc = L.fusor_cuda_flash_attention_noalloc(ctypes.c_void_p(device.stream()), ctypes.byref(cs), ctypes.byref(ch), ctypes.byref(cs),
                                              ctypes.c_float(0.1), _lib.MASK_NONE, ctypes.byref(co))
    assert rc == _lib.INVALID_ARGUMENT
    assert b"not device memory of the current device" in L.fusor_cuda_last_error(None)
