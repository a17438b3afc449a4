"""The C-ABI library without a GPU: it loads, exports every symbol include/fusor_cuda.h declares,
reports NO_DEVICE instead of computing on the CPU, and its host-only logic (the split-KV plan) is right."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fusor_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fusor_cuda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from floneum_b200 import _lib
    L = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in include/fusor_cuda.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == declared


def test_integration_doc_binds_every_declared_symbol():
    """The Rust `extern "C"` block a maintainer would add names every entry point of the header."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    bound = set(re.findall(r"pub fn (fusor_cuda_[a-z0-9_]+)\(", text))
    assert sorted(bound) == _declared_symbols()


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from floneum_b200 import Device, FusorCudaError, _lib
    with pytest.raises(FusorCudaError) as e:
        Device.gpu(0)
    assert e.value.code == _lib.NO_DEVICE
    with pytest.raises(FusorCudaError):
        Device.cpu()


def test_null_arguments_are_status_codes():
    from floneum_b200 import _lib
    L = _lib.load()
    assert L.fusor_cuda_ctx_create(0, None, None) == _lib.INVALID_ARGUMENT
    assert L.fusor_cuda_flash_attention(None, None, None, None, 1.0, None, 0, 0, None) == _lib.INVALID_ARGUMENT
    assert L.fusor_cuda_kvcache_reset(None) == _lib.INVALID_ARGUMENT
    assert b"null" in L.fusor_cuda_last_error(None)


def _plan(kv_len, Hkv, grid):
    from floneum_b200 import _lib
    L = _lib.load()
    kv = np.ascontiguousarray(kv_len, np.int32)
    B = kv.size
    cap = B * Hkv + grid
    segs = np.zeros((cap, 9), np.int32)
    n = ctypes.c_int32()
    cta = np.zeros(grid + 1, np.int32)
    p = ctypes.POINTER(ctypes.c_int32)
    rc = L.fusor_cuda_decode_plan(kv.ctypes.data_as(p), B, Hkv, grid, segs.ctypes.data_as(p), cap, ctypes.byref(n),
                                  cta.ctypes.data_as(p))
    assert rc == 0, L.fusor_cuda_last_error(None)
    return segs[:n.value], cta


@pytest.mark.parametrize("kv_len,Hkv,grid", [([1], 1, 1), ([17, 5, 300], 2, 7), ([1024, 8192, 4000, 1025], 8, 296),
                                             ([131072], 8, 296), (list(range(1, 70)), 3, 148), ([16] * 5, 2, 10),
                                             ([33, 1, 1, 2000], 1, 592), ([7], 4, 3), ([0, 40, 0, 0, 1000, 0], 2, 37),
                                             ([0, 0, 5], 1, 4)])
def test_decode_plan_partitions_every_page_once_and_evenly(kv_len, Hkv, grid):
    """The deal the decode kernel computes per CTA (same functions, walked on the host): every page exactly once, shares
    within one page of each other, and the partial records of one (sequence, kv head) in a contiguous run of slots that
    no other (sequence, kv head) touches."""
    pages = [(n + 15) // 16 for n in kv_len]
    total = sum(pages) * Hkv
    grid = min(grid, total)  # (empty sequences, as a rank's KV chunk of a short sequence can be, own no page and no record)
    segs, cta = _plan(kv_len, Hkv, grid)
    seen = {}
    per_cta = np.zeros(grid, np.int64)
    assert cta[0] == 0 and cta[-1] == len(segs) and np.all(np.diff(cta) >= 0)
    slots = {}
    for c in range(grid):
        off = 0
        for i in range(cta[c], cta[c + 1]):
            b, hk, p0, p1, n, slot, coff, n_rec, first = segs[i]
            assert n == kv_len[b] and 0 <= p0 < p1 <= pages[b] and coff == off
            assert slot == b * Hkv + hk + c and first <= slot < first + n_rec and slot < len(kv_len) * Hkv + grid
            assert slot not in slots, "two segments share a record slot"
            slots[slot] = (b, hk)
            for pg in range(p0, p1):
                assert (b, hk, pg) not in seen
                seen[(b, hk, pg)] = c
            off += p1 - p0
        per_cta[c] = off
    assert len(seen) == total
    assert per_cta.max() - per_cta.min() <= 1  # even split
    # per (sequence, kv head): n_records segments, in page order, filling exactly [first_slot, first_slot + n_records)
    by_seq = {}
    for sg in segs:
        by_seq.setdefault((sg[0], sg[1]), []).append(sg)
    assert len(by_seq) == sum(1 for n in kv_len if n > 0) * Hkv
    for (b, hk), lst in by_seq.items():
        lst.sort(key=lambda s: s[2])
        assert lst[0][2] == 0 and lst[-1][3] == pages[b] and all(lst[i][3] == lst[i + 1][2] for i in range(len(lst) - 1))
        n_rec, first = lst[0][7], lst[0][8]
        assert all(s[7] == n_rec and s[8] == first for s in lst) and len(lst) == n_rec
        assert sorted(s[5] for s in lst) == list(range(first, first + n_rec))


def test_decode_plan_seeded_fuzz():
    """The same properties on 60 seeded random cases: ragged lengths with empty sequences among them, 1-8 kv heads, grids
    from one CTA to four per SM, and grids larger than the number of pages clipped as the host does."""
    rng = np.random.default_rng(424242)
    for _ in range(60):
        B = int(rng.integers(1, 40))
        kv_len = [int(x) for x in rng.integers(0, int(rng.choice([3, 40, 700, 9000])), B)]
        if sum(kv_len) == 0:
            kv_len[0] = 1
        Hkv = int(rng.integers(1, 9))
        grid = int(rng.choice([1, 2, 7, 148, 296, 592]))
        test_decode_plan_partitions_every_page_once_and_evenly(kv_len, Hkv, grid)


def test_decode_plan_rejects_bad_input():
    from floneum_b200 import _lib
    L = _lib.load()
    kv = np.array([-1], np.int32)
    p = ctypes.POINTER(ctypes.c_int32)
    buf = np.zeros(64, np.int32)
    n = ctypes.c_int32()
    rc = L.fusor_cuda_decode_plan(kv.ctypes.data_as(p), 1, 1, 1, buf.ctypes.data_as(p), 8, ctypes.byref(n),
                                  buf.ctypes.data_as(p))
    assert rc == _lib.INVALID_ARGUMENT


def test_mask_mirror_matches_reference_patterns():
    """AttentionMask / MaskCache mirrors produce the dense values of the reference without a device."""
    from floneum_b200.cache import AttentionMask, MaskCache
    from oracle import oracle as O
    NEG = float("-inf")
    m = AttentionMask.causal(None, 3)
    assert m.host_values().tolist() == [[0.0, NEG, NEG], [0.0, 0.0, NEG], [0.0, 0.0, 0.0]]
    mc = MaskCache()
    assert mc.get_mask(3, 0, None, None) is mc.get_mask(3, 0, None, None)  # memoised
    assert mc.get_mask(2, 3, None, None).shape() == (2, 5)
    for (s, off, w) in [(2, 3, None), (4, 0, 2), (4, 9, 6), (5, 2, 3), (1, 17, None)]:
        assert np.array_equal(mc.get_mask(s, off, w, None).host_values(), O.get_mask(s, off, w)), (s, off, w)
    from floneum_b200 import _lib
    assert mc.get_mask(4, 6, None, None).analytic_kind(4, 10) == (_lib.MASK_CAUSAL, 0)
    assert mc.get_mask(4, 6, None, None).analytic_kind(4, 11) is None
