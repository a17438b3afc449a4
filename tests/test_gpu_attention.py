"""GPU parity tests of Tensor.flash_attention through the C ABI, against the CPU oracle.

They follow the reference's own attention tests (fusor-ml/core/src/composite/flash_attention.rs:559-1060,
fusor-ml/fusor/src/composite/flash_attention.rs:203-360) with seeded data and the oracle as the expected value.
Tolerance of the path: max-abs <= 2e-3 and mean-abs <= 2e-4 against the f32 oracle on the same
(bf16-rounded where the kernel takes bf16) inputs; f32 inputs through the general kernel are held to 2e-5."""
import numpy as np
import pytest

from conftest import assert_close
from oracle import oracle as O

pytestmark = pytest.mark.gpu
NEG = float("-inf")


def _mods():
    import floneum_b200 as fb
    return fb


def _run(device, q, k, v, scale, mask=None, dtype=0, out_dtype=0):
    fb = _mods()
    tq = fb.Tensor.from_slice(device, q.shape, q, dtype)
    tk = fb.Tensor.from_slice(device, k.shape, k, dtype)
    tv = fb.Tensor.from_slice(device, v.shape, v, dtype)
    return tq.flash_attention(tk, tv, float(scale), mask, out_dtype).as_slice()


def test_flash_attention(device):
    """test_flash_attention: [1,1,2,2] identity q,k vs unfused attention, tol 0.01 in the reference."""
    z = np.load(__file__.replace("test_gpu_attention.py", "golden/ref_identity.npz"))
    out = _run(device, z["q"], z["k"], z["v"], z["scale"])
    assert out.shape == (1, 1, 2, 2)
    assert np.abs(out - z["out"]).max() < 1e-6


def test_flash_attention_causal_mask(device):
    """test_flash_attention_causal_mask: explicit [[0,-inf],[0,0]] mask tensor; row 0 equals V row 0."""
    fb = _mods()
    z = np.load(__file__.replace("test_gpu_attention.py", "golden/ref_identity_causal.npz"))
    mask = fb.Tensor.from_slice(device, (2, 2), z["mask"])
    out = _run(device, z["q"], z["k"], z["v"], z["scale"], (mask, fb.MaskKind.QKMask))
    assert np.abs(out - z["out"]).max() < 1e-6
    assert abs(out[0, 0, 0, 0] - 1.0) < 0.01 and abs(out[0, 0, 0, 1] - 2.0) < 0.01
    # AttentionMask::causal applied analytically gives the same values
    out2 = _run(device, z["q"], z["k"], z["v"], z["scale"], (fb.AttentionMask.causal(device, 2), fb.MaskKind.QKMask))
    assert np.array_equal(out, out2)
    # and its dense tensor is the reference's
    assert fb.AttentionMask.causal(device, 3).mask().as_slice().tolist() == [[0, NEG, NEG], [0, 0, NEG], [0, 0, 0]]


def test_flash_attention_gqa_and_batch_key_mask(device):
    fb = _mods()
    z = np.load(__file__.replace("test_gpu_attention.py", "golden/ref_gqa.npz"))
    out = _run(device, z["q"], z["k"], z["v"], z["scale"])
    assert out.shape == (1, 4, 2, 2) and np.abs(out - z["out"]).max() < 1e-6
    z = np.load(__file__.replace("test_gpu_attention.py", "golden/ref_batch_key.npz"))
    mask = fb.Tensor.from_slice(device, z["mask"].shape, z["mask"])
    out = _run(device, z["q"], z["k"], z["v"], z["scale"], (mask, fb.MaskKind.BatchKeyMask))
    assert out.shape == (2, 1, 3, 2) and np.abs(out - z["out"]).max() < 1e-6


def test_asserts_like_the_reference(device):
    fb = _mods()
    q = fb.Tensor.zeros(device, (1, 3, 2, 2))
    k = fb.Tensor.zeros(device, (1, 2, 2, 2))
    with pytest.raises(AssertionError, match="must be divisible"):
        q.flash_attention(k, k, 1.0, None)
    q = fb.Tensor.zeros(device, (1, 2, 2, 2))
    bad = fb.Tensor.zeros(device, (3, 2))
    with pytest.raises(AssertionError, match="QKMask shape"):
        q.flash_attention(k, k, 1.0, (bad, fb.MaskKind.QKMask))
    # the same misuse through the raw C ABI comes back as a status code
    import ctypes
    from floneum_b200 import _lib
    L = _lib.load()
    q3 = fb.Tensor.zeros(device, (1, 3, 2, 2))
    out = fb.Tensor.zeros(device, (1, 3, 2, 2))
    cq, ck, co = q3._c4(), k._c4(), out._c4()
    rc = L.fusor_cuda_flash_attention(device.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(ck), 1.0, None, 0, 0,
                                      ctypes.byref(co))
    assert rc == _lib.SHAPE_MISMATCH and b"divisible" in L.fusor_cuda_last_error(device.handle)


@pytest.mark.parametrize("it", range(12))
def test_flash_attention_masked_fuzz(device, it):
    """Seeded test_flash_attention_masked_fuzz: batch 1-2, heads 1-16, seq 1-128, head_dim 1-64, U(-1,1),
    causal mask with random +-0.25 on the allowed part (general kernel, f32)."""
    fb = _mods()
    rng = np.random.default_rng(100 + it)
    B, H, S, D = int(rng.integers(1, 3)), int(rng.integers(1, 17)), int(rng.integers(1, 129)), int(rng.integers(1, 65))
    q, k, v = (rng.uniform(-1, 1, (B, H, S, D)).astype(np.float32) for _ in range(3))
    mask = O.causal_mask(S)
    mask = np.where(np.isinf(mask), mask, rng.uniform(-0.25, 0.25, (S, S)).astype(np.float32))
    scale = np.float32(1.0 / np.sqrt(D))
    want = O.flash_attention(q, k, v, scale, mask, O.MASK_QK)
    got = _run(device, q, k, v, scale, (fb.Tensor.from_slice(device, mask.shape, mask), fb.MaskKind.QKMask))
    assert_close(got, want, 2e-5, 2e-6, f"masked fuzz {B}x{H}x{S}x{D}")


@pytest.mark.parametrize("it", range(8))
def test_flash_attention_kv_cache_fuzz(device, it):
    """Seeded test_flash_attention_kv_cache_fuzz: q_len 1-4 < kv_len <= q_len+31, zero mask."""
    fb = _mods()
    rng = np.random.default_rng(200 + it)
    B, H, D = int(rng.integers(1, 3)), int(rng.integers(1, 9)), int(rng.integers(1, 65))
    Sq = int(rng.integers(1, 5))
    Skv = Sq + int(rng.integers(1, 32))
    q = rng.uniform(-1, 1, (B, H, Sq, D)).astype(np.float32)
    k, v = (rng.uniform(-1, 1, (B, H, Skv, D)).astype(np.float32) for _ in range(2))
    mask = np.zeros((Sq, Skv), np.float32)
    scale = np.float32(1.0 / np.sqrt(D))
    want = O.flash_attention(q, k, v, scale, mask, O.MASK_QK)
    got = _run(device, q, k, v, scale, (fb.Tensor.from_slice(device, mask.shape, mask), fb.MaskKind.QKMask))
    assert_close(got, want, 2e-5, 2e-6, "kv cache fuzz")


@pytest.mark.parametrize("it", range(8))
def test_flash_attention_gqa_fuzz(device, it):
    """Seeded test_flash_attention_gqa_fuzz: kv_heads 1-4 x groups 1-4, reference head map kv_h = h / groups."""
    rng = np.random.default_rng(300 + it)
    Hkv, g = int(rng.integers(1, 5)), int(rng.integers(1, 5))
    B, S, D = int(rng.integers(1, 3)), int(rng.integers(1, 65)), int(rng.integers(1, 33))
    q = rng.uniform(-1, 1, (B, Hkv * g, S, D)).astype(np.float32)
    k, v = (rng.uniform(-1, 1, (B, Hkv, S, D)).astype(np.float32) for _ in range(2))
    scale = np.float32(1.0 / np.sqrt(D))
    assert_close(_run(device, q, k, v, scale), O.flash_attention(q, k, v, scale), 2e-5, 2e-6, "gqa fuzz")


def test_sliding_window_and_offset_masks(device):
    """MaskCache masks (sliding window, left-padded offset) applied analytically equal the dense tensors."""
    fb = _mods()
    rng = np.random.default_rng(5)
    mc = fb.MaskCache()
    for (Sq, off, w) in [(40, 0, 8), (6, 10, 16), (33, 5, None), (1, 50, None)]:
        Skv = Sq + (min(off, max(w - Sq, 0)) if w is not None else off)
        q = rng.standard_normal((1, 4, Sq, 32), dtype=np.float32)
        k, v = (rng.standard_normal((1, 2, Skv, 32), dtype=np.float32) for _ in range(2))
        m = mc.get_mask(Sq, off, w, device)
        want = O.flash_attention(q, k, v, 0.2, O.get_mask(Sq, off, w), O.MASK_QK)
        assert_close(_run(device, q, k, v, 0.2, (m, fb.MaskKind.QKMask)), want, 2e-5, 2e-6, f"analytic {Sq},{off},{w}")
        dense = fb.AttentionMask.new(m.mask())
        assert_close(_run(device, q, k, v, 0.2, (dense, fb.MaskKind.QKMask)), want, 2e-5, 2e-6, "dense")


def test_cfg1_cpu_reference_config_f32(device):
    """BASELINE config 1 in full: B1 S512 Hq32 Hkv8 D64 f32, causal, scale 1/8."""
    fb = _mods()
    from oracle import workloads as W
    w = W.cfg1()
    want = O.flash_attention(w.q, w.k, w.v, w.scale, O.causal_mask(512), O.MASK_QK)
    got = _run(device, w.q, w.k, w.v, w.scale, (fb.AttentionMask.causal(device, 512), fb.MaskKind.QKMask))
    assert_close(got, want, 2e-5, 2e-6, "cfg1")


def test_host_entry_point(device):
    """fusor_cuda_flash_attention_host: host buffers in, host buffer out."""
    import ctypes
    from floneum_b200 import _lib
    L = _lib.load()
    rng = np.random.default_rng(9)
    q = rng.standard_normal((2, 4, 50, 64), dtype=np.float32)
    k, v = (rng.standard_normal((2, 2, 70, 64), dtype=np.float32) for _ in range(2))
    out = np.empty_like(q)

    def t4(a):
        t = _lib.Tensor4()
        t.data, t.dtype = a.ctypes.data, _lib.F32
        acc = 1
        for i in range(3, -1, -1):
            t.shape[i], t.stride[i] = a.shape[i], acc
            acc *= a.shape[i]
        return t
    cq, ck, cv, co = t4(q), t4(k), t4(v), t4(out)
    rc = L.fusor_cuda_flash_attention_host(device.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv), 0.125, None,
                                           _lib.MASK_CAUSAL, 0, ctypes.byref(co))
    _lib.check(rc, device.handle)
    assert_close(out, O.flash_attention(q, k, v, 0.125, mask_kind=O.MASK_CAUSAL), 2e-5, 2e-6, "host entry")


# ----------------------------------------------------------------------------- tensor-core prefill (bf16, D = 128)
def _bf16_case(seed, B, Hq, Hkv, Sq, Skv, sigma=1.0):
    from oracle import workloads as W
    rng = np.random.default_rng(seed)
    q = W.bf16_round(sigma * rng.standard_normal((B, Hq, Sq, 128), dtype=np.float32))
    k = W.bf16_round(sigma * rng.standard_normal((B, Hkv, Skv, 128), dtype=np.float32))
    v = W.bf16_round(sigma * rng.standard_normal((B, Hkv, Skv, 128), dtype=np.float32))
    return q, k, v, np.float32(1.0 / np.sqrt(128.0))


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", [
    (1, 1, 1, 128, 128, True), (1, 4, 2, 200, 200, True), (2, 8, 2, 256, 256, False), (1, 4, 1, 1, 300, True),
    (1, 2, 2, 129, 257, True), (1, 4, 4, 384, 512, True), (2, 4, 2, 77, 77, False), (1, 8, 8, 640, 640, True),
    (1, 2, 1, 1000, 1000, True), (1, 1, 1, 5, 5, True),
])
def test_prefill_tensor_core_shapes(device, B, Hq, Hkv, Sq, Skv, causal):
    """Ragged and offset shapes through the tcgen05 kernel: partial query/key tiles, Skv > Sq, GQA, batch."""
    fb = _mods()
    q, k, v, scale = _bf16_case(1000 * Sq + Skv, B, Hq, Hkv, Sq, Skv)
    mask = (fb.MaskCache().get_mask(Sq, Skv - Sq, None, device), fb.MaskKind.QKMask) if causal else None
    got = _run(device, q, k, v, scale, mask, dtype=1)
    want = O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL if causal else O.MASK_NONE, skip_masked=True)
    assert_close(got, want, what=f"prefill {B}x{Hq}/{Hkv}x{Sq}/{Skv} causal={causal}")


@pytest.mark.parametrize("Sq,off,w", [(300, 0, 64), (300, 0, 7), (256, 0, 128), (200, 56, 256), (513, 0, 200), (130, 0, 1000)])
def test_prefill_sliding_window_tensor_core(device, Sq, off, w):
    """Sliding-window masks from MaskCache run analytically in the tcgen05 kernel (tiles left of the window are skipped,
    rows whose first visited tile is entirely outside their window stay exact)."""
    fb = _mods()
    eff_off = min(off, max(w - Sq, 0))
    Skv = Sq + eff_off
    q, k, v, scale = _bf16_case(7 * Sq + w, 1, 4, 2, Sq, Skv)
    m = fb.MaskCache().get_mask(Sq, off, w, device)
    got = _run(device, q, k, v, scale, (m, fb.MaskKind.QKMask), dtype=1)
    want = O.flash_attention(q, k, v, scale, O.get_mask(Sq, off, w), O.MASK_QK)
    assert_close(got, want, what=f"sliding window {Sq},{off},{w}")


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,kind", [
    (1, 4, 4, 64, 64, "causal"), (2, 8, 2, 300, 300, "causal"), (1, 4, 1, 130, 257, "offset"), (1, 2, 2, 513, 513, "window"),
    (1, 4, 2, 77, 200, "dense"), (1, 2, 1, 1, 90, "dense"),
])
def test_additive_mask_tensor_on_the_tensor_core_kernel(device, B, Hq, Hkv, Sq, Skv, kind):
    """The reference's main fuzz pattern (a causal mask with random +-0.25 on the allowed part, passed as a plain [Sq, Skv]
    tensor, so nothing about it is analytic) on bf16 tensors of head_dim 128: the call runs on the tensor-core kernel (two
    launches: the V pre-pass and the 64-key kernel, also from 256 rows on), rows whose first key tiles are entirely masked
    included, and agrees with the oracle and with the f32-arithmetic kernel."""
    import ctypes
    fb = _mods()
    from floneum_b200 import _lib
    rng = np.random.default_rng(5000 + Sq + Skv)
    q, k, v, scale = _bf16_case(31 * Sq + Skv, B, Hq, Hkv, Sq, Skv)
    if kind == "dense":
        base = np.zeros((Sq, Skv), np.float32)
    elif kind == "window":
        base = O.get_mask(Sq, Skv - Sq, 100)  # the leading key tiles of later rows are all -inf
    else:
        base = O.get_mask(Sq, Skv - Sq, None)
    mask = np.where(np.isinf(base), base, rng.uniform(-0.25, 0.25, base.shape).astype(np.float32)).astype(np.float32)
    want = O.flash_attention(q, k, v, scale, mask, O.MASK_QK)
    tm = fb.Tensor.from_slice(device, mask.shape, mask)
    before = device.launch_count()
    got = _run(device, q, k, v, scale, (tm, fb.MaskKind.QKMask), dtype=1)
    # upload of three tensors costs no kernel; the attention is the pre-pass + the 64-key tensor-core kernel
    assert device.launch_count() - before == 2
    assert_close(got, want, what=f"additive mask {kind} {B}x{Hq}/{Hkv}x{Sq}/{Skv}")
    # the f32-arithmetic kernel on the same inputs
    L = _lib.load()
    tq, tk, tv = (fb.Tensor.from_slice(device, a.shape, a, 1) for a in (q, k, v))
    out = fb.Tensor.empty(device, q.shape, 0)
    cq, ck, cv, co, cm = tq._c4(), tk._c4(), tv._c4(), out._c4(), tm._c2()
    _lib.check(L.fusor_cuda_flash_attention_general(device.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv),
                                                    ctypes.c_float(scale), ctypes.byref(cm), _lib.MASK_QK, 0, ctypes.byref(co)),
               device.handle)
    assert_close(got, out.as_slice(), what="tensor-core against general kernel")


def test_prefill_golden_fixture(device):
    fb = _mods()
    z = np.load(__file__.replace("test_gpu_attention.py", "golden/seeded_bf16_d128_causal.npz"))
    got = _run(device, z["q"], z["k"], z["v"], z["scale"], (fb.AttentionMask.causal(device, 200), fb.MaskKind.QKMask), dtype=1)
    assert_close(got, z["out"], what="golden bf16 d128")


def test_prefill_matches_general_kernel(device):
    """The two GPU kernels agree on the same bf16 inputs (general kernel = f32 arithmetic)."""
    import ctypes
    fb = _mods()
    from floneum_b200 import _lib
    q, k, v, scale = _bf16_case(77, 1, 8, 2, 300, 300)
    tq, tk, tv = (fb.Tensor.from_slice(device, a.shape, a, 1) for a in (q, k, v))
    fast = tq.flash_attention(tk, tv, float(scale), (fb.AttentionMask.causal(device, 300), fb.MaskKind.QKMask)).as_slice()
    out = fb.Tensor.empty(device, q.shape, 0)
    cq, ck, cv, co = tq._c4(), tk._c4(), tv._c4(), out._c4()
    _lib.check(_lib.load().fusor_cuda_flash_attention_general(device.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv),
                                                              ctypes.c_float(scale), None, _lib.MASK_CAUSAL, 0, ctypes.byref(co)),
               device.handle)
    assert_close(fast, out.as_slice(), what="tcgen05 vs general")


def test_prefill_strided_views_and_bf16_out(device):
    """Non-contiguous [B,H,S,D] views (a transposed [B,S,H,D] buffer, as after the projection reshape) and bf16 output."""
    fb = _mods()
    q, k, v, scale = _bf16_case(31, 2, 4, 2, 160, 160)

    def strided(a):
        B, H, S, D = a.shape
        buf = fb.Tensor.from_slice(device, (B, S, H, D), np.ascontiguousarray(a.transpose(0, 2, 1, 3)), 1)
        return fb.Tensor(device, buf.ptr, (B, H, S, D), 1, (S * H * D, D, H * D, 1), owner=buf)
    got = strided(q).flash_attention(strided(k), strided(v), float(scale), (fb.AttentionMask.causal(device, 160), fb.MaskKind.QKMask), out_dtype=1).as_slice()
    want = O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL)
    assert_close(got, O.bf16_round(want), max_tol=2e-3 + 2.0 ** -7, mean_tol=2e-3, what="strided, bf16 out")


def test_prefill_cfg5_value_distribution(device):
    """cfg5's distribution at reduced length: N(0, 0.5^2) with 5% of K rows x8 (softmax range stress)."""
    fb = _mods()
    from oracle import workloads as W
    w = W.cfg5(S=1536, Hq=8, Hkv=2)
    got = _run(device, w.q, w.k, w.v, w.scale, (fb.AttentionMask.causal(device, 1536), fb.MaskKind.QKMask), dtype=1)
    want = O.flash_attention(w.q, w.k, w.v, w.scale, mask_kind=O.MASK_CAUSAL, skip_masked=True)
    assert_close(got, want, what="cfg5 distribution")


def test_prefill_cfg2_full_size_sampled_rows(device):
    """BASELINE config 2 at full size (B4 S4096 Hq32 Hkv8 D128): sampled rows against the oracle, plus
    size-independent properties: row 0 of every head equals V row 0, and permuting batches permutes outputs."""
    fb = _mods()
    from oracle import workloads as W
    w = W.cfg2()
    B, Hq, S, D = w.q.shape
    tq, tk, tv = (fb.Tensor.from_slice(device, a.shape, a, 1) for a in (w.q, w.k, w.v))
    mask = (fb.AttentionMask.causal(device, S), fb.MaskKind.QKMask)
    got = tq.flash_attention(tk, tv, w.scale, mask).as_slice()
    assert np.isfinite(got).all()
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([rng.integers(0, B * Hq * S, 1500), np.arange(0, B * Hq * S, S), np.arange(S - 1, B * Hq * S, S),
                                     np.arange(127, B * Hq * S, 8 * S), np.arange(128, B * Hq * S, 8 * S)]))
    want = O.flash_attention(w.q, w.k, w.v, w.scale, mask_kind=O.MASK_CAUSAL, rows=rows, skip_masked=True)
    assert_close(got.reshape(-1, D)[rows], want, what="cfg2 sampled rows")
    g = Hq // w.k.shape[1]
    for b in range(B):
        for h in range(Hq):
            assert np.abs(got[b, h, 0] - w.v[b, h // g, 0]).max() <= 2e-3
    perm = [2, 0, 3, 1]
    tq2, tk2, tv2 = (fb.Tensor.from_slice(device, a.shape, np.ascontiguousarray(a[perm]), 1) for a in (w.q, w.k, w.v))
    got2 = tq2.flash_attention(tk2, tv2, w.scale, mask).as_slice()
    assert np.array_equal(got2, got[perm])


def test_prefill_two_tile_kernel_many_items_and_bf16_out(device):
    """More (row block, head, batch) items than SMs, so persistent CTAs of the two-tile kernel run several items each and
    its barrier phases carry over; output in bf16 (the 64-column TMA store path) and f32."""
    fb = _mods()
    B, Hq, Hkv, S = 2, 40, 8, 512  # 2 * 40 * 2 = 160 items
    q, k, v, scale = _bf16_case(4242, B, Hq, Hkv, S, S)
    mask = (fb.MaskCache().get_mask(S, 0, None, device), fb.MaskKind.QKMask)
    want = O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL, skip_masked=True)
    got32 = _run(device, q, k, v, scale, mask, dtype=1)
    assert_close(got32, want, what="two-tile kernel, 160 items, f32 out")
    got16 = _run(device, q, k, v, scale, mask, dtype=1, out_dtype=1)
    assert np.array_equal(got16.view(np.uint32), O.bf16_round(got32).view(np.uint32)), "bf16 output is the f32 output rounded once"


def test_prefill_value_overflowing_f16_falls_back(device):
    """|v| > 65504 cannot be held in the f16 copy of V: the kernels switch to bf16 weights and values (looser tolerance)."""
    fb = _mods()
    q, k, v, scale = _bf16_case(77, 1, 2, 1, 512, 512)
    v = v.copy()
    v[0, 0, 3, 5] = float(np.ravel(O.bf16_round(np.float32(1.0e5)))[0])
    mask = (fb.MaskCache().get_mask(512, 0, None, device), fb.MaskKind.QKMask)
    got = _run(device, q, k, v, scale, mask, dtype=1)
    want = O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL, skip_masked=True)
    assert np.isfinite(got).all()
    rel = np.abs(got - want) / (1.0 + np.abs(want))
    assert rel.max() < 8e-3, rel.max()


def test_host_entry_point_pipelined_chunks_match_device_path(device):
    """A host call above 8 MB is cut into (batch, kv-head group) chunks whose copies and kernels overlap; the result
    must be bit-identical to the one-piece device path (here with ordinary pageable host memory)."""
    import ctypes
    from floneum_b200 import _lib
    fb = _mods()
    L = _lib.load()
    B, Hq, Hkv, S = 3, 8, 4, 640
    q, k, v, scale = _bf16_case(31, B, Hq, Hkv, S, S)
    bits = lambda a: np.ascontiguousarray(O.bf16_bits(a))
    hq, hk, hv = bits(q), bits(k), bits(v)
    out = np.empty(q.shape, np.float32)

    def t4(a, dtype):
        t = _lib.Tensor4()
        t.data, t.dtype = a.ctypes.data, dtype
        acc = 1
        for i in range(3, -1, -1):
            t.shape[i], t.stride[i] = a.shape[i], acc
            acc *= a.shape[i]
        return t
    cq, ck, cv, co = t4(hq, _lib.BF16), t4(hk, _lib.BF16), t4(hv, _lib.BF16), t4(out, _lib.F32)
    assert hq.nbytes + hk.nbytes + hv.nbytes + out.nbytes > (8 << 20)
    for _ in range(2):  # the second call reuses the copy streams and the scratch buffers
        out[:] = np.nan
        rc = L.fusor_cuda_flash_attention_host(device.handle, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv),
                                               ctypes.c_float(scale), None, _lib.MASK_CAUSAL, 0, ctypes.byref(co))
        _lib.check(rc, device.handle)
        mask = (fb.MaskCache().get_mask(S, 0, None, device), fb.MaskKind.QKMask)
        assert np.array_equal(out, _run(device, q, k, v, scale, mask, dtype=1))


@pytest.mark.parametrize("B,Hq,Hkv,S,neg", [(3, 4, 2, 200, -np.inf), (2, 8, 8, 512, -10000.0), (4, 4, 1, 333, -np.inf)])
def test_batch_key_mask_on_the_tensor_core_kernels(device, B, Hq, Hkv, S, neg):
    """MaskKind::BatchKeyMask ([B, Skv] additive padding mask, bidirectional attention; rbert's Qwen embedding uses -10000,
    models/rbert/src/raw/qwen/attention.rs:93-113) through the tcgen05 kernels (64-key kernel below 256 rows, two-tile
    kernel from 256), against the composite with the same mask."""
    fb = _mods()
    q, k, v, scale = _bf16_case(900 + S, B, Hq, Hkv, S, S)
    rng = np.random.default_rng(S)
    lens = rng.integers(S // 3, S + 1, B)
    lens[0] = S
    mask = np.zeros((B, S), np.float32)
    for b in range(B):
        mask[b, lens[b]:] = neg
    mt = fb.Tensor.from_slice(device, mask.shape, mask)
    before = device.launch_count()
    got = _run(device, q, k, v, scale, (mt, fb.MaskKind.BatchKeyMask), dtype=1)
    assert device.launch_count() - before == 2, "V pre-pass + one tensor-core kernel, not the general kernel"
    want = O.flash_attention(q, k, v, scale, mask, O.MASK_BATCH_KEY)
    assert_close(got, want, what=f"batch key mask B{B} S{S} pad {neg}")


@pytest.mark.parametrize("it", range(10))
def test_prefill_two_tile_kernel_shape_fuzz(device, it):
    """Seeded shapes for the two-tile kernel (Sq >= 256): ragged query and key counts, key offsets (Skv > Sq), no mask /
    causal / sliding window / key mask, GQA groups 1-4, against the composite."""
    fb = _mods()
    rng = np.random.default_rng(7000 + it)
    B, Hkv, g = int(rng.integers(1, 3)), int(rng.integers(1, 3)), int(rng.integers(1, 5))
    Sq = int(rng.integers(256, 700))
    off = int(rng.choice([0, 0, 1, 77, 128, 300]))
    kind = ["none", "causal", "window", "keymask"][it % 4]
    if kind == "window":
        w = int(rng.integers(1, Sq + 50))
        off = min(off, max(w - Sq, 0))
    Skv = Sq + off
    q, k, v, scale = _bf16_case(8000 + it, B, Hkv * g, Hkv, Sq, Skv)
    if kind == "none":
        got = _run(device, q, k, v, scale, None, dtype=1)
        want = O.flash_attention(q, k, v, scale)
    elif kind == "causal":
        got = _run(device, q, k, v, scale, (fb.MaskCache().get_mask(Sq, off, None, device), fb.MaskKind.QKMask), dtype=1)
        want = O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL, skip_masked=True)
    elif kind == "window":
        got = _run(device, q, k, v, scale, (fb.MaskCache().get_mask(Sq, off, w, device), fb.MaskKind.QKMask), dtype=1)
        want = O.flash_attention(q, k, v, scale, O.get_mask(Sq, off, w), O.MASK_QK)
    else:
        mask = np.where(rng.random((B, Skv)) < 0.3, -np.inf, 0.0).astype(np.float32)
        mask[:, 0] = 0.0
        got = _run(device, q, k, v, scale, (fb.Tensor.from_slice(device, mask.shape, mask), fb.MaskKind.BatchKeyMask), dtype=1)
        want = O.flash_attention(q, k, v, scale, mask, O.MASK_BATCH_KEY)
    assert_close(got, want, what=f"two-tile fuzz {it}: B{B} Hq{Hkv * g}/{Hkv} Sq{Sq} Skv{Skv} {kind}")


def test_prefill_cfg5_full_size_sampled_rows(device):
    """BASELINE config 5 at full size (B1 S16384 Hq64 Hkv8 D128, N(0, 0.5^2), 5 % of the K rows x 8): sampled rows against
    the oracle, among them the first and last row of every head and the rows either side of every 256-row item edge of
    a few heads; row 0 of every head equals V row 0."""
    fb = _mods()
    from oracle import workloads as W
    w = W.cfg5()
    B, Hq, S, D = w.q.shape
    tq, tk, tv = (fb.Tensor.from_slice(device, a.shape, a, 1) for a in (w.q, w.k, w.v))
    got = tq.flash_attention(tk, tv, w.scale, (fb.AttentionMask.causal(device, S), fb.MaskKind.QKMask)).as_slice()
    assert np.isfinite(got).all()
    rng = np.random.default_rng(5)
    edges = np.concatenate([np.arange(255, S, 256), np.arange(256, S, 256), np.arange(127, S, 256), np.arange(128, S, 256)])
    rows = np.unique(np.concatenate([rng.integers(0, Hq * S, 700), np.arange(0, Hq * S, S), np.arange(S - 1, Hq * S, S)] +
                                    [h * S + edges for h in (0, 9, 37, 63)]))
    want = O.flash_attention(w.q, w.k, w.v, w.scale, mask_kind=O.MASK_CAUSAL, rows=rows, skip_masked=True)
    assert_close(got.reshape(-1, D)[rows], want, what="cfg5 sampled rows")
    g = Hq // w.k.shape[1]
    for h in range(Hq):
        assert np.abs(got[0, h, 0] - w.v[0, h // g, 0]).max() <= 2e-3


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", [(1, 4, 2, 130, 130, True), (2, 8, 2, 512, 512, True), (1, 4, 4, 300, 777, False),
                                                     (1, 2, 1, 1024, 1024, True)])
def test_prefill_f16_tensors(device, B, Hq, Hkv, Sq, Skv, causal):
    """f16 q, k, v (the reference's GPU arm is generic over f32 / f16 with f32 accumulation,
    fusor-ml/core/src/composite/flash_attention.rs:28-38,189): both tensor-core kernels, f32 and f16 outputs, against the
    oracle on the same f16-rounded inputs; and the general kernel on a head_dim the tensor-core kernels do not take."""
    fb = _mods()
    rng = np.random.default_rng(1000 * Sq + Skv)
    h = lambda a: a.astype(np.float16).astype(np.float32)
    q, k, v = (h(rng.standard_normal(s, dtype=np.float32)) for s in ((B, Hq, Sq, 128), (B, Hkv, Skv, 128), (B, Hkv, Skv, 128)))
    scale = 128 ** -0.5
    if causal:
        mask = (fb.AttentionMask.causal(device, Sq), fb.MaskKind.QKMask) if Sq == Skv else None
        want = O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL)
    else:
        mask, want = None, O.flash_attention(q, k, v, scale)
    before = device.launch_count()
    got = _run(device, q, k, v, scale, mask, dtype=2)
    assert device.launch_count() - before == 1  # no copy of V: the weights are f16 against V itself
    assert_close(got, want, what="f16 in, f32 out")
    got16 = _run(device, q, k, v, scale, mask, dtype=2, out_dtype=2)
    assert_close(got16, h(want), max_tol=2e-3 + 2.0 ** -10, mean_tol=4e-4, what="f16 in, f16 out")
    if Sq == 130:
        q64, k64, v64 = q[..., :64].copy(), k[..., :64].copy(), v[..., :64].copy()
        got64 = _run(device, q64, k64, v64, 0.125, mask, dtype=2, out_dtype=2)
        assert_close(got64, h(O.flash_attention(q64, k64, v64, 0.125, mask_kind=O.MASK_CAUSAL)), max_tol=2.0 ** -10 + 2e-5, mean_tol=2e-4,
                     what="f16 through the general kernel")
