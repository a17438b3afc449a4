"""Pins the CPU oracle: every known answer the reference's own tests hold for the attention path,
an independent float64 cross-check, and the committed golden fixtures.  CPU only."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

NEG = float("-inf")
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _identity_case():
    # fusor-ml/fusor/src/composite/flash_attention.rs:208-217, core/src/composite/flash_attention.rs:567-577
    q = np.array([1.0, 0.0, 0.0, 1.0], np.float32).reshape(1, 1, 2, 2)
    k = q.copy()
    v = np.array([1.0, 2.0, 3.0, 4.0], np.float32).reshape(1, 1, 2, 2)
    return q, k, v, np.float32(1.0 / np.sqrt(np.float32(2.0)))


def _softmax_attention_f64(q, k, v, scale, mask=None):
    g = q.shape[1] // k.shape[1]
    tq, tk, tv = (torch.from_numpy(np.asarray(a, np.float64)) for a in (q, k, v))
    tk, tv = tk.repeat_interleave(g, 1), tv.repeat_interleave(g, 1)
    s = tq @ tk.transpose(2, 3) * float(scale)
    if mask is not None:
        s = s + torch.from_numpy(np.asarray(mask, np.float64))
    return (torch.softmax(s, -1) @ tv).numpy()


def test_unmasked_known_answer():
    """test_flash_attention: equals unfused softmax attention within 0.01 (core/.../flash_attention.rs:561-603)."""
    q, k, v, scale = _identity_case()
    out = O.flash_attention(q, k, v, scale)
    assert out.shape == (1, 1, 2, 2) and np.isfinite(out).all()
    # closed form: row 0 weights softmax([s, 0]), row 1 softmax([0, s])
    e = np.exp(np.float64(scale))
    w = e / (e + 1.0)
    want = np.array([[w * 1 + (1 - w) * 3, w * 2 + (1 - w) * 4], [(1 - w) * 1 + w * 3, (1 - w) * 2 + w * 4]])
    assert np.abs(out[0, 0] - want).max() < 1e-6
    assert np.abs(out - _softmax_attention_f64(q, k, v, scale)).max() < 0.01


def test_causal_known_answer():
    """test_flash_attention_cpu_with_mask: with [[0,-inf],[0,0]] row 0 equals V row 0 (fusor/.../flash_attention.rs:242-277)."""
    q, k, v, scale = _identity_case()
    mask = np.array([[0.0, NEG], [0.0, 0.0]], np.float32)
    out = O.flash_attention(q, k, v, scale, mask, O.MASK_QK)
    assert abs(out[0, 0, 0, 0] - 1.0) < 0.01 and abs(out[0, 0, 0, 1] - 2.0) < 0.01
    assert out[0, 0, 0, 0] == 1.0 and out[0, 0, 0, 1] == 2.0  # exp(-inf) is an exact zero
    assert np.abs(out - _softmax_attention_f64(q, k, v, scale, mask)).max() < 1e-6
    # the analytic causal mode is the same mask
    assert np.array_equal(out, O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL))
    assert np.array_equal(out, O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL, skip_masked=True))


def test_gqa_case():
    """test_flash_attention_gqa_cpu inputs (fusor/.../flash_attention.rs:280-316): shape, finite, head h reads kv head h/2."""
    q = (np.arange(16, dtype=np.float32) * np.float32(0.1)).reshape(1, 4, 2, 2)
    k = (np.arange(8, dtype=np.float32) * np.float32(0.1) + 1).reshape(1, 2, 2, 2)
    v = (np.arange(8, dtype=np.float32) * np.float32(0.1) + 2).reshape(1, 2, 2, 2)
    scale = np.float32(1.0 / np.sqrt(np.float32(2.0)))
    out = O.flash_attention(q, k, v, scale)
    assert out.shape == (1, 4, 2, 2) and np.isfinite(out).all()
    assert np.abs(out - _softmax_attention_f64(q, k, v, scale)).max() < 1e-6
    for h in range(4):  # same as attending with the expanded heads
        single = O.flash_attention(q[:, h:h + 1], k[:, h // 2:h // 2 + 1], v[:, h // 2:h // 2 + 1], scale)
        assert np.array_equal(single[0, 0], out[0, h])


def test_batch_key_mask_case():
    """test_flash_attention_cpu_with_batch_key_mask (fusor/.../flash_attention.rs:319-359)."""
    q = (np.arange(12, dtype=np.float32) * np.float32(0.1)).reshape(2, 1, 3, 2)
    k = (np.arange(12, dtype=np.float32) * np.float32(0.1) + 1).reshape(2, 1, 3, 2)
    v = (np.arange(12, dtype=np.float32) * np.float32(0.1) + 2).reshape(2, 1, 3, 2)
    mask = np.array([[0, 0, 0], [0, 0, NEG]], np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(2.0)))
    out = O.flash_attention(q, k, v, scale, mask, O.MASK_BATCH_KEY)
    assert out.shape == (2, 1, 3, 2) and np.isfinite(out).all()
    want = _softmax_attention_f64(q, k, v, scale, mask[:, None, None, :])
    assert np.abs(out - want).max() < 1e-6


def test_head_divisibility_assert():
    """assert!(num_heads.is_multiple_of(num_kv_heads)) (fusor/.../flash_attention.rs:94-99)."""
    q = np.zeros((1, 3, 2, 2), np.float32)
    k = np.zeros((1, 2, 2, 2), np.float32)
    with pytest.raises(AssertionError, match="must be divisible"):
        O.flash_attention(q, k, k, 1.0)


def test_mask_shape_assert():
    q = np.zeros((1, 1, 2, 2), np.float32)
    with pytest.raises(AssertionError, match="QKMask shape"):
        O.flash_attention(q, q, q, 1.0, np.zeros((3, 2), np.float32), O.MASK_QK)


def test_causal_mask_pattern():
    """test_attention_mask_causal (fusor/src/cache/attention_mask.rs:84-111)."""
    m = O.causal_mask(3)
    assert m.tolist() == [[0.0, NEG, NEG], [0.0, 0.0, NEG], [0.0, 0.0, 0.0]]


def test_mask_cache_offset_and_window():
    """test_mask_cache_with_offset / _sliding_window (fusor/src/cache/mask_cache.rs:131-176)."""
    assert O.get_mask(3, 0).shape == (3, 3) and O.get_mask(5, 0).shape == (5, 5)
    m = O.get_mask(2, 3)
    assert m.shape == (2, 5)
    assert m.tolist() == [[0, 0, 0, 0, NEG], [0, 0, 0, 0, 0]]
    w = O.get_mask(4, 0, 2)
    assert w.tolist() == [[0, NEG, NEG, NEG], [0, 0, NEG, NEG], [NEG, 0, 0, NEG], [NEG, NEG, 0, 0]]


def test_tensor_cache_sequences():
    """TensorCache / KvCache unit tests (tensor_cache.rs:126-187, kv_cache.rs:70-158) on the numpy restatement."""
    c = O.TensorCacheOracle(1, 2)
    r = c.append(np.array([1, 2, 3, 4], np.float32).reshape(2, 1, 2))
    assert r.shape == (2, 1, 2) and c.current_seq_len == 1 and r.reshape(-1).tolist() == [1, 2, 3, 4]
    c = O.TensorCacheOracle(1, 3)
    c.append(np.array([1, 2], np.float32).reshape(1, 1, 2))
    r = c.append(np.array([3, 4], np.float32).reshape(1, 1, 2))
    assert r.shape == (1, 2, 2) and c.current_seq_len == 2 and r.reshape(-1).tolist() == [1, 2, 3, 4]
    c.reset()
    assert c.current_seq_len == 0 and c.current_data() is None
    kv = O.KvCacheOracle(1, 3)
    kv.append(np.array([1, 2], np.float32).reshape(1, 1, 1, 2), np.array([3, 4], np.float32).reshape(1, 1, 1, 2))
    k, v = kv.append(np.array([5, 6], np.float32).reshape(1, 1, 1, 2), np.array([7, 8], np.float32).reshape(1, 1, 1, 2))
    assert k.shape == (1, 2, 1, 2) and k.reshape(-1).tolist() == [1, 2, 5, 6] and v.reshape(-1).tolist() == [3, 4, 7, 8]
    kv.reset()
    assert kv.k() is None and kv.v() is None
    # growth to the next power of two and eviction past max_sequence_len (tensor_cache.rs:55-96)
    c = O.TensorCacheOracle(0, 5)
    for i in range(3):
        c.append(np.full((1, 2), i, np.float32))
    assert c.allocated_seq_len == 4 and c.current_seq_len == 3
    r = c.append(np.arange(8, dtype=np.float32).reshape(4, 2) + 10)
    assert c.current_seq_len == 5 and r[:, 0].tolist() == [2, 10, 12, 14, 16]


@pytest.mark.parametrize("seed", range(4))
def test_composite_vs_float64_and_online_order(seed):
    """Seeded version of the reference's fuzz grids (core/.../flash_attention.rs:683-688,933-939), CPU side:
    the composite restatement and the fused-kernel-order restatement agree with float64 softmax attention."""
    rng = np.random.default_rng(seed)
    B, Hkv, g = int(rng.integers(1, 3)), int(rng.integers(1, 5)), int(rng.integers(1, 5))
    Sq, D = int(rng.integers(1, 65)), int(rng.integers(1, 65))
    Skv = Sq + int(rng.integers(0, 32))
    q = rng.uniform(-1, 1, (B, Hkv * g, Sq, D)).astype(np.float32)
    k = rng.uniform(-1, 1, (B, Hkv, Skv, D)).astype(np.float32)
    v = rng.uniform(-1, 1, (B, Hkv, Skv, D)).astype(np.float32)
    scale = np.float32(1.0 / np.sqrt(D))
    mask = O.get_mask(Sq, Skv - Sq)
    want = _softmax_attention_f64(q, k, v, scale, mask)
    assert np.abs(O.flash_attention(q, k, v, scale, mask, O.MASK_QK) - want).max() < 2e-6
    assert np.abs(O.flash_attention_online(q, k, v, scale, mask) - want).max() < 5e-6
    assert np.array_equal(O.flash_attention(q, k, v, scale, mask, O.MASK_QK),
                          O.flash_attention(q, k, v, scale, mask_kind=O.MASK_CAUSAL, skip_masked=True))


def test_split_kv_partials_combine_to_full():
    rng = np.random.default_rng(7)
    q = rng.standard_normal((2, 4, 1, 16), dtype=np.float32)
    k = rng.standard_normal((2, 2, 100, 16), dtype=np.float32)
    v = rng.standard_normal((2, 2, 100, 16), dtype=np.float32)
    full = O.flash_attention(q, k, v, 0.25)
    parts = np.stack([O.attention_partial(q, k, v, 0.25, a, b) for a, b in ((0, 33), (33, 34), (34, 100))])
    assert np.abs(O.lse_combine(parts) - full).max() < 2e-6
    # an empty part (m = -inf, l = 0) is a no-op and produces no NaN
    empty = np.zeros_like(parts[:1])
    empty[..., 0] = NEG
    assert np.array_equal(O.lse_combine(np.concatenate([parts, empty])), O.lse_combine(parts))
    # a row whose parts are all empty attends to nothing: zeros, not 0 / 0
    assert np.array_equal(O.lse_combine(np.concatenate([empty, empty])), np.zeros_like(O.lse_combine(parts)))


def test_bf16_rounding_helper():
    a = np.array([1.0, 1.00390625, 1.01171875, -3.14159, 65504.0, 1e-40], np.float32)
    t = torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(O.bf16_round(a), t)
    assert np.array_equal(O.bf16_from_bits(O.bf16_bits(a)), t)


@pytest.mark.parametrize("name", ["ref_identity", "ref_identity_causal", "ref_gqa", "ref_batch_key", "seeded_f32_gqa_causal",
                                  "seeded_bf16_d128_causal", "seeded_decode_paged"])
def test_golden_fixture(name):
    """Committed fixtures (tests/golden/make_golden.py): inputs + expected output of the composite."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    if name == "seeded_decode_paged":
        dense_k = O.depage(O.bf16_from_bits(z["k_pages"]), z["page_table"], z["kv_len"])
        dense_v = O.depage(O.bf16_from_bits(z["v_pages"]), z["page_table"], z["kv_len"])
        for b in range(len(dense_k)):
            out = O.flash_attention(z["q"][b:b + 1], dense_k[b][None], dense_v[b][None], float(z["scale"]))
            assert np.array_equal(out[0], z["out"][b])
        return
    kind = int(z["mask_kind"])
    mask = z["mask"] if kind in (O.MASK_QK, O.MASK_BATCH_KEY) else None
    out = O.flash_attention(z["q"], z["k"], z["v"], float(z["scale"]), mask, kind)
    assert np.array_equal(out, z["out"]) or np.abs(out - z["out"]).max() < 1e-6


# --------------------------------------------------------------------------- rotary embedding
def test_rope_reference_inputs_shape_and_finite():
    """fusor-ml/fusor/src/composite/rope.rs:272-352: [1,3,11,64] of sin(i % 64), RopeCache::new(64, 11, 10000)."""
    x = np.sin((np.arange(3 * 11 * 64) % 64).astype(np.float32)).astype(np.float32).reshape(1, 3, 11, 64)
    cos, sin = O.rope_tables(64, 11, 10000.0)
    assert cos.shape == (11, 32) and sin.shape == (11, 32)
    for interleaved in (False, True):
        y = O.rope(x, cos, sin, 0, interleaved)
        assert y.shape == (1, 3, 11, 64) and np.isfinite(y).all()
        # position 0 has cos = 1, sin = 0: the row is unchanged
        assert np.array_equal(y[:, :, 0], x[:, :, 0])


def test_rope_hand_computed_pairs():
    """A quarter turn: cos = 0, sin = 1 sends (a, b) to (-b, a) in both pairings (rope.rs:8-19, 52-67, 96-117)."""
    x = np.array([1.0, 2.0, 3.0, 4.0], np.float32).reshape(1, 1, 1, 4)
    cos = np.zeros((1, 2), np.float32)
    sin = np.ones((1, 2), np.float32)
    assert O.rope(x, cos, sin, 0, False).ravel().tolist() == [-3.0, -4.0, 1.0, 2.0]   # pairs (0,2), (1,3)
    assert O.rope(x, cos, sin, 0, True).ravel().tolist() == [-2.0, 1.0, -4.0, 3.0]    # pairs (0,1), (2,3)
    # general angle, against the closed form in float64
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 2, 5, 8)).astype(np.float32)
    cos, sin = O.rope_tables(8, 16, 10000.0)
    y = O.rope(x, cos, sin, 7, False).astype(np.float64)
    c, s = cos[7:12].astype(np.float64), sin[7:12].astype(np.float64)
    want = np.concatenate([x[..., :4] * c - x[..., 4:] * s, x[..., 4:] * c + x[..., :4] * s], axis=-1)
    np.testing.assert_allclose(y, want, atol=1e-6)


def test_rope_inverse_frequency():
    """base_inverse_frequency (rope.rs:189-194): 1 / theta^(i/dim), i = 0, 2, .."""
    cos, sin = O.rope_tables(4, 2, 10000.0)
    np.testing.assert_allclose(cos[1], np.cos([1.0, 0.01]), rtol=1e-6)
    np.testing.assert_allclose(sin[1], np.sin([1.0, 0.01]), rtol=1e-6)


# --------------------------------------------------------------------------- output projection
def test_out_proj_is_transpose_reshape_linear():
    """attention_layer.rs:450-454 + linear.rs:72-115: transpose(1, 2), reshape to [b, q_len, hidden], x @ W^T + bias."""
    rng = np.random.default_rng(4)
    attn = rng.standard_normal((2, 3, 5, 4)).astype(np.float32)
    w = rng.standard_normal((7, 12)).astype(np.float32)
    b = rng.standard_normal(7).astype(np.float32)
    want = attn.transpose(0, 2, 1, 3).reshape(2, 5, 12).astype(np.float64) @ w.T.astype(np.float64) + b
    np.testing.assert_allclose(O.out_proj(attn, w, b), want, atol=1e-5)
    np.testing.assert_allclose(O.out_proj(attn, w), want - b, atol=1e-5)
    # identity weight: the projection is just the head-interleaving transpose
    eye = np.eye(12, dtype=np.float32)
    assert np.array_equal(O.out_proj(attn, eye), attn.transpose(0, 2, 1, 3).reshape(2, 5, 12))
