"""Rotary embedding and the fused RoPE + KV-cache append against the CPU oracle (bit-exact).

Reference tests for this op (fusor-ml/fusor/src/composite/rope.rs:272-352, test_rope_cpu / test_rope_interleaved_cpu)
feed x[b,h,s,d] = sin(flat index % 64) of shape [1,3,11,64] with RopeCache::new(64, 11, 10000) tables and assert the
output shape and finiteness; the same input is used here, compared bit for bit with the oracle's restatement.
"""
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _tables(device, D, ctx, theta=10000.0):
    from floneum_b200 import Tensor
    cos, sin = O.rope_tables(D, ctx, theta)
    return cos, sin, Tensor.from_slice(device, cos.shape, cos), Tensor.from_slice(device, sin.shape, sin)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_reference_case(device, interleaved):
    from floneum_b200 import Tensor
    x = np.sin((np.arange(1 * 3 * 11 * 64) % 64).astype(np.float32)).astype(np.float32).reshape(1, 3, 11, 64)
    cos, sin, dc, ds = _tables(device, 64, 11)
    t = Tensor.from_slice(device, x.shape, x)
    got = (t.rope_interleaved(dc, ds) if interleaved else t.rope(dc, ds)).as_slice()
    assert got.shape == (1, 3, 11, 64) and np.isfinite(got).all()
    want = O.rope(x, cos, sin, 0, interleaved)
    assert np.array_equal(_bits(got), _bits(want))


def test_rope_cache_tables_match_oracle(device):
    from floneum_b200 import RopeCache
    rc = RopeCache.new(128, 257, 500000.0, device)
    cos, sin = O.rope_tables(128, 257, 500000.0)
    assert np.array_equal(_bits(rc.cos.as_slice()), _bits(cos)) and np.array_equal(_bits(rc.sin.as_slice()), _bits(sin))


@pytest.mark.parametrize("shape,start,interleaved", [((2, 4, 33, 128), 5, False), ((1, 8, 1, 128), 4000, True),
                                                     ((3, 2, 17, 64), 0, True), ((2, 3, 7, 96), 9, False),
                                                     ((1, 2, 5, 72), 2, True), ((2, 2, 3, 40), 1, False)])
def test_rope_shapes_start_pos_and_norms(device, shape, start, interleaved):
    from floneum_b200 import Tensor, rope
    rng = np.random.default_rng(11)
    x = rng.standard_normal(shape).astype(np.float32)
    cos, sin, dc, ds = _tables(device, shape[3], start + shape[2] + 3)
    got = rope(Tensor.from_slice(device, shape, x), dc, ds, start, interleaved).as_slice()
    assert np.array_equal(_bits(got), _bits(O.rope(x, cos, sin, start, interleaved)))
    # a rotation keeps the norm of every pair
    h = shape[3] // 2
    pair = (lambda a: a[..., 0::2] ** 2 + a[..., 1::2] ** 2) if interleaved else (lambda a: a[..., :h] ** 2 + a[..., h:] ** 2)
    np.testing.assert_allclose(pair(got), pair(x), rtol=0, atol=2e-5)


def test_rope_bf16_in_and_out(device):
    from floneum_b200 import Tensor, rope
    from floneum_b200.tensor import BF16
    rng = np.random.default_rng(12)
    x = O.bf16_round(rng.standard_normal((2, 4, 9, 128)).astype(np.float32))
    cos, sin, dc, ds = _tables(device, 128, 64)
    got = rope(Tensor.from_slice(device, x.shape, x, BF16), dc, ds, 3, False).as_slice()
    assert np.array_equal(_bits(got), _bits(O.bf16_round(O.rope(x, cos, sin, 3, False))))


def test_rope_argument_checks(device):
    from floneum_b200 import FusorCudaError, Tensor, rope
    cos, sin, dc, ds = _tables(device, 64, 8)
    x = Tensor.zeros(device, (1, 2, 9, 64))
    with pytest.raises(FusorCudaError):  # positions beyond the tables
        rope(x, dc, ds, 0, False)
    with pytest.raises(AssertionError):  # table width does not match head_dim
        rope(Tensor.zeros(device, (1, 2, 4, 128)), dc, ds, 0, False)


@pytest.mark.parametrize("interleaved", [False, True])
def test_fused_rope_append_matches_rope_then_append(device, interleaved):
    """Two steps (a 37-token prompt, then one token) into a paged cache; rotated q, gathered K and V bit-exact."""
    from floneum_b200 import PagedKvCache, Tensor
    rng = np.random.default_rng(13)
    B, Hq, Hkv, D = 2, 8, 2, 128
    cos, sin, dc, ds = _tables(device, D, 64)
    cache = PagedKvCache(device, B, Hkv, D, num_pages=16, max_pages_per_seq=8)
    ks, vs, pos = [], [], 0
    for n in (37, 1):
        q = rng.standard_normal((B, Hq, n, D)).astype(np.float32)
        k = rng.standard_normal((B, Hkv, n, D)).astype(np.float32)
        v = rng.standard_normal((B, Hkv, n, D)).astype(np.float32)
        before = device.launch_count()
        q_rot = cache.rope_append(Tensor.from_slice(device, q.shape, q), Tensor.from_slice(device, k.shape, k),
                                  Tensor.from_slice(device, v.shape, v), dc, ds, start_pos=pos, interleaved=interleaved)
        assert device.launch_count() - before == 1
        assert np.array_equal(_bits(q_rot.as_slice()), _bits(O.rope(q, cos, sin, pos, interleaved)))
        ks.append(O.bf16_round(O.rope(k, cos, sin, pos, interleaved)))
        vs.append(O.bf16_round(v))
        pos += n
    gk, gv = cache.gather(B, pos)
    assert np.array_equal(_bits(gk.as_slice()), _bits(np.concatenate(ks, axis=2)))
    assert np.array_equal(_bits(gv.as_slice()), _bits(np.concatenate(vs, axis=2)))


def test_fused_rope_append_ragged_positions(device):
    """start_pos < 0: each sequence rotates at its own cache length."""
    from floneum_b200 import PagedKvCache, Tensor
    rng = np.random.default_rng(14)
    B, Hq, Hkv, D = 3, 4, 2, 64
    cos, sin, dc, ds = _tables(device, D, 128)
    cache = PagedKvCache(device, B, Hkv, D, num_pages=24, max_pages_per_seq=8)
    lens = np.array([5, 40, 17], np.int32)
    table = np.zeros((B, 8), np.int32)
    nxt = 0
    for b in range(B):
        for p in range((lens[b] + 1 + 15) // 16):
            table[b, p] = nxt
            nxt += 1
    cache.set_page_table(table, lens)
    q = rng.standard_normal((B, Hq, 1, D)).astype(np.float32)
    k = rng.standard_normal((B, Hkv, 1, D)).astype(np.float32)
    v = rng.standard_normal((B, Hkv, 1, D)).astype(np.float32)
    q_rot = cache.rope_append(Tensor.from_slice(device, q.shape, q), Tensor.from_slice(device, k.shape, k),
                              Tensor.from_slice(device, v.shape, v), dc, ds, start_pos=-1).as_slice()
    gk, _ = cache.gather(B, int(lens.max()) + 1)
    gk = gk.as_slice()
    for b in range(B):
        assert cache.seq_len(b) == lens[b] + 1
        assert np.array_equal(_bits(q_rot[b:b + 1]), _bits(O.rope(q[b:b + 1], cos, sin, int(lens[b]), False)))
        want = O.bf16_round(O.rope(k[b:b + 1], cos, sin, int(lens[b]), False))
        assert np.array_equal(_bits(gk[b:b + 1, :, lens[b]:lens[b] + 1]), _bits(want))


def test_kvcache_forward_append_then_attention(device):
    """RopeCache.forward_append + flash_attention on the cached views equals rope -> append -> attention in the oracle."""
    from floneum_b200 import KvCache, RopeCache, Tensor
    from conftest import assert_close
    rng = np.random.default_rng(15)
    B, Hq, Hkv, D = 1, 8, 2, 128
    rc = RopeCache.new(D, 256, 10000.0, device)
    cos, sin = O.rope_tables(D, 256)
    cache = KvCache.new(2, 200)
    k_all = np.zeros((B, Hkv, 0, D), np.float32)
    v_all = np.zeros((B, Hkv, 0, D), np.float32)
    pos = 0
    for n in (48, 1, 1):
        q = rng.standard_normal((B, Hq, n, D)).astype(np.float32)
        k = rng.standard_normal((B, Hkv, n, D)).astype(np.float32)
        v = rng.standard_normal((B, Hkv, n, D)).astype(np.float32)
        q_rot, ck, cv = rc.forward_append(Tensor.from_slice(device, q.shape, q), Tensor.from_slice(device, k.shape, k),
                                          Tensor.from_slice(device, v.shape, v), cache, start_pos=pos)
        k_all = np.concatenate([k_all, O.bf16_round(O.rope(k, cos, sin, pos))], axis=2)
        v_all = np.concatenate([v_all, O.bf16_round(v)], axis=2)
        pos += n
        assert cache.current_seq_len() == pos
        if n == 1:
            out = q_rot.flash_attention(ck, cv, D ** -0.5).as_slice()
            want = O.flash_attention(O.bf16_round(O.rope(q, cos, sin, pos - 1)), k_all, v_all, D ** -0.5)
            assert_close(out, want)
