"""GPU parity tests of the paged KV cache, split-KV decode and the KvCache mirror, against the CPU oracle."""
import numpy as np
import pytest

from conftest import assert_close
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _fb():
    import floneum_b200 as fb
    return fb


def _install(device, w):
    fb = _fb()
    B = w.q.shape[0]
    cache = fb.PagedKvCache(device, B, w.k_pages.shape[1], w.k_pages.shape[3], w.k_pages.shape[0], w.page_table.shape[1])
    cache.write_pages(0, w.k_pages, w.v_pages)
    cache.set_page_table(w.page_table, w.kv_len)
    return cache


def _oracle_decode(w):
    return np.stack([O.flash_attention(w.q[b:b + 1], w.k_dense[b][None], w.v_dense[b][None], w.scale)[0]
                     for b in range(w.q.shape[0])])


@pytest.mark.parametrize("B,Hq,Hkv,lo,hi", [(1, 4, 1, 1, 1), (3, 8, 2, 20, 90), (4, 32, 8, 100, 700), (2, 8, 8, 15, 17),
                                             (5, 16, 2, 1, 40), (2, 64, 8, 3000, 5000)])
def test_paged_decode_ragged(device, B, Hq, Hkv, lo, hi):
    """Ragged lengths (including partial last pages and 1-token sequences), permuted page table, g = 1..8."""
    fb = _fb()
    from oracle import workloads as W
    w = W.cfg3(B=B, Hq=Hq, Hkv=Hkv, lo=lo, hi=hi)
    cache = _install(device, w)
    q = fb.Tensor.from_slice(device, w.q.shape, w.q, 1)
    got = cache.decode(q, w.scale).as_slice()
    assert_close(got, _oracle_decode(w), what=f"decode B{B} Hq{Hq}/{Hkv} len[{lo},{hi}]")
    # f32 query tensor (the reference call site passes f32) gives the same result
    got32 = cache.decode(fb.Tensor.from_slice(device, w.q.shape, w.q, 0), w.scale).as_slice()
    assert np.array_equal(got, got32)
    # host-memory entry point
    assert np.array_equal(cache.decode_host(w.q, w.scale), got)


def test_paged_decode_golden_fixture(device):
    fb = _fb()
    z = np.load(__file__.replace("test_gpu_decode.py", "golden/seeded_decode_paged.npz"))
    cache = fb.PagedKvCache(device, 3, 2, 128, z["k_pages"].shape[0], z["page_table"].shape[1])
    cache.write_pages(0, z["k_pages"], z["v_pages"])
    cache.set_page_table(z["page_table"], z["kv_len"])
    got = cache.decode(fb.Tensor.from_slice(device, z["q"].shape, z["q"], 1), float(z["scale"])).as_slice()
    assert_close(got, z["out"], what="golden decode")


def test_decode_head_dim_64(device):
    fb = _fb()
    from oracle import workloads as W
    rng = np.random.default_rng(12)
    B, Hq, Hkv, D = 2, 8, 2, 64
    lens = np.array([75, 130])
    q = W.bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
    cache = fb.KvCache.new(2, 1024)
    ks = W.bf16_round(rng.standard_normal((B, Hkv, 130, D), dtype=np.float32))
    vs = W.bf16_round(rng.standard_normal((B, Hkv, 130, D), dtype=np.float32))
    paged = fb.PagedKvCache(device, B, Hkv, D, 32, 16)
    pt = np.arange(32, dtype=np.int32).reshape(2, 16)[:, ::-1].copy()
    kp = np.zeros((32, Hkv, 16, D), np.uint16)
    vp = np.zeros_like(kp)
    for b in range(B):
        for t in range(lens[b]):
            kp[pt[b, t // 16], :, t % 16] = W.bf16_bits(ks[b, :, t])
            vp[pt[b, t // 16], :, t % 16] = W.bf16_bits(vs[b, :, t])
    paged.write_pages(0, kp, vp)
    paged.set_page_table(pt, lens)
    got = paged.decode(fb.Tensor.from_slice(device, q.shape, q, 1), 0.125).as_slice()
    want = np.stack([O.flash_attention(q[b:b + 1], ks[b:b + 1, :, :lens[b]], vs[b:b + 1, :, :lens[b]], 0.125)[0] for b in range(B)])
    assert_close(got, want, what="decode D=64")
    del cache


def test_decode_partial_and_lse_combine(device):
    """KV-sequence chunks: per-chunk partials {m, l, O} merged by log-sum-exp equal attention over all keys,
    and each partial matches the oracle's partial of that key range."""
    fb = _fb()
    from oracle import workloads as W
    from floneum_b200.cache import lse_combine
    world = 4
    full = W.cfg4(Skv=4096 + 160, Hq=16, Hkv=2)
    parts = []
    for r in range(world):
        w = W.cfg4(Skv=4096 + 160, Hq=16, Hkv=2, rank=r, world=world)
        cache = _install(device, w)
        p = cache.decode_partial(fb.Tensor.from_slice(device, w.q.shape, w.q, 1), w.scale)
        parts.append(p.as_slice())
        lo, hi = r * (4096 + 160) // world, (r + 1) * (4096 + 160) // world
        want = O.attention_partial(full.q, full.k_dense[0][None], full.v_dense[0][None], full.scale, lo, hi)[:, :, 0]
        got = parts[-1]
        assert np.abs(got[..., 0] - want[..., 0]).max() < 1e-4          # m
        assert np.abs(got[..., 1] / want[..., 1] - 1).max() < 2e-3      # l
        assert np.abs(got[..., 2:] - want[..., 2:]).max() < 2e-2 * np.abs(want[..., 2:]).max()
    stacked = fb.Tensor.from_slice(device, (world,) + parts[0].shape, np.stack(parts))
    got = lse_combine(device, stacked).as_slice()
    want = O.flash_attention(full.q, full.k_dense[0][None], full.v_dense[0][None], full.scale)[:, :, 0]
    assert_close(got, want, what="chunked decode + combine")
    # an empty part is a no-op
    empty = np.zeros_like(parts[0])
    empty[..., 0] = -np.inf
    stacked = fb.Tensor.from_slice(device, (world + 1,) + parts[0].shape, np.stack(parts + [empty]))
    assert np.array_equal(lse_combine(device, stacked).as_slice(), got)


def test_kv_cache_append_reset_like_the_reference(device):
    """test_kv_cache_first_append / _multiple_appends / _reset (fusor/src/cache/kv_cache.rs:70-158), with the
    sequence on axis 2 of [B, Hkv, S, D] as kalosm-llama uses the cache."""
    fb = _fb()
    D = 128
    cache = fb.KvCache.new(2, 64)
    # values exactly representable in bf16: the cache stores bf16
    k1 = np.arange(D, dtype=np.float32).reshape(1, 1, 1, D)
    v1 = k1 * np.float32(0.5)
    k, v = cache.append(device, fb.Tensor.from_slice(device, k1.shape, k1), fb.Tensor.from_slice(device, v1.shape, v1))
    assert k.shape() == (1, 1, 1, D) and v.shape() == (1, 1, 1, D)
    assert np.array_equal(k.as_slice(), k1) and np.array_equal(v.as_slice(), v1)
    k2, v2 = k1 + 128, v1 + 64
    k, v = cache.append(device, fb.Tensor.from_slice(device, k2.shape, k2), fb.Tensor.from_slice(device, v2.shape, v2))
    assert k.shape() == (1, 1, 2, D) and cache.current_seq_len() == 2
    assert np.array_equal(k.as_slice(), np.concatenate([k1, k2], 2)) and np.array_equal(v.as_slice(), np.concatenate([v1, v2], 2))
    cache.reset()
    assert cache.k() is None and cache.v() is None and cache.current_seq_len() == 0


def test_kv_cache_growth_eviction_matches_tensor_cache_semantics(device):
    """Append / evict sequences against the numpy restatement of TensorCache (tensor_cache.rs:48-118)."""
    fb = _fb()
    rng = np.random.default_rng(3)
    B, Hkv, D, mx = 2, 2, 64, 50
    cache, ref = fb.KvCache.new(2, mx), O.KvCacheOracle(2, mx)
    for n in [1, 7, 16, 1, 20, 9, 33, 60, 2]:
        k = O.bf16_round(rng.standard_normal((B, Hkv, n, D), dtype=np.float32))
        v = O.bf16_round(rng.standard_normal((B, Hkv, n, D), dtype=np.float32))
        gk, gv = cache.append(device, fb.Tensor.from_slice(device, k.shape, k), fb.Tensor.from_slice(device, v.shape, v))
        rk, rv = ref.append(k, v)
        assert cache.current_seq_len() == ref.current_seq_len()
        assert gk.shape() == rk.shape
        assert np.array_equal(gk.as_slice(), rk) and np.array_equal(gv.as_slice(), rv), f"after append of {n}"


def test_decode_through_the_reference_call_pattern(device):
    """LlamaAttention::forward's sequence (attention_layer.rs:405-448): prefill appends S tokens and attends with the
    causal mask; every decode step appends one token and attends with get_mask(1, index_pos)."""
    fb = _fb()
    rng = np.random.default_rng(21)
    B, Hq, Hkv, D, S, steps = 1, 8, 2, 128, 70, 5
    scale = float(1 / np.sqrt(D))
    ks = O.bf16_round(rng.standard_normal((B, Hkv, S + steps, D), dtype=np.float32))
    vs = O.bf16_round(rng.standard_normal((B, Hkv, S + steps, D), dtype=np.float32))
    qs = O.bf16_round(rng.standard_normal((B, Hq, S + steps, D), dtype=np.float32))
    cache, masks = fb.KvCache.new(2, 4096), fb.MaskCache()
    T = lambda a: fb.Tensor.from_slice(device, a.shape, np.ascontiguousarray(a))
    k, v = cache.append(device, T(ks[:, :, :S]), T(vs[:, :, :S]))
    out = T(qs[:, :, :S]).flash_attention(k, v, scale, (masks.get_mask(S, 0, None, device), fb.MaskKind.QKMask)).as_slice()
    assert_close(out, O.flash_attention(qs[:, :, :S], ks[:, :, :S], vs[:, :, :S], scale, mask_kind=O.MASK_CAUSAL), what="prefill via cache")
    for t in range(S, S + steps):
        k, v = cache.append(device, T(ks[:, :, t:t + 1]), T(vs[:, :, t:t + 1]))
        before = device.launch_count()
        out = T(qs[:, :, t:t + 1]).flash_attention(k, v, scale, (masks.get_mask(1, t, None, device), fb.MaskKind.QKMask)).as_slice()
        assert device.launch_count() - before == 2  # split-KV kernel + merge of its records: the pages are read in place, nothing is planned on the host
        want = O.flash_attention(qs[:, :, t:t + 1], ks[:, :, :t + 1], vs[:, :, :t + 1], scale)
        assert_close(out, want, what=f"decode step {t}")
    # chunked continuation: 3 new tokens on a warm cache (structured.rs:143-150)
    cache2 = fb.KvCache.new(2, 4096)
    cache2.append(device, T(ks[:, :, :S]), T(vs[:, :, :S]))
    k, v = cache2.append(device, T(ks[:, :, S:S + 3]), T(vs[:, :, S:S + 3]))
    out = T(qs[:, :, S:S + 3]).flash_attention(k, v, scale, (masks.get_mask(3, S, None, device), fb.MaskKind.QKMask)).as_slice()
    want = O.flash_attention(qs[:, :, S:S + 3], ks[:, :, :S + 3], vs[:, :, :S + 3], scale, mask_kind=O.MASK_CAUSAL)
    assert_close(out, want, what="chunked continuation")


def test_bad_page_table_is_rejected_on_the_host(device):
    fb = _fb()
    cache = fb.PagedKvCache(device, 1, 1, 128, 4, 4)
    with pytest.raises(fb.FusorCudaError, match="outside the pool"):
        cache.set_page_table(np.array([[0, 9, 0, 0]], np.int32), np.array([20], np.int32))
    with pytest.raises(fb.FusorCudaError, match="mapped twice"):
        cache.set_page_table(np.array([[1, 1, 0, 0]], np.int32), np.array([20], np.int32))
    with pytest.raises(fb.FusorCudaError):
        fb.PagedKvCache(device, 1, 1, 128, 2, 2).append(fb.Tensor.zeros(device, (1, 1, 40, 128)), fb.Tensor.zeros(device, (1, 1, 40, 128)))


def test_cfg3_full_size(device):
    """BASELINE config 3 at full size: B64, Hq32, Hkv8, D128, kv_len ~ U[1024, 8192], permuted pages."""
    fb = _fb()
    from oracle import workloads as W
    w = W.cfg3()
    cache = _install(device, w)
    got = cache.decode(fb.Tensor.from_slice(device, w.q.shape, w.q, 1), w.scale).as_slice()
    assert_close(got, _oracle_decode(w), what="cfg3 full")


def test_bounded_wait_reports_timeout_and_context_survives(device):
    """Failure detection without a GPU fault: a wait on a barrier nothing signals runs out (about a second), the
    kernel returns, the host sees TIMEOUT, and the same context computes correctly afterwards."""
    import ctypes
    fb = _fb()
    from floneum_b200 import _lib
    L = _lib.load()
    rc = L.fusor_cuda_selftest_wait_limit(device.handle)
    assert rc == _lib.TIMEOUT
    assert b"wait site 99" in L.fusor_cuda_last_error(device.handle)
    device.synchronize()  # the error word was cleared; the stream is healthy
    q = np.ones((1, 2, 4, 16), np.float32)
    out = fb.Tensor.from_slice(device, q.shape, q).flash_attention(fb.Tensor.from_slice(device, q.shape, q),
                                                                   fb.Tensor.from_slice(device, q.shape, q), 0.25).as_slice()
    assert np.allclose(out, 1.0, atol=1e-6)


def test_session_export_import_round_trip(device):
    """KvCache.export_session / import_session (the reference's session save of the cache is stubbed out,
    models/kalosm-llama/src/session.rs:51-69): the re-imported cache holds the same rows and decodes to the same bits."""
    from floneum_b200 import KvCache, Tensor
    rng = np.random.default_rng(21)
    B, Hq, Hkv, D = 2, 8, 2, 128
    cache = KvCache.new(2, 96)
    for n in (70, 1, 40):  # the last append overflows max_sequence_len: the oldest rows are dropped
        k = O.bf16_round(rng.standard_normal((B, Hkv, n, D)).astype(np.float32))
        v = O.bf16_round(rng.standard_normal((B, Hkv, n, D)).astype(np.float32))
        ck, cv = cache.append(device, Tensor.from_slice(device, k.shape, k), Tensor.from_slice(device, v.shape, v))
    assert cache.current_seq_len() == 96
    sess = cache.export_session()
    assert sess["k"].shape == (B, Hkv, 96, D)
    again = KvCache.import_session(device, sess)
    assert again.current_seq_len() == 96
    s2 = again.export_session()
    assert np.array_equal(s2["k"], sess["k"]) and np.array_equal(s2["v"], sess["v"])
    q = O.bf16_round(rng.standard_normal((B, Hq, 1, D)).astype(np.float32))
    tq = Tensor.from_slice(device, q.shape, q)
    a = tq.flash_attention(ck, cv, D ** -0.5).as_slice()
    b = tq.flash_attention(again.k(), again.v(), D ** -0.5).as_slice()
    assert np.array_equal(a, b)
    assert_close(a, O.flash_attention(q, sess["k"], sess["v"], D ** -0.5))


def test_peer_exchange_world_of_one_merges_like_lse_combine(device):
    """The peer-memory exchange with a single rank: the push goes to the rank's own slots, the merge waits for its own
    epoch; repeated steps alternate the slot parity.  (Two or more ranks need as many GPUs: bench.py --workload cfg4.)"""
    from floneum_b200 import Tensor
    from floneum_b200.sharding import PeerExchange
    rng = np.random.default_rng(33)
    rows, D = 64, 128
    ex = PeerExchange(device, 0, 1, rows * (D + 2))
    for step in range(3):
        rec = rng.standard_normal((rows, D + 2)).astype(np.float32)
        rec[:, 1] = np.abs(rec[:, 1]) + 0.5
        out = Tensor.zeros(device, (rows, D))
        ex.lse_combine(Tensor.from_slice(device, rec.shape, rec), out)
        got = out.as_slice()
        want = O.lse_combine(rec[None])
        assert np.abs(got - want).max() < 1e-5, step
    ex.close()


@pytest.mark.parametrize("ctas", [1, 3, 37, 148, 592])
def test_decode_grid_sizes_give_the_same_answer(device, ctas):
    """The deal of pages to CTAs is computed inside the kernel from the lengths on the device: any grid size must merge to
    the same attention (1 CTA: every sequence-head is whole inside it and written by it; 592: most are spread over several
    CTAs and merged by the second kernel, which finds their records with the same deal)."""
    fb = _fb()
    from oracle import workloads as W
    w = W.cfg3(B=6, Hq=16, Hkv=4, lo=30, hi=2500)
    cache = _install(device, w)
    cache.set_decode_ctas(ctas)
    q = fb.Tensor.from_slice(device, w.q.shape, w.q, 1)
    want = _oracle_decode(w)
    runs = [cache.decode(q, w.scale).as_slice() for _ in range(3)]
    assert_close(runs[0], want, what=f"decode with {ctas} CTAs")
    # the records of a head are merged in slot order whichever CTA does it: repeated steps agree bit for bit
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    # 16-bit outputs and an f16 query tensor
    got_bf16 = cache.decode(q, w.scale, out_dtype=1).as_slice()
    assert_close(got_bf16, O.bf16_round(want), max_tol=2e-3 + 2.0 ** -7, mean_tol=2e-3, what="bf16 out")
    # the bf16-representable q values are f16-representable too (normal range): same inputs, f16 output rounding on top
    got_f16 = cache.decode(fb.Tensor.from_slice(device, w.q.shape, w.q, 2), w.scale, out_dtype=2).as_slice()
    assert_close(got_f16, want, max_tol=2e-3 + 2.0 ** -10, mean_tol=4e-4, what="f16 q and out")


def test_live_decode_steps_need_no_plan(device):
    """Append one token per sequence and decode, 40 times, lengths crossing page boundaries at different steps: the kernel
    reads the lengths the append uploaded, nothing else is planned or uploaded per step."""
    fb = _fb()
    rng = np.random.default_rng(77)
    B, Hq, Hkv, D = 3, 8, 2, 128
    cache = fb.PagedKvCache(device, B, Hkv, D, num_pages=64, max_pages_per_seq=16)
    n0 = 9
    ks = [O.bf16_round(rng.standard_normal((B, Hkv, n0, D)).astype(np.float32))]
    vs = [O.bf16_round(rng.standard_normal((B, Hkv, n0, D)).astype(np.float32))]
    cache.append(fb.Tensor.from_slice(device, ks[0].shape, ks[0]), fb.Tensor.from_slice(device, vs[0].shape, vs[0]))
    for step in range(40):
        k1 = O.bf16_round(rng.standard_normal((B, Hkv, 1, D)).astype(np.float32))
        v1 = O.bf16_round(rng.standard_normal((B, Hkv, 1, D)).astype(np.float32))
        ks.append(k1); vs.append(v1)
        cache.append(fb.Tensor.from_slice(device, k1.shape, k1), fb.Tensor.from_slice(device, v1.shape, v1))
        q = O.bf16_round(rng.standard_normal((B, Hq, 1, D)).astype(np.float32))
        got = cache.decode(fb.Tensor.from_slice(device, q.shape, q, 1), D ** -0.5).as_slice()
        want = O.flash_attention(q, np.concatenate(ks, 2), np.concatenate(vs, 2), D ** -0.5)
        assert_close(got, want, what=f"live decode step {step}")


def test_decode_partial_of_empty_chunks(device):
    """A sequence shorter than the number of ranks leaves some ranks an empty KV chunk: their partial record is the empty
    one {-inf, 0, 0...}, the merge over all chunks equals attention over the whole sequence, and the normalising decode
    still rejects an empty sequence (attention over no keys has no value) without harming the context."""
    fb = _fb()
    from floneum_b200 import _lib
    from floneum_b200.cache import lse_combine
    from floneum_b200.sharding import kv_chunk_range
    rng = np.random.default_rng(91)
    B, Hq, Hkv, D, world = 3, 8, 2, 128, 8
    lens = [5, 0, 37]  # sequence 1 holds nothing anywhere: zeros after the merge
    k = [O.bf16_round(rng.standard_normal((Hkv, n, D)).astype(np.float32)) for n in lens]
    v = [O.bf16_round(rng.standard_normal((Hkv, n, D)).astype(np.float32)) for n in lens]
    qn = O.bf16_round(rng.standard_normal((B, Hq, 1, D)).astype(np.float32))
    q = fb.Tensor.from_slice(device, qn.shape, qn, 1)
    scale = D ** -0.5
    parts = []
    for r in range(world):
        cache = fb.PagedKvCache(device, B, Hkv, D, num_pages=8, max_pages_per_seq=2)
        table = np.zeros((B, 2), np.int32)
        kp = np.zeros((8, Hkv, 16, D), np.float32)
        vp = np.zeros_like(kp)
        mine, page = [], 0
        for b in range(B):
            lo, hi = kv_chunk_range(lens[b], r, world)
            mine.append(hi - lo)
            for j in range((hi - lo + 15) // 16):
                n = min(16, hi - lo - 16 * j)
                kp[page, :, :n] = k[b][:, lo + 16 * j:lo + 16 * j + n]
                vp[page, :, :n] = v[b][:, lo + 16 * j:lo + 16 * j + n]
                table[b, j] = page
                page += 1
        cache.write_pages(0, O.bf16_bits(kp), O.bf16_bits(vp))
        cache.set_page_table(table, np.array(mine, np.int32))
        rec = cache.decode_partial(q, scale).as_slice()
        for b in range(B):
            if mine[b] == 0:
                assert np.all(rec[b, :, 0] == -np.inf) and np.all(rec[b, :, 1:] == 0), (r, b)
            else:
                lo, hi = kv_chunk_range(lens[b], r, world)
                want = O.attention_partial(qn[b:b + 1], k[b][None], v[b][None], scale, lo, hi)[0, :, 0]
                assert np.abs(rec[b, :, 0] - want[:, 0]).max() < 1e-4 and np.abs(rec[b, :, 1] / want[:, 1] - 1).max() < 2e-3
        if any(n == 0 for n in mine):
            with pytest.raises(fb.FusorCudaError) as e:
                cache.decode(q, scale)
            assert e.value.code == _lib.INVALID_ARGUMENT and "empty" in str(e.value)
        parts.append(rec)
        cache.close()
    merged = lse_combine(device, fb.Tensor.from_slice(device, (world,) + parts[0].shape, np.stack(parts))).as_slice()
    for b in range(B):
        if lens[b] == 0:
            assert np.all(merged[b] == 0)
        else:
            want = O.flash_attention(qn[b:b + 1], k[b][None], v[b][None], scale)[0, :, 0]
            assert_close(merged[b], want, what=f"sequence {b} of {lens[b]} keys in {world} chunks")


def test_cfg4_full_size_eight_chunks_on_one_gpu(device):
    """BASELINE config 4 at full size (B1 Hq64 Hkv8 D128, 131072 keys) on one GPU: the whole sequence in one call, and as
    the 8 contiguous KV chunks of the multi-GPU partition, each through decode_partial, merged by lse_combine and by the
    peer exchange's own merge (world of one per chunk is not a merge: the records go through fusor_cuda_lse_combine)."""
    fb = _fb()
    from oracle import workloads as W
    from floneum_b200.cache import lse_combine
    w = W.cfg4()
    want = O.flash_attention(w.q, w.k_dense[0][None], w.v_dense[0][None], w.scale)
    cache = _install(device, w)
    q = fb.Tensor.from_slice(device, w.q.shape, w.q, 1)
    got = cache.decode(q, w.scale).as_slice()
    assert_close(got, want, what="cfg4 whole sequence")
    cache.close()
    world, npg = 8, w.k_pages.shape[0]
    per = npg // world
    parts = []
    for r in range(world):
        c = fb.PagedKvCache(device, 1, 8, 128, per, per)
        c.write_pages(0, w.k_pages[r * per:(r + 1) * per], w.v_pages[r * per:(r + 1) * per])
        c.set_page_table(np.arange(per, dtype=np.int32)[None], np.array([per * 16], np.int32))
        parts.append(c.decode_partial(q, w.scale).as_slice())
        c.close()
    stacked = fb.Tensor.from_slice(device, (world,) + parts[0].shape, np.stack(parts))
    merged = lse_combine(device, stacked).as_slice()
    assert_close(merged, want[:, :, 0], what="cfg4 in 8 chunks")
    # an oracle restatement of the same merge on the records the GPU produced
    assert np.abs(merged - O.lse_combine(np.stack(parts).reshape(world, -1, 130)).reshape(merged.shape)).max() < 1e-5


def test_lse_combine_of_empty_rows_gives_zeros(device):
    """A row whose parts are all empty (l == 0) has no keys to attend to: the merge writes zeros, not 0/0."""
    fb = _fb()
    from floneum_b200.cache import lse_combine
    from floneum_b200.sharding import PeerExchange
    parts = np.zeros((3, 4, 18), np.float32)
    parts[..., 0] = -np.inf
    parts[1, 2] = np.arange(18, dtype=np.float32) + 1  # one live record in row 2
    got = lse_combine(device, fb.Tensor.from_slice(device, parts.shape, parts)).as_slice()
    assert np.array_equal(got[[0, 1, 3]], np.zeros((3, 16), np.float32))
    assert np.allclose(got[2], parts[1, 2, 2:] / parts[1, 2, 1])
    ex = PeerExchange(device, 0, 1, 4 * 18 + 0)
    out = fb.Tensor.from_slice(device, (4, 16), np.ones((4, 16), np.float32))
    ex.lse_combine(fb.Tensor.from_slice(device, (4, 18), parts[0]), out)
    assert np.array_equal(out.as_slice(), np.zeros((4, 16), np.float32))
    ex.close()


def test_exchange_decode_world_of_one(device):
    """fusor_cuda_exchange_decode with a single rank: the merge kernel stores the rank's merged records into its own
    slot, publishes, waits for its own epoch and merges.  Three steps: both slot parities."""
    fb = _fb()
    from oracle import workloads as W
    from floneum_b200.sharding import PeerExchange
    w = W.cfg4(Skv=6000, Hq=32, Hkv=4)
    cache = _install(device, w)
    B, Hq, _, D = w.q.shape
    ex = PeerExchange(device, 0, 1, B * Hq * (D + 2))
    q = fb.Tensor.from_slice(device, w.q.shape, w.q, 1)
    want = O.flash_attention(w.q, w.k_dense[0][None], w.v_dense[0][None], w.scale)[:, :, 0]
    for ctas in (0, 5, 0):
        cache.set_decode_ctas(ctas)
        out = fb.Tensor.zeros(device, (B, Hq, D))
        ex.decode(cache, q, w.scale, out)
        assert_close(out.as_slice(), want, what=f"exchange decode, {ctas} CTAs")
    # a rank whose chunk of every sequence is empty only runs the merge kernel: its records are the empty ones, and with
    # no other rank the merged result is zeros (two steps: both slot parities again)
    none = fb.PagedKvCache(device, B, w.k_pages.shape[1], D, num_pages=2, max_pages_per_seq=1)
    none.set_page_table(np.zeros((B, 1), np.int32), np.zeros(B, np.int32))
    for _ in range(2):
        out = fb.Tensor.from_slice(device, (B, Hq, D), np.full((B, Hq, D), 7.0, np.float32))
        before = device.launch_count()
        ex.decode(none, q, w.scale, out)
        assert device.launch_count() - before == 1
        assert np.all(out.as_slice() == 0)
    none.close()
    ex.close()


def test_token_granular_eviction_is_two_launches(device):
    """TensorCache eviction at full cache (tensor_cache.rs:55-78) drops one token per decode step: the kept rows move
    with two kernel launches whatever the length, and the cache then holds the newest rows."""
    fb = _fb()
    rng = np.random.default_rng(5)
    B, Hkv, D, n = 2, 4, 128, 200
    cache = fb.PagedKvCache(device, B, Hkv, D, num_pages=40, max_pages_per_seq=16)
    k = O.bf16_round(rng.standard_normal((B, Hkv, n, D)).astype(np.float32))
    v = O.bf16_round(rng.standard_normal((B, Hkv, n, D)).astype(np.float32))
    cache.append(fb.Tensor.from_slice(device, k.shape, k), fb.Tensor.from_slice(device, v.shape, v))
    cache.truncate_front(0, n - 3)  # first use allocates the staging buffer
    before = device.launch_count()
    cache.truncate_front(1, n - 3)
    assert device.launch_count() - before == 2
    gk, gv = cache.gather(B, n - 3)
    assert np.array_equal(gk.as_slice(), k[:, :, 3:]) and np.array_equal(gv.as_slice(), v[:, :, 3:])
    before = device.launch_count()
    cache.truncate_front(0, n - 3 - 32)  # whole pages: table edit only
    assert device.launch_count() == before
    assert np.array_equal(cache.gather(B, n - 3)[0].as_slice()[0, :, :n - 35], k[0, :, 35:])


def test_llama_cache_layers_keep_their_own_lengths(device):
    """LlamaCache (models/kalosm-llama/src/raw/cache.rs:14-54): sliding layers keep `sliding_window_size` tokens, every
    `sliding_window_type`-th layer the whole context."""
    from floneum_b200 import LlamaCache, Tensor
    rng = np.random.default_rng(9)
    cache = LlamaCache(n_layer=4, context_length=96, sliding_window_type=2, sliding_window_size=24)
    assert [b.max_sequence_len for b in cache.blocks] == [24, 96, 24, 96]
    ks = []
    for step_len in (20, 10, 1, 1):
        k = O.bf16_round(rng.standard_normal((1, 2, step_len, 128)).astype(np.float32))
        ks.append(k)
        for block in cache.blocks:
            block.append(device, Tensor.from_slice(device, k.shape, k), Tensor.from_slice(device, k.shape, k))
    allk = np.concatenate(ks, 2)
    assert [b.current_seq_len() for b in cache.blocks] == [24, 32, 24, 32]
    assert np.array_equal(cache.blocks[0].k().as_slice(), allk[:, :, -24:])
    assert np.array_equal(cache.blocks[1].k().as_slice(), allk)
    cache.clear()
    assert [b.current_seq_len() for b in cache.blocks] == [0, 0, 0, 0]
