"""Output projection after attention (tcgen05 GEMM reading the [B,Hq,S,D] attention output in place) against the oracle.

bf16 inputs, f32 accumulation: the only difference from the oracle is the summation order inside the tensor core, so the
tolerance is relative to the magnitude of the sum (K up to 4096 terms of size ~1): 1e-3 of sqrt(K), far below one bf16 ulp
of the inputs' contribution."""
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _case(seed, B, Hq, S, D, N, bias=True):
    rng = np.random.default_rng(seed)
    attn = O.bf16_round(rng.standard_normal((B, Hq, S, D)).astype(np.float32))
    w = O.bf16_round((rng.standard_normal((N, Hq * D)) / np.sqrt(Hq * D)).astype(np.float32))
    b = rng.standard_normal(N).astype(np.float32) if bias else None
    return attn, w, b


def _run(device, attn, w, b, out_dtype=0):
    from floneum_b200 import Tensor
    from floneum_b200.tensor import BF16
    ta = Tensor.from_slice(device, attn.shape, attn, BF16)
    tw = Tensor.from_slice(device, w.shape, w, BF16)
    tb = Tensor.from_slice(device, b.shape, b) if b is not None else None
    return ta.out_proj(tw, tb, out_dtype).as_slice()


@pytest.mark.parametrize("B,Hq,S,D,N,bias", [
    (1, 2, 128, 128, 256, True),      # one tile, 4 K steps
    (2, 4, 200, 128, 512, False),     # ragged rows, two n tiles
    (1, 8, 384, 64, 320, True),       # head_dim 64, n not a multiple of 256
    (2, 32, 512, 128, 1024, True),    # K = 4096, more tiles than... 2*4*4 = 32 tiles
    (1, 3, 77, 128, 40, True),        # everything ragged
    (3, 16, 1024, 128, 2048, False),  # 3*8*8 = 192 tiles > 148 SMs: persistent CTAs take two tiles, both accumulators
])
def test_out_proj_matches_oracle(device, B, Hq, S, D, N, bias):
    attn, w, b = _case(100 * S + N, B, Hq, S, D, N, bias)
    got = _run(device, attn, w, b)
    want = O.out_proj(attn, w, b)
    assert got.shape == (B, S, N)
    err = np.abs(got - want)
    assert err.max() <= 2e-4 and err.mean() <= 2e-5, (err.max(), err.mean())


def test_out_proj_bf16_output(device):
    attn, w, b = _case(5, 2, 8, 300, 128, 768)
    got32 = _run(device, attn, w, b)
    got16 = _run(device, attn, w, b, out_dtype=1)
    assert np.array_equal(got16.view(np.uint32), O.bf16_round(got32).view(np.uint32))


def test_out_proj_head_shards_add_up(device):
    """Tensor-parallel form: each shard of query heads with its columns of the weight gives a partial sum; the partial
    sums add up to the full projection (the all-reduce that follows attention when KV heads are split over GPUs)."""
    attn, w, b = _case(6, 1, 8, 256, 128, 512)
    full = _run(device, attn, w, b)
    D = 128
    parts = []
    for r in range(2):
        hs = slice(4 * r, 4 * r + 4)
        parts.append(_run(device, attn[:, hs], np.ascontiguousarray(w[:, 4 * r * D:(4 * r + 4) * D]), b if r == 0 else None))
    assert np.abs(parts[0] + parts[1] - full).max() <= 1e-4


def test_out_proj_after_attention(device):
    """flash_attention (bf16 out) -> out_proj, against the oracle chain on the same rounded intermediate."""
    from floneum_b200 import MaskCache, MaskKind, Tensor
    from floneum_b200.tensor import BF16
    rng = np.random.default_rng(8)
    B, Hq, Hkv, S, D, N = 1, 8, 2, 256, 128, 512
    q, k, v = (O.bf16_round(rng.standard_normal((B, h, S, D)).astype(np.float32)) for h in (Hq, Hkv, Hkv))
    w = O.bf16_round((rng.standard_normal((N, Hq * D)) / 32).astype(np.float32))
    tq, tk, tv = (Tensor.from_slice(device, a.shape, a, BF16) for a in (q, k, v))
    mask = (MaskCache().get_mask(S, 0, None, device), MaskKind.QKMask)
    attn = tq.flash_attention(tk, tv, D ** -0.5, mask, BF16)
    got = attn.out_proj(Tensor.from_slice(device, w.shape, w, BF16)).as_slice()
    want = O.out_proj(attn.as_slice(), w)
    assert np.abs(got - want).max() <= 2e-4


def test_out_proj_argument_checks(device):
    from floneum_b200 import FusorCudaError, Tensor
    from floneum_b200.tensor import BF16
    a = Tensor.zeros(device, (1, 2, 16, 128), BF16)
    with pytest.raises(AssertionError):
        a.out_proj(Tensor.zeros(device, (64, 128), BF16))          # in_features != Hq * D
    with pytest.raises(FusorCudaError):
        Tensor.zeros(device, (1, 2, 16, 128)).out_proj(Tensor.zeros(device, (64, 256), BF16))  # f32 attention output
