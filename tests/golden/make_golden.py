"""Writes the golden fixtures in this folder.

The reference (Rust; no toolchain here) cannot be run, so the fixtures are (a) the literal
inputs of the reference's own attention tests with the composite's output, checked against
float64 softmax attention when generated, and (b) small seeded cases.  Run from the repo root:
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402
from oracle import workloads as W  # noqa: E402

NEG = float("-inf")


def f64(q, k, v, scale, mask=None):
    g = q.shape[1] // k.shape[1]
    tq, tk, tv = (torch.from_numpy(np.asarray(a, np.float64)) for a in (q, k, v))
    s = tq @ tk.repeat_interleave(g, 1).transpose(2, 3) * float(scale)
    if mask is not None:
        s = s + torch.from_numpy(np.asarray(mask, np.float64))
    return (torch.softmax(s, -1) @ tv.repeat_interleave(g, 1)).numpy()


def save(name, q, k, v, scale, mask_kind=O.MASK_NONE, mask=None, bmask=None):
    out = O.flash_attention(q, k, v, scale, mask, mask_kind)
    dense = None
    if mask_kind == O.MASK_QK:
        dense = mask
    elif mask_kind == O.MASK_BATCH_KEY:
        dense = mask[:, None, None, :]
    elif mask_kind == O.MASK_CAUSAL:
        dense = O.get_mask(q.shape[2], k.shape[2] - q.shape[2])
    assert np.abs(out - f64(q, k, v, scale, dense)).max() < 5e-6, name
    np.savez_compressed(os.path.join(HERE, name + ".npz"), q=q, k=k, v=v, scale=np.float32(scale), mask_kind=mask_kind,
                        mask=mask if mask is not None else np.zeros((0, 0), np.float32), out=out)


def main():
    s2 = np.float32(1.0 / np.sqrt(np.float32(2.0)))
    eye = np.array([1, 0, 0, 1], np.float32).reshape(1, 1, 2, 2)
    v = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2)
    save("ref_identity", eye, eye.copy(), v, s2)
    save("ref_identity_causal", eye, eye.copy(), v, s2, O.MASK_QK, np.array([[0, NEG], [0, 0]], np.float32))
    save("ref_gqa", (np.arange(16, dtype=np.float32) * np.float32(0.1)).reshape(1, 4, 2, 2),
         (np.arange(8, dtype=np.float32) * np.float32(0.1) + 1).reshape(1, 2, 2, 2),
         (np.arange(8, dtype=np.float32) * np.float32(0.1) + 2).reshape(1, 2, 2, 2), s2)
    save("ref_batch_key", (np.arange(12, dtype=np.float32) * np.float32(0.1)).reshape(2, 1, 3, 2),
         (np.arange(12, dtype=np.float32) * np.float32(0.1) + 1).reshape(2, 1, 3, 2),
         (np.arange(12, dtype=np.float32) * np.float32(0.1) + 2).reshape(2, 1, 3, 2), s2, O.MASK_BATCH_KEY,
         np.array([[0, 0, 0], [0, 0, NEG]], np.float32))
    rng = np.random.default_rng(2001)
    save("seeded_f32_gqa_causal", rng.standard_normal((2, 6, 37, 24), dtype=np.float32),
         rng.standard_normal((2, 2, 45, 24), dtype=np.float32), rng.standard_normal((2, 2, 45, 24), dtype=np.float32),
         np.float32(1 / np.sqrt(24)), O.MASK_CAUSAL)
    rng = np.random.default_rng(2002)
    save("seeded_bf16_d128_causal", W.bf16_round(rng.standard_normal((1, 4, 200, 128), dtype=np.float32)),
         W.bf16_round(rng.standard_normal((1, 2, 200, 128), dtype=np.float32)),
         W.bf16_round(rng.standard_normal((1, 2, 200, 128), dtype=np.float32)), np.float32(1 / np.sqrt(128)), O.MASK_CAUSAL)
    w = W.cfg3(B=3, Hq=8, Hkv=2, lo=20, hi=90)
    outs = [O.flash_attention(w.q[b:b + 1], w.k_dense[b][None], w.v_dense[b][None], w.scale)[0] for b in range(3)]
    np.savez_compressed(os.path.join(HERE, "seeded_decode_paged.npz"), q=w.q, k_pages=w.k_pages, v_pages=w.v_pages,
                        page_table=w.page_table, kv_len=w.kv_len, scale=np.float32(w.scale), out=np.stack(outs))


if __name__ == "__main__":
    main()
