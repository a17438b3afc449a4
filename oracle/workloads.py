"""Seeded synthetic inputs for the five benchmark / parity configurations.

No public dataset is involved: the shapes are Llama-3-8B / 70B *attention shapes* and the
values are drawn from numpy's PCG64 (`default_rng(1000 + config)`), in the order Q, K, V,
then lengths, page permutation and outlier rows.  bf16 configurations are rounded to
nearest-even once on the host and the same rounded values feed both the oracle and the GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

PAGE_TOKENS = 16


def bf16_round(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(a.shape)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


@dataclass
class PrefillWorkload:
    name: str
    q: np.ndarray  # f32 [B,Hq,S,D] (bf16-representable when bf16 is True)
    k: np.ndarray
    v: np.ndarray
    scale: float
    bf16: bool

    @property
    def flops(self) -> float:
        """Algorithmic causal FLOPs: 4 B Hq D S(S+1)/2."""
        B, Hq, S, D = self.q.shape
        return 4.0 * B * Hq * D * S * (S + 1) / 2


@dataclass
class DecodeWorkload:
    name: str
    q: np.ndarray          # f32 [B,Hq,1,D], bf16-representable
    k_pages: np.ndarray    # uint16 bf16 bits [num_pages,Hkv,16,D]
    v_pages: np.ndarray
    page_table: np.ndarray  # int32 [B,max_pages]
    kv_len: np.ndarray      # int32 [B]
    scale: float
    k_dense: Optional[list] = field(default=None)  # per-sequence f32 [Hkv,len,D] (for the oracle)
    v_dense: Optional[list] = field(default=None)

    @property
    def bytes(self) -> float:
        """Algorithmic bytes: K+V bf16 once, q bf16 in + out f32, page-table entries."""
        B, Hq, _, D = self.q.shape
        Hkv = self.k_pages.shape[1]
        pages = int(np.sum((self.kv_len + PAGE_TOKENS - 1) // PAGE_TOKENS))
        return float(np.sum(self.kv_len)) * 2 * Hkv * D * 2 + B * Hq * D * 6 + 4 * pages


def _normal(rng, shape, sigma=1.0):
    a = rng.standard_normal(shape, dtype=np.float32)
    return a if sigma == 1.0 else (np.float32(sigma) * a)


def cfg1(S: int = 512) -> PrefillWorkload:
    """CPU-reference config: B1 S512 Hq32 Hkv8 D64 f32 N(0,1), causal, scale 1/8."""
    rng = np.random.default_rng(1001)
    q, k, v = _normal(rng, (1, 32, S, 64)), _normal(rng, (1, 8, S, 64)), _normal(rng, (1, 8, S, 64))
    return PrefillWorkload("cfg1", q, k, v, 0.125, False)


def cfg2(B: int = 4, S: int = 4096, Hq: int = 32, Hkv: int = 8) -> PrefillWorkload:
    """Llama-3-8B prefill: B4 S4096 Hq32 Hkv8 D128 bf16 N(0,1), causal, scale 1/sqrt(128)."""
    rng = np.random.default_rng(1002)
    q, k, v = (bf16_round(_normal(rng, (B, Hq, S, 128))), bf16_round(_normal(rng, (B, Hkv, S, 128))),
               bf16_round(_normal(rng, (B, Hkv, S, 128))))
    return PrefillWorkload("cfg2", q, k, v, float(1.0 / np.sqrt(128.0)), True)


def cfg5(S: int = 16384, Hq: int = 64, Hkv: int = 8) -> PrefillWorkload:
    """Llama-3-70B long prefill: B1 S16384 Hq64 Hkv8 D128 bf16 N(0,0.5^2), 5% of K rows x8."""
    rng = np.random.default_rng(1005)
    q, k, v = _normal(rng, (1, Hq, S, 128), 0.5), _normal(rng, (1, Hkv, S, 128), 0.5), _normal(rng, (1, Hkv, S, 128), 0.5)
    outlier = rng.random((1, Hkv, S)) < 0.05
    k = np.where(outlier[..., None], k * np.float32(8.0), k)
    return PrefillWorkload("cfg5", bf16_round(q), bf16_round(k), bf16_round(v), float(1.0 / np.sqrt(128.0)), True)


def _paged(name, rng, B, Hq, Hkv, D, kv_len, permute, keep_dense):
    pages_per = (kv_len + PAGE_TOKENS - 1) // PAGE_TOKENS
    total = int(pages_per.sum())
    max_pages = int(pages_per.max())
    q = bf16_round(_normal(rng, (B, Hq, 1, D)))
    # values are drawn per sequence in logical order, then scattered to physical pages
    kd = [bf16_round(_normal(rng, (Hkv, int(n), D))) for n in kv_len]
    vd = [bf16_round(_normal(rng, (Hkv, int(n), D))) for n in kv_len]
    phys = rng.permutation(total).astype(np.int32) if permute else np.arange(total, dtype=np.int32)
    page_table = np.zeros((B, max_pages), np.int32)
    k_pages = np.zeros((total, Hkv, PAGE_TOKENS, D), np.uint16)
    v_pages = np.zeros((total, Hkv, PAGE_TOKENS, D), np.uint16)
    cur = 0
    for b in range(B):
        npg = int(pages_per[b])
        ids = phys[cur:cur + npg]
        cur += npg
        page_table[b, :npg] = ids
        pad = npg * PAGE_TOKENS - int(kv_len[b])
        kb = np.pad(kd[b], ((0, 0), (0, pad), (0, 0))).reshape(Hkv, npg, PAGE_TOKENS, D).transpose(1, 0, 2, 3)
        vb = np.pad(vd[b], ((0, 0), (0, pad), (0, 0))).reshape(Hkv, npg, PAGE_TOKENS, D).transpose(1, 0, 2, 3)
        k_pages[ids] = bf16_bits(kb)
        v_pages[ids] = bf16_bits(vb)
    return DecodeWorkload(name, q, k_pages, v_pages, page_table, kv_len.astype(np.int32), float(1.0 / np.sqrt(D)),
                          kd if keep_dense else None, vd if keep_dense else None)


def cfg3(B: int = 64, Hq: int = 32, Hkv: int = 8, lo: int = 1024, hi: int = 8192, keep_dense: bool = True) -> DecodeWorkload:
    """Llama-3-8B paged decode: B64, one query token, kv_len ~ U[1024, 8192], 16-token pages, permuted table."""
    rng = np.random.default_rng(1003)
    # draw order: lengths first so the tensor shapes are known, then Q, K, V, then the permutation
    kv_len = rng.integers(lo, hi + 1, size=B)
    return _paged("cfg3", rng, B, Hq, Hkv, 128, kv_len, True, keep_dense)


def cfg4(Skv: int = 131072, Hq: int = 64, Hkv: int = 8, rank: int = 0, world: int = 1, keep_dense: bool = True) -> DecodeWorkload:
    """Long-context decode: B1 Hq64 Hkv8 D128 Skv131072; rank r of `world` holds keys [r*Skv/world, (r+1)*Skv/world)."""
    rng = np.random.default_rng(1004)
    D = 128
    q = bf16_round(_normal(rng, (1, Hq, 1, D)))
    k = bf16_round(_normal(rng, (Hkv, Skv, D)))
    v = bf16_round(_normal(rng, (Hkv, Skv, D)))
    lo, hi = rank * Skv // world, (rank + 1) * Skv // world
    n = hi - lo
    npg = (n + PAGE_TOKENS - 1) // PAGE_TOKENS
    pad = npg * PAGE_TOKENS - n
    kb = np.pad(k[:, lo:hi], ((0, 0), (0, pad), (0, 0))).reshape(Hkv, npg, PAGE_TOKENS, D).transpose(1, 0, 2, 3)
    vb = np.pad(v[:, lo:hi], ((0, 0), (0, pad), (0, 0))).reshape(Hkv, npg, PAGE_TOKENS, D).transpose(1, 0, 2, 3)
    page_table = np.arange(npg, dtype=np.int32)[None, :]
    return DecodeWorkload("cfg4", q, bf16_bits(kb), bf16_bits(vb), page_table, np.array([n], np.int32),
                          float(1.0 / np.sqrt(D)), [k[:, lo:hi]] if keep_dense else None, [v[:, lo:hi]] if keep_dense else None)
