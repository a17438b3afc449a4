"""ctypes front end of the CPU oracle (oracle/attention_oracle.c).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by ``__graft_entry__.smoke()`` and by
``bench.py``'s CPU-baseline / reference legs as the checker and the timed CPU baseline.
The product package (floneum_b200) never imports this module.

Besides the C composite it holds numpy restatements of the reference's host-side
cache logic, used as the expected behaviour in the cache tests:
  * TensorCacheOracle / KvCacheOracle: fusor-ml/fusor/src/cache/tensor_cache.rs:9-124,
    kv_cache.rs:12-68 (append / power-of-two growth / eviction / reset)
  * mask builders: fusor-ml/fusor/src/cache/attention_mask.rs:26-46,
    mask_cache.rs:36-116
Parity status: bit-level parity with the Rust reference is unpinned (its gemm is a
third-party crate and no Rust toolchain exists here); the known answers of the
reference's own tests are pinned in tests/test_oracle_pins.py.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libattention_oracle.so")

MASK_NONE, MASK_QK, MASK_BATCH_KEY, MASK_CAUSAL = 0, 1, 2, 3

_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the system gcc (see oracle/Makefile)."""
    src = os.path.join(_HERE, "attention_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libattention_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        fp = ctypes.POINTER(ctypes.c_float)
        i64p = ctypes.POINTER(ctypes.c_int64)
        L.oracle_attention_f32.argtypes = [fp, fp, fp, fp, ctypes.c_int, ctypes.c_int64, fp] + [ctypes.c_int] * 6 + [
            ctypes.c_float, i64p, ctypes.c_int64, ctypes.c_int]
        L.oracle_attention_f32.restype = ctypes.c_int
        L.oracle_attention_online_f32.argtypes = [fp, fp, fp, fp, fp] + [ctypes.c_int] * 6 + [ctypes.c_float]
        L.oracle_attention_online_f32.restype = ctypes.c_int
        L.oracle_causal_mask.argtypes = [fp, ctypes.c_int]
        L.oracle_sliding_window_mask.argtypes = [fp, ctypes.c_int, ctypes.c_int]
        L.oracle_lse_combine.argtypes = [fp, ctypes.c_int, ctypes.c_int64, ctypes.c_int, fp]
        L.oracle_attention_partial_f32.argtypes = [fp, fp, fp, fp] + [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_int,
                                                                                        ctypes.c_int]
        L.oracle_attention_partial_f32.restype = ctypes.c_int
        L.oracle_num_threads.restype = ctypes.c_int
        L.oracle_rope_f32.argtypes = [fp, fp, fp, fp] + [ctypes.c_int] * 6
        L.oracle_out_proj_f32.argtypes = [fp, fp, fp, fp] + [ctypes.c_int] * 5
        L.oracle_out_proj_f32.restype = ctypes.c_int
        L.oracle_rope_f32.restype = ctypes.c_int
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Sets the OpenMP thread count to the cores this process may run on (a launcher such as torchrun exports
    OMP_NUM_THREADS=1, which would make the CPU baseline single-threaded) and returns it."""
    import os
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) if a is not None else None


# --------------------------------------------------------------------------- numerics helpers
def bf16_round(a) -> np.ndarray:
    """Round f32 to the nearest bf16 (ties to even), returned as f32."""
    a = _f32(a)
    u = a.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32).reshape(a.shape)
    nan = np.isnan(a)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out


def bf16_bits(a) -> np.ndarray:
    """f32 values that are exactly representable in bf16 -> uint16 bit patterns."""
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- the composite
def flash_attention(q, k, v, scale, mask=None, mask_kind=MASK_NONE, causal_offset=None, rows=None,
                    skip_masked=False) -> np.ndarray:
    """The reference composite (flash_attention.rs:77-200) on f32 [B,H,S,D] arrays.

    mask_kind MASK_CAUSAL evaluates the 0/-inf mask of AttentionMask::causal padded by
    ``causal_offset`` (default Skv - Sq) analytically.  ``rows`` selects flat output rows
    ((b*Hq+h)*Sq+q, ascending) and returns [len(rows), D]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Hq, Sq, D = q.shape
    Bk, Hkv, Skv, Dk = k.shape
    assert (Bk, Dk) == (B, D) and v.shape == k.shape
    if Hq % Hkv != 0:
        raise AssertionError(
            f"Number of Q heads ({Hq}) must be divisible by number of K/V heads ({Hkv})")
    m = None
    if mask_kind == MASK_QK:
        m = _f32(mask)
        assert m.shape == (Sq, Skv), f"QKMask shape {m.shape} does not match expected [{Sq}, {Skv}]"
    elif mask_kind == MASK_BATCH_KEY:
        m = _f32(mask)
        assert m.shape == (B, Skv), f"BatchKeyMask shape {m.shape} does not match expected [{B}, {Skv}]"
    if causal_offset is None:
        causal_offset = Skv - Sq
    r = None
    n_rows = 0
    if rows is not None:
        r = np.ascontiguousarray(rows, dtype=np.int64)
        assert np.all(np.diff(r) > 0)
        n_rows = r.size
        out = np.empty((n_rows, D), np.float32)
    else:
        out = np.empty_like(q)
    rc = lib().oracle_attention_f32(_p(q), _p(k), _p(v), _p(m), mask_kind, int(causal_offset), _p(out), B, Hq, Hkv,
                                    Sq, Skv, D, float(scale),
                                    r.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)) if r is not None else None,
                                    n_rows, int(bool(skip_masked)))
    assert rc == 0, f"oracle_attention_f32 -> {rc}"
    return out


def flash_attention_online(q, k, v, scale, mask=None) -> np.ndarray:
    """The fused WGSL kernel's order (core/src/composite/flash_attention.rs:147-331)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    m = _f32(mask) if mask is not None else None
    out = np.empty_like(q)
    rc = lib().oracle_attention_online_f32(_p(q), _p(k), _p(v), _p(m), _p(out), B, Hq, Hkv, Sq, Skv, D, float(scale))
    assert rc == 0
    return out


def attention_partial(q, k, v, scale, k0, k1) -> np.ndarray:
    """Split-KV partial {m, l, O[D]} of keys [k0, k1): [B, Hq, Sq, D+2]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    part = np.empty((B, Hq, Sq, D + 2), np.float32)
    rc = lib().oracle_attention_partial_f32(_p(q), _p(k), _p(v), _p(part), B, Hq, Hkv, Sq, Skv, D, float(scale),
                                            int(k0), int(k1))
    assert rc == 0
    return part


def lse_combine(parts) -> np.ndarray:
    """parts [P, rows..., D+2] -> [rows..., D]."""
    parts = _f32(parts)
    P = parts.shape[0]
    D = parts.shape[-1] - 2
    n_rows = int(np.prod(parts.shape[1:-1]))
    out = np.empty(parts.shape[1:-1] + (D,), np.float32)
    lib().oracle_lse_combine(_p(parts), P, n_rows, D, _p(out))
    return out


# --------------------------------------------------------------------------- output projection
def out_proj(attn, w, bias=None) -> np.ndarray:
    """attn [B,Hq,S,D], w [N, Hq*D], bias [N] or None -> [B,S,N]: transpose(1,2).reshape then x @ w.T + bias
    (models/kalosm-llama/src/raw/attention_layer.rs:450-454; fusor-ml/fusor/src/layers/linear.rs:72-115)."""
    attn, w = _f32(attn), _f32(w)
    B, Hq, S, D = attn.shape
    N, K = w.shape
    assert K == Hq * D
    b = _f32(bias) if bias is not None else None
    out = np.empty((B, S, N), np.float32)
    rc = lib().oracle_out_proj_f32(_p(attn), _p(w), _p(b), _p(out), B, Hq, S, D, N)
    assert rc == 0
    return out


# --------------------------------------------------------------------------- rotary embedding
def rope_tables(head_dim: int, context_length: int, rope_theta: float = 10000.0):
    """RopeCache::new (fusor-ml/fusor/src/composite/rope.rs:186-219): cos, sin [context_length, head_dim/2] in f32."""
    inv = np.array([1.0 / np.float32(rope_theta) ** (np.float32(i) / np.float32(head_dim)) for i in range(0, head_dim, 2)],
                   dtype=np.float32)
    outer = np.arange(context_length, dtype=np.float32)[:, None] * inv[None, :]
    return np.cos(outer).astype(np.float32), np.sin(outer).astype(np.float32)


def rope(x, cos, sin, start_pos: int = 0, interleaved: bool = False) -> np.ndarray:
    """Tensor::rope / rope_interleaved on f32 [B,H,S,D] with table rows start_pos .. start_pos+S."""
    x, cos, sin = _f32(x), _f32(cos), _f32(sin)
    B, H, S, D = x.shape
    assert cos.shape == sin.shape and cos.shape[1] == D // 2 and start_pos + S <= cos.shape[0]
    out = np.empty_like(x)
    rc = lib().oracle_rope_f32(_p(x), _p(cos), _p(sin), _p(out), B, H, S, D, int(start_pos), int(bool(interleaved)))
    assert rc == 0
    return out


# --------------------------------------------------------------------------- masks (A6)
def causal_mask(S: int) -> np.ndarray:
    m = np.empty((S, S), np.float32)
    lib().oracle_causal_mask(_p(m), S)
    return m


def sliding_window_mask(S: int, window: int) -> np.ndarray:
    m = np.empty((S, S), np.float32)
    lib().oracle_sliding_window_mask(_p(m), S, window)
    return m


def get_mask(seq_len: int, seqlen_offset: int, sliding_window_size=None) -> np.ndarray:
    """MaskCache::get_mask (mask_cache.rs:36-86) without the memoisation."""
    if sliding_window_size is not None:
        seqlen_offset = min(seqlen_offset, max(sliding_window_size - seq_len, 0))
        base = sliding_window_mask(seq_len, sliding_window_size)
    else:
        base = causal_mask(seq_len)
    if seqlen_offset > 0:
        padded = np.zeros((seq_len, seqlen_offset + seq_len), np.float32)
        padded[:, seqlen_offset:] = base
        return padded
    return base


# --------------------------------------------------------------------------- caches (A7)
class TensorCacheOracle:
    """numpy restatement of TensorCache (tensor_cache.rs:9-124)."""

    def __init__(self, concat_dim: int, max_sequence_len: int):
        self.all_data = None
        self.current_seq_len = 0
        self.allocated_seq_len = 0
        self.concat_dim = concat_dim
        self.max_sequence_len = max_sequence_len

    def reset(self):
        self.all_data = None
        self.current_seq_len = 0
        self.allocated_seq_len = 0

    def current_data(self):
        return self.all_data

    def append(self, v: np.ndarray) -> np.ndarray:
        ax = self.concat_dim
        seq_len = v.shape[ax]
        required = self.current_seq_len + seq_len
        if required > self.max_sequence_len:
            mx = self.max_sequence_len
            new_start = required - mx
            parts = []
            if self.all_data is not None:
                parts.append(np.take(self.all_data, range(new_start, self.current_seq_len), axis=ax)
                             if new_start < self.current_seq_len else
                             np.take(self.all_data, [], axis=ax))
            parts.append(v)
            allv = np.concatenate(parts, axis=ax)
            n = allv.shape[ax]
            self.all_data = np.take(allv, range(n - mx, n), axis=ax)
            self.current_seq_len = mx
            self.allocated_seq_len = mx
            return self.all_data.copy()
        if self.all_data is not None:
            if required > self.allocated_seq_len:
                new_alloc = 1 << (required - 1).bit_length()
                self.allocated_seq_len = new_alloc
                shape = list(v.shape)
                shape[ax] = new_alloc - self.all_data.shape[ax]
                self.all_data = np.concatenate([self.all_data, np.zeros(shape, v.dtype)], axis=ax)
            idx = [slice(None)] * v.ndim
            idx[ax] = slice(self.current_seq_len, required)
            self.all_data[tuple(idx)] = v
            self.current_seq_len = required
            idx[ax] = slice(0, required)
            return self.all_data[tuple(idx)].copy()
        self.all_data = v.copy()
        self.current_seq_len = seq_len
        self.allocated_seq_len = seq_len
        return v.copy()


class KvCacheOracle:
    """numpy restatement of KvCache (kv_cache.rs:12-68)."""

    def __init__(self, concat_dim: int, max_sequence_len: int):
        self.key = TensorCacheOracle(concat_dim, max_sequence_len)
        self.value = TensorCacheOracle(concat_dim, max_sequence_len)

    def k(self):
        return self.key.current_data()

    def v(self):
        return self.value.current_data()

    def reset(self):
        self.key.reset()
        self.value.reset()

    def append(self, k, v):
        return self.key.append(k), self.value.append(v)

    def current_seq_len(self):
        return self.key.current_seq_len


# --------------------------------------------------------------------------- paged cache (N1)
def depage(pages: np.ndarray, page_table: np.ndarray, kv_len: np.ndarray) -> list:
    """pages [num_pages, Hkv, page_tokens, D], page_table [B, max_pages], kv_len [B]
    -> list over b of dense [Hkv, kv_len[b], D]."""
    out = []
    T = pages.shape[2]
    for b in range(page_table.shape[0]):
        n = int(kv_len[b])
        npg = (n + T - 1) // T
        dense = pages[page_table[b, :npg]]                      # [npg, Hkv, T, D]
        dense = dense.transpose(1, 0, 2, 3).reshape(pages.shape[1], npg * T, pages.shape[3])
        out.append(np.ascontiguousarray(dense[:, :n]))
    return out
