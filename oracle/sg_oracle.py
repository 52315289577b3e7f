"""ctypes + numpy front end of the CPU oracle (``sg_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline / reference arm of ``bench.py``.  The product package never imports it.

Every function names the reference item it restates in ``sg_oracle.c``; this file only marshals
numpy arrays.  Arrays use the kernels' own storage types: f16 as ``uint16`` bit patterns (or
``float16`` viewed as such), Q8_0 quants as ``int8``, scales as ``uint16`` bits, page tables and the
step buffer as ``uint32``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsgoracle.so")


def build(force: bool = False) -> str:
    """Compile ``libsgoracle.so`` with the Makefile beside this file."""
    src = os.path.join(_HERE, "sg_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True)
    return _LIB_PATH


class _KvSrc(C.Structure):
    _fields_ = [
        ("f16", C.c_void_p),
        ("quants", C.c_void_p),
        ("scales", C.c_void_p),
        ("page_table", C.c_void_p),
        ("page", C.c_uint32),
        ("round_f16", C.c_uint32),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        vp, u32, u64, sz, f32, f64, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t, C.c_float, C.c_double, C.c_int
        L.sgo_f16_to_f32.restype = f32
        L.sgo_f16_to_f32.argtypes = [C.c_uint16]
        L.sgo_f32_to_f16.restype = C.c_uint16
        L.sgo_f32_to_f16.argtypes = [f32]
        L.sgo_h2f_fast.restype = f32
        L.sgo_h2f_fast.argtypes = [C.c_uint16]
        L.sgo_round_through_f16_fast.restype = f32
        L.sgo_round_through_f16_fast.argtypes = [f32]
        L.sgo_f32_to_f16_vec.argtypes = [vp, vp, sz]
        L.sgo_f16_to_f32_vec.argtypes = [vp, vp, sz]
        L.sgo_through_f16.argtypes = [vp, vp, sz]
        L.sgo_rng_seed.argtypes = [vp, u64]
        L.sgo_rng_next_u64.restype = u64
        L.sgo_rng_next_u64.argtypes = [vp]
        L.sgo_rng_f32_vec.argtypes = [vp, vp, sz]
        L.sgo_quant_q8_0.argtypes = [vp, sz, vp, vp]
        L.sgo_q8_quant_div.argtypes = [vp, sz, vp, vp, vp]
        L.sgo_dequant_q8_0_f16.argtypes = [vp, vp, sz, vp]
        L.sgo_dequant_q8_0_f32.argtypes = [vp, vp, sz, vp]
        L.sgo_kv_append.argtypes = [vp, vp, sz, sz, u32, u32]
        L.sgo_kv_append_q8.argtypes = [vp, vp, vp, sz, sz, u32, vp, u32]
        L.sgo_kv_materialize.argtypes = [C.POINTER(_KvSrc), sz, i32, i32, vp]
        L.sgo_attention_head.argtypes = [vp, vp, vp, sz, i32, i32, i32, i32, f64, sz, sz, vp]
        L.sgo_attention_f64.argtypes = [vp, vp, vp, sz, sz, i32, i32, i32, sz, f64, vp, sz, vp, sz, vp]
        L.sgo_decode_partials_f32.argtypes = [vp, C.POINTER(_KvSrc), C.POINTER(_KvSrc), vp, i32, i32, i32, u32, u32, f32, u32]
        L.sgo_reduce_f32.argtypes = [vp, vp, vp, sz, i32, u32, i32]
        L.sgo_prefill_stream_f32.argtypes = [vp, C.POINTER(_KvSrc), C.POINTER(_KvSrc), C.POINTER(_KvSrc), C.POINTER(_KvSrc),
                                             vp, vp, sz, u32, i32, i32, i32, u32, u32, f32]
        L.sgo_prefill_flash_f32.argtypes = [vp, C.POINTER(_KvSrc), C.POINTER(_KvSrc), vp, sz, u32, i32, i32, i32, u32, f32,
                                            u32, vp, sz]
        L.sgo_num_threads.restype = i32
        L.sgo_set_threads.argtypes = [i32]
        _lib = L
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16 and dtype == np.uint16:
        a = a.view(np.uint16)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


def num_threads() -> int:
    return lib().sgo_num_threads()


def set_threads(n: int) -> None:
    lib().sgo_set_threads(n)


# ---- f16 -----------------------------------------------------------------------------------
def f32_to_f16_bits(x) -> np.ndarray:
    x = _c(np.asarray(x, dtype=np.float32), np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().sgo_f32_to_f16_vec(_p(x), _p(out), x.size)
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().sgo_f16_to_f32_vec(_p(h), _p(out), h.size)
    return out


def through_f16(x) -> np.ndarray:
    x = _c(np.asarray(x, dtype=np.float32), np.float32)
    out = np.empty_like(x)
    lib().sgo_through_f16(_p(x), _p(out), x.size)
    return out


# ---- the reference tests' generator ------------------------------------------------------------
class Rng:
    """xorshift64* of crates/sg-gpu/tests/reference/mod.rs:8-32."""

    def __init__(self, seed: int):
        self._s = C.c_uint64(0)
        lib().sgo_rng_seed(C.byref(self._s), seed)

    def next_u64(self) -> int:
        return lib().sgo_rng_next_u64(C.byref(self._s))

    def f32_vec(self, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib().sgo_rng_f32_vec(C.byref(self._s), _p(out), n)
        return out


# ---- Q8_0 codec ----------------------------------------------------------------------------------
def quant_q8_0(x):
    """GPU-exact quantiser (multiply form). Returns (scales u16 bits, quants i8)."""
    x = _c(np.asarray(x, dtype=np.float32).reshape(-1), np.float32)
    assert x.size % 32 == 0
    scales = np.empty(x.size // 32, np.uint16)
    quants = np.empty(x.size, np.int8)
    lib().sgo_quant_q8_0(_p(x), x.size, _p(scales), _p(quants))
    return scales, quants


def q8_quant_div(x):
    """Division-form helper of the attention tests. Returns (scales, quants, dequantised f32)."""
    x = _c(np.asarray(x, dtype=np.float32).reshape(-1), np.float32)
    scales = np.empty(x.size // 32, np.uint16)
    quants = np.empty(x.size, np.int8)
    deq = np.empty(x.size, np.float32)
    lib().sgo_q8_quant_div(_p(x), x.size, _p(scales), _p(quants), _p(deq))
    return scales, quants, deq


def dequant_q8_0_f16(scales, quants) -> np.ndarray:
    scales, quants = _c(scales, np.uint16).reshape(-1), _c(quants, np.int8).reshape(-1)
    out = np.empty(quants.size, np.uint16)
    lib().sgo_dequant_q8_0_f16(_p(scales), _p(quants), quants.size, _p(out))
    return out


def dequant_q8_0_f32(scales, quants) -> np.ndarray:
    scales, quants = _c(scales, np.uint16).reshape(-1), _c(quants, np.int8).reshape(-1)
    out = np.empty(quants.size, np.float32)
    lib().sgo_dequant_q8_0_f32(_p(scales), _p(quants), quants.size, _p(out))
    return out


# ---- KV placement ------------------------------------------------------------------------------
def kv_append(src, dst, row_len: int, pos: int, ring: int = 0) -> None:
    src, dst_c = _c(src, np.uint16), _c(dst, np.uint16)
    assert dst_c is dst or np.shares_memory(dst_c, dst), "dst must be contiguous (written in place)"
    lib().sgo_kv_append(_p(src), _p(dst_c), src.size // row_len, row_len, pos, ring)


def kv_append_q8(src, scales, quants, row_len: int, pos: int, page_table=None, page: int = 256) -> None:
    src = _c(src, np.uint16)
    assert scales.flags.c_contiguous and quants.flags.c_contiguous
    pt = None if page_table is None else _c(page_table, np.uint32)
    lib().sgo_kv_append_q8(_p(src), _p(scales), _p(quants), src.size // row_len, row_len, pos, _p(pt), page)


# ---- K/V sources -------------------------------------------------------------------------------
@dataclass
class KvSrc:
    """One K or V operand as a kernel sees it: f16 rows, or Q8_0 quants+scales, linear or paged."""

    f16: Optional[np.ndarray] = None
    quants: Optional[np.ndarray] = None
    scales: Optional[np.ndarray] = None
    page_table: Optional[np.ndarray] = None
    page: int = 256
    round_f16: bool = False

    def _c(self) -> _KvSrc:
        self._keep = [
            None if self.f16 is None else _c(self.f16, np.uint16),
            None if self.quants is None else _c(self.quants, np.int8),
            None if self.scales is None else _c(self.scales, np.uint16),
            None if self.page_table is None else _c(self.page_table, np.uint32),
        ]
        k = self._keep
        return _KvSrc(*(None if a is None else a.ctypes.data for a in k), self.page, int(self.round_f16))


def kv_materialize(src: KvSrc, n_tokens: int, n_kv: int, hd: int) -> np.ndarray:
    out = np.empty((n_tokens, n_kv, hd), np.float32)
    s = src._c()
    lib().sgo_kv_materialize(C.byref(s), n_tokens, n_kv, hd, _p(out))
    return out


# ---- ground truth ------------------------------------------------------------------------------
def attention_head(q, k, v, i, qh, n_q, n_kv, hd, scale, t0, t1) -> np.ndarray:
    q, k, v = (_c(np.asarray(a, np.float32), np.float32) for a in (q, k, v))
    out = np.empty(hd, np.float32)
    lib().sgo_attention_head(_p(q), _p(k), _p(v), i, qh, n_q, n_kv, hd, float(scale), t0, t1, _p(out))
    return out


def attention_f64(q, k, v, m, q0, n_q, n_kv, hd, scale, window=0, tokens=None, heads=None) -> np.ndarray:
    q, k, v = (_c(np.asarray(a, np.float32), np.float32) for a in (q, k, v))
    tok = None if tokens is None else _c(np.asarray(tokens, np.uint32), np.uint32)
    hds = None if heads is None else _c(np.asarray(heads, np.uint32), np.uint32)
    nt = m if tok is None else tok.size
    nh = n_q if hds is None else hds.size
    out = np.empty((nt, nh, hd), np.float32)
    lib().sgo_attention_f64(_p(q), _p(k), _p(v), m, q0, n_q, n_kv, hd, window, float(scale), _p(tok),
                            0 if tok is None else tok.size, _p(hds), 0 if hds is None else hds.size, _p(out))
    return out


# ---- f32 shader-order forms ------------------------------------------------------------------
def decode_partials_f32(q_f16, ks: KvSrc, vs: KvSrc, n_q, n_kv, hd, kv_len, n_splits, scale, m_q=1) -> np.ndarray:
    q = _c(q_f16, np.uint16)
    part = np.zeros((m_q * n_q, n_splits, hd + 2), np.float32)
    a, b = ks._c(), vs._c()
    lib().sgo_decode_partials_f32(_p(q), C.byref(a), C.byref(b), _p(part), n_q, n_kv, hd, kv_len, n_splits, scale, m_q)
    return part


def reduce_f32(part, hd, n_splits, out_mode=0, f16_out=False):
    part = _c(part, np.float32)
    rows = part.size // (n_splits * (hd + 2))
    if out_mode == 1:
        out = np.empty((rows, hd + 2), np.float32)
        lib().sgo_reduce_f32(_p(part), _p(out), None, rows, hd, n_splits, 1)
        return out
    out = np.empty((rows, hd), np.float32)
    o16 = np.empty((rows, hd), np.uint16) if f16_out else None
    lib().sgo_reduce_f32(_p(part), _p(out), _p(o16), rows, hd, n_splits, 0)
    return o16 if f16_out else out


def prefill_stream_f32(q_f16, k_hist: KvSrc, v_hist: KvSrc, k_chunk: Optional[KvSrc], v_chunk: Optional[KvSrc], m, q0,
                       n_q, n_kv, hd, window, ring, scale) -> np.ndarray:
    q = _c(q_f16, np.uint16)
    out = np.empty((m, n_q, hd), np.float32)
    kh, vh = k_hist._c(), v_hist._c()
    kc = None if k_chunk is None else k_chunk._c()
    vc = None if v_chunk is None else v_chunk._c()
    lib().sgo_prefill_stream_f32(_p(q), C.byref(kh), C.byref(vh), None if kc is None else C.byref(kc),
                                 None if vc is None else C.byref(vc), _p(out), None, m, q0, n_q, n_kv, hd, window, ring,
                                 scale)
    return out


def prefill_flash_f32(q_f16, ks: KvSrc, vs: KvSrc, m, q0, n_q, n_kv, hd, window, scale, tile_k=64, tokens=None) -> np.ndarray:
    q = _c(q_f16, np.uint16)
    tok = None if tokens is None else _c(np.asarray(tokens, np.uint32), np.uint32)
    nt = m if tok is None else tok.size
    out = np.empty((nt, n_q, hd), np.float32)
    a, b = ks._c(), vs._c()
    lib().sgo_prefill_flash_f32(_p(q), C.byref(a), C.byref(b), _p(out), m, q0, n_q, n_kv, hd, window, scale, tile_k,
                                _p(tok), 0 if tok is None else tok.size)
    return out


# ---- pre-attention elementwise steps (crates/sg-gpu/tests/reference/mod.rs:156-216) -------------------------
def rmsnorm_f64(x, w, row_len: int, eps: float = 1e-6, plus_one: bool = False) -> np.ndarray:
    """RMSNorm over rows of `row_len` in f64, rounded to f32 (reference/mod.rs:156-172)."""
    x64 = np.asarray(x, np.float64).reshape(-1, row_len)
    w64 = np.asarray(w, np.float64).reshape(row_len)
    inv = 1.0 / np.sqrt((x64 * x64).sum(axis=1, keepdims=True) / row_len + eps)
    return (x64 * inv * ((1.0 + w64) if plus_one else w64)).astype(np.float32).reshape(-1)


def inv_freqs(rot_dims: int, theta: float) -> np.ndarray:
    """theta^(-2i/rot_dims), i < rot_dims/2 (reference/mod.rs:176-180)."""
    i = np.arange(rot_dims // 2, dtype=np.float64)
    return np.power(np.float64(theta), -2.0 * i / rot_dims)


def cos_sin_table(inv_freq, start_pos: int, tokens: int) -> np.ndarray:
    """[token x half_rot] of interleaved (cos, sin): f64 math, f32 storage (reference/mod.rs:185-197)."""
    pos = (np.arange(tokens, dtype=np.float64) + float(start_pos))[:, None] * np.asarray(inv_freq, np.float64)[None, :]
    return np.stack([np.cos(pos), np.sin(pos)], axis=-1).astype(np.float32).reshape(-1)


def rope_f64(x, head_dim: int, rot_dims: int, n_heads: int, cos_sin) -> np.ndarray:
    """Rotate-half (NeoX) RoPE over rows [token x head x head_dim]: pair i couples dims (i, i + head_dim/2),
    only the first rot_dims/2 pairs rotate; f64 math, rounded to f32 (reference/mod.rs:202-216)."""
    live, partner = rot_dims // 2, head_dim // 2
    rows = np.asarray(x, np.float64).reshape(-1, n_heads, head_dim).copy()
    cs = np.asarray(cos_sin, np.float32).astype(np.float64).reshape(rows.shape[0], live, 2)
    c, s = cs[:, None, :, 0], cs[:, None, :, 1]
    a, b = rows[:, :, :live].copy(), rows[:, :, partner:partner + live].copy()
    rows[:, :, :live] = a * c - b * s
    rows[:, :, partner:partner + live] = b * c + a * s
    return rows.astype(np.float32).reshape(-1)
