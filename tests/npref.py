"""An independent numpy restatement of the attention math, used to cross-check the C oracle and
to generate the committed golden fixtures.  It shares no code with ``oracle/``: float64 numpy
throughout, numpy's own float16 for rounding."""
from __future__ import annotations

import numpy as np


def xorshift64star(seed: int, n: int) -> np.ndarray:
    """n draws of the reference tests' generator (crates/sg-gpu/tests/reference/mod.rs:8-32),
    as the f32 values in [-2, 2) it produces."""
    mask = (1 << 64) - 1
    x = seed if seed else 1
    out = np.empty(n, np.float32)
    for i in range(n):
        x ^= x >> 12
        x ^= (x << 25) & mask
        x ^= x >> 27
        r = (x * 0x2545F4914F6CDD1D) & mask
        out[i] = np.float32(np.float32(r >> 40) / np.float32(1 << 24) * np.float32(4.0) - np.float32(2.0))
    return out


def quant_q8_0(x: np.ndarray):
    """Multiply-form Q8_0 (crates/sg-gpu/shaders/kv_quant_q8.wgsl:36-56)."""
    x = np.asarray(x, np.float32).reshape(-1, 32)
    amax = np.abs(x).max(axis=1)
    d = (amax * np.float32(1.0 / 127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    q = np.rint((x * inv[:, None]).astype(np.float32)).astype(np.int8)
    return d.astype(np.float16).view(np.uint16), q.reshape(-1)


def dequant_f32(scales_bits: np.ndarray, quants: np.ndarray) -> np.ndarray:
    s = scales_bits.view(np.float16).astype(np.float32)
    return (np.repeat(s, 32) * quants.astype(np.float32)).astype(np.float32)


def attention(q, k, v, q0, n_q, n_kv, window=0, scale=1.0):
    """Causal (optionally windowed) GQA attention in float64 over linear K/V.
    q [m, n_q, hd]; k, v [l, n_kv, hd]; query i sits at position q0 + i and sees
    [max(0, pos + 1 - window), pos] (crates/sg-model/src/reference.rs:482-530)."""
    q, k, v = (np.asarray(a, np.float64) for a in (q, k, v))
    m, _, hd = q.shape
    g = n_q // n_kv
    out = np.empty((m, n_q, hd), np.float64)
    for i in range(m):
        pos = q0 + i
        lo = max(0, pos + 1 - window) if window else 0
        for h in range(n_q):
            kk = k[lo : pos + 1, h // g]
            s = kk @ q[i, h] * scale
            p = np.exp(s - s.max())
            out[i, h] = (p[:, None] * v[lo : pos + 1, h // g]).sum(0) / p.sum()
    return out.astype(np.float32)


def attention_rows(q_rows, k, v, hi, lo, scale):
    """q_rows [r, hd] all reading the same kv head slice k, v [l, hd]; row j sees keys lo[j]..hi[j]."""
    out = np.empty(q_rows.shape, np.float64)
    for j in range(q_rows.shape[0]):
        kk = np.asarray(k[lo[j] : hi[j] + 1], np.float64)
        s = kk @ np.asarray(q_rows[j], np.float64) * scale
        p = np.exp(s - s.max())
        out[j] = (p[:, None] * np.asarray(v[lo[j] : hi[j] + 1], np.float64)).sum(0) / p.sum()
    return out.astype(np.float32)
