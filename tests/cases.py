"""Seeded inputs for the parity tests: N(0,1) values rounded to f16, Q8_0 pools quantised with the
oracle's GPU-exact quantiser, identity or Fisher-Yates page tables, and helpers that run a kernel
through the C ABI the way the reference's tests drive sg-gpu (crates/sg-gpu/tests/parity_attn.rs)."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from oracle import sg_oracle as O

H, KV, D, G, PAGE = 32, 16, 128, 2, 256
SCALE = 0.08838834764831845  # 1/sqrt(128)

# Tolerance for attention outputs in f32: |got - want| <= 2e-3 + 1e-2 * |want|
ATOL, RTOL = 2e-3, 1e-2


def normal_f16(seed: int, *shape) -> np.ndarray:
    """i.i.d. N(0,1) in f32, rounded to f16 (RTNE); returned as float16."""
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32).astype(np.float16)


def page_table(seed: int, n_pages: int, identity: bool = False) -> np.ndarray:
    if identity:
        return np.arange(n_pages, dtype=np.uint32)
    return np.random.default_rng(seed).permutation(n_pages).astype(np.uint32)


@dataclass
class Q8Pool:
    """K or V of `n_tokens` logical tokens stored in a paged Q8_0 pool of `pool_pages` pages."""

    quants: np.ndarray  # int8 [pool_rows, n_kv, D]
    scales: np.ndarray  # uint16 [pool_rows, n_kv, D/32]
    deq: np.ndarray     # float32 [n_tokens, n_kv, D], logical order, exact f32(scale)*f32(q)
    deq16: np.ndarray   # float32 [n_tokens, n_kv, D], the f16-rounded dequantised values


def q8_pool(x16: np.ndarray, table: np.ndarray, page: int, pool_pages: int | None = None, fill_seed: int = 99) -> Q8Pool:
    """Quantise logical rows x16 [n_tokens, n_kv, D] and scatter them through `table`.  Unused
    rows of the pool hold other seeded data, not zeros, so an indexing slip cannot hide."""
    n_tokens, n_kv, d = x16.shape
    pool_pages = pool_pages or int(table.max()) + 1
    rows = pool_pages * page
    rng = np.random.default_rng(fill_seed)
    quants = rng.integers(-127, 128, size=(rows, n_kv, d), dtype=np.int8)
    scales = (rng.random((rows, n_kv, d // 32), dtype=np.float32) * 0.05).astype(np.float16).view(np.uint16)
    s, q = O.quant_q8_0(x16.astype(np.float32))
    s, q = s.reshape(n_tokens, n_kv, d // 32), q.reshape(n_tokens, n_kv, d)
    t = np.arange(n_tokens)
    phys = table[t // page].astype(np.int64) * page + t % page
    quants[phys] = q
    scales[phys] = s
    deq = O.dequant_q8_0_f32(s, q).reshape(n_tokens, n_kv, d)
    deq16 = O.f16_bits_to_f32(O.dequant_q8_0_f16(s, q)).reshape(n_tokens, n_kv, d)
    return Q8Pool(quants, scales, deq, deq16)


def assert_close(got, want, atol=ATOL, rtol=RTOL, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    excess = np.abs(got - want) - rtol * np.abs(want)
    i = int(np.argmax(excess))
    assert excess.flat[i] <= atol, (f"{what}: element {np.unravel_index(i, got.shape)}: got {got.flat[i]} want {want.flat[i]} "
                                    f"(max abs err {np.abs(got - want).max():.3e})")


def B(index, buf):
    from super_gemma_b200 import BufferBinding

    return BufferBinding.buffer(index, buf)


def bind(*bufs):
    return [B(i, b) for i, b in enumerate(bufs)]
