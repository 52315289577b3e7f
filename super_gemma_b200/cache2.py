"""Host-side page-table manager for the paged KV kernels, over the ``sgb_cache2_*`` C ABI.

The reference has the design of cache2 only (``docs/plans/04-kv-cache.md:40-51``: a radix trie in
RAM keyed by token-id sequences whose nodes own pages of global KV; ``crates/sg-cache/src/lib.rs:9-13``
holds the page-size constants).  ``PageCache`` is that trie at page granularity plus the physical page
pool; ``Sequence.table`` is the ``page_table`` binding of ``attn_decode_paged_q8kv_d128``,
``kv_append_paged_q8_d128`` and the paged prefill kernels.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from .gpu import _Cache2Stats, _check, lib

# crates/sg-cache/src/lib.rs:9-13
MIN_PAGE_SIZE = 16
MAX_PAGE_SIZE = 512
DEFAULT_PAGE_SIZE = 256


def _ids(tokens) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(-1))


@dataclass
class Sequence:
    """One live sequence: ``table[i]`` is the physical page of logical page ``i``; K/V of the first
    ``reused_tokens`` tokens is already in the pool."""
    handle: int
    table: np.ndarray
    reused_tokens: int


class PageCache:
    def __init__(self, pool_pages: int, page_tokens: int = DEFAULT_PAGE_SIZE):
        self._L = lib()
        self._h = C.c_void_p()
        _check(self._L.sgb_cache2_create(page_tokens, pool_pages, C.byref(self._h)))
        self.page_tokens, self.pool_pages = page_tokens, pool_pages

    def close(self) -> None:
        if self._h:
            self._L.sgb_cache2_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def lookup(self, tokens) -> int:
        """Tokens of the longest cached page-aligned prefix."""
        t = _ids(tokens)
        out = C.c_uint64()
        _check(self._L.sgb_cache2_lookup(self._h, t.ctypes.data, t.size, C.byref(out)))
        return out.value

    def acquire(self, tokens, capacity_tokens: int = 0) -> Sequence:
        t = _ids(tokens)
        cap = max(int(capacity_tokens), t.size)
        n_table = (cap + self.page_tokens - 1) // self.page_tokens
        table = np.zeros(max(n_table, 1), np.uint32)
        n_pages, reused, seq = C.c_uint32(), C.c_uint64(), C.c_uint64()
        _check(self._L.sgb_cache2_acquire(self._h, t.ctypes.data, t.size, cap, table.ctypes.data, table.size, C.byref(n_pages),
                                          C.byref(reused), C.byref(seq)))
        return Sequence(seq.value, table[: n_pages.value].copy(), reused.value)

    def commit(self, seq: Sequence, tokens) -> None:
        t = _ids(tokens)
        _check(self._L.sgb_cache2_commit(self._h, seq.handle, t.ctypes.data, t.size))

    def release(self, seq: Sequence) -> None:
        _check(self._L.sgb_cache2_release(self._h, seq.handle))

    def stats(self) -> dict:
        s = _Cache2Stats()
        _check(self._L.sgb_cache2_stats(self._h, C.byref(s)))
        return {name: getattr(s, name) for name, _ in _Cache2Stats._fields_ if name != "reserved"}
