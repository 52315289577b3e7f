"""CPU tests of the cache2 page-table manager (host code of the shared library, no GPU needed).

The reference has no cache2 code to compare with (docs/plans/04-kv-cache.md is a design), so the
checks are a naive model of the trie (a set of page-aligned token prefixes) and the invariants a
page table must keep: a physical page is never shared between sequences whose tokens differ up to
the end of that page, and free + reclaimable + held pages always add up to the pool."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def sg():
    from super_gemma_b200 import build

    build.build()
    import super_gemma_b200 as sg

    return sg


@pytest.fixture()
def cache2(sg):
    from super_gemma_b200 import cache2

    return cache2


P = 16


def toks(rng, n, vocab=5):
    return rng.integers(0, vocab, size=n).astype(np.int32)


def test_page_size_limits(sg, cache2):
    # crates/sg-cache/src/lib.rs:9-13: 16..512 tokens
    for bad in (8, 24, 1024):
        with pytest.raises(sg.Validation):
            cache2.PageCache(4, bad)
    with pytest.raises(sg.Validation):
        cache2.PageCache(0, 16)
    for ok in (cache2.MIN_PAGE_SIZE, cache2.DEFAULT_PAGE_SIZE, cache2.MAX_PAGE_SIZE):
        cache2.PageCache(2, ok).close()


def test_miss_then_hit_shares_the_prefix_pages(cache2):
    c = cache2.PageCache(64, P)
    rng = np.random.default_rng(1)
    a = toks(rng, 5 * P + 3, vocab=1000)
    assert c.lookup(a) == 0
    sa = c.acquire(a, capacity_tokens=8 * P)
    assert sa.reused_tokens == 0 and len(sa.table) == 8 and len(set(sa.table)) == 8
    assert c.lookup(a) == 0, "nothing is shareable before commit"
    c.commit(sa, a)
    assert c.lookup(a) == 5 * P
    # same first 3 pages, then different
    b = np.concatenate([a[: 3 * P + 5], toks(rng, 40, vocab=1000) + 2000])
    assert c.lookup(b) == 3 * P
    sb = c.acquire(b)
    assert sb.reused_tokens == 3 * P
    assert list(sb.table[:3]) == list(sa.table[:3])
    assert not set(sb.table[3:]) & set(sa.table)
    st = c.stats()
    assert st["hits"] == 1 and st["misses"] == 1 and st["live_sequences"] == 2
    # a's table is unchanged by its commit and by b
    c.release(sa)
    c.release(sb)
    st = c.stats()
    assert st["live_sequences"] == 0
    assert st["free_pages"] + st["reclaimable_pages"] <= 64
    # the 5 committed pages stay cached (3 of them inner nodes), everything else is free again
    assert st["free_pages"] == 64 - 5
    assert c.lookup(a) == 5 * P
    c.close()


def test_page_being_appended_into_is_private(cache2):
    c = cache2.PageCache(16, P)
    a = np.arange(2 * P, dtype=np.int32)
    sa = c.acquire(a, capacity_tokens=3 * P)
    c.commit(sa, a)
    # the same prompt again: both full pages are shared, the third (append target) is private
    sb = c.acquire(a, capacity_tokens=3 * P)
    assert sb.reused_tokens == 2 * P
    assert list(sb.table[:2]) == list(sa.table[:2]) and sb.table[2] != sa.table[2]
    # a shorter prompt that ends inside page 1 shares only page 0
    sc = c.acquire(a[: P + 4], capacity_tokens=2 * P)
    assert sc.reused_tokens == P and sc.table[0] == sa.table[0] and sc.table[1] != sa.table[1]
    c.close()


def test_exhaustion_is_an_error_and_changes_nothing(sg, cache2):
    c = cache2.PageCache(4, P)
    a = np.arange(3 * P, dtype=np.int32)
    sa = c.acquire(a)
    before = c.stats()
    with pytest.raises(sg.State):
        c.acquire(a + 100)  # needs 3, only 1 free, nothing reclaimable
    assert c.stats() == before
    with pytest.raises(sg.Validation):
        c.release(cache2.Sequence(999, sa.table, 0))
    c.release(sa)
    assert c.stats()["free_pages"] == 4
    c.close()


def test_least_recently_used_pages_are_reclaimed_leaf_first(cache2):
    c = cache2.PageCache(6, P)
    a = np.arange(3 * P, dtype=np.int32)
    b = np.arange(3 * P, dtype=np.int32) + 1000
    for t in (a, b):
        s = c.acquire(t)
        c.commit(s, t)
        c.release(s)
    assert c.stats()["free_pages"] == 0 and c.lookup(a) == 3 * P and c.lookup(b) == 3 * P
    # touch a, so b is the older chain
    s = c.acquire(a)
    c.release(s)
    x = np.arange(2 * P, dtype=np.int32) + 5000
    sx = c.acquire(x)  # reclaims b's two deepest pages
    assert c.lookup(a) == 3 * P
    assert c.lookup(b) == P
    assert c.stats()["evictions"] == 2
    c.release(sx)
    c.close()


def test_random_workload_against_a_naive_model(cache2):
    """Big pool (no reclaim): lookup equals the naive longest-committed-prefix; tables of live
    sequences share a page exactly where the page-aligned token prefixes agree and were cached."""
    rng = np.random.default_rng(7)
    c = cache2.PageCache(4096, P)
    committed = set()  # tuples of tokens, page-aligned prefixes
    live = []
    for step in range(300):
        n = int(rng.integers(0, 6 * P))
        base = toks(rng, n, vocab=2)  # tiny vocabulary and a shared stem: many prefix collisions
        if live and rng.random() < 0.6:
            other = live[int(rng.integers(len(live)))][1]
            k = int(rng.integers(0, len(other) + 1))
            base = np.concatenate([other[:k], base])[: 6 * P]
        expect = 0
        while (expect + 1) * P <= len(base) and tuple(base[: (expect + 1) * P]) in committed:
            expect += 1
        assert c.lookup(base) == expect * P
        s = c.acquire(base, capacity_tokens=len(base) + int(rng.integers(0, 2 * P)))
        assert s.reused_tokens == expect * P
        if rng.random() < 0.7:
            c.commit(s, base)
            for k in range(1, len(base) // P + 1):
                committed.add(tuple(base[: k * P]))
        live.append((s, base))
        if len(live) > 12:
            s0, _ = live.pop(int(rng.integers(len(live))))
            c.release(s0)
        # invariants over the live sequences
        owner = {}
        for s1, t1 in live:
            for i, phys in enumerate(s1.table):
                key = tuple(t1[: (i + 1) * P]) if (i + 1) * P <= len(t1) else ("private", s1.handle, i)
                assert owner.setdefault(int(phys), key) == key, "one physical page, two different contents"
        st = c.stats()
        assert st["live_sequences"] == len(live)
    for s1, _ in live:
        c.release(s1)
    st = c.stats()
    assert st["free_pages"] + len(committed) == 4096
    c.close()


def test_random_workload_with_reclaim_keeps_pages_disjoint(sg, cache2):
    rng = np.random.default_rng(11)
    pool = 40
    c = cache2.PageCache(pool, P)
    live = []
    for step in range(400):
        base = toks(rng, int(rng.integers(1, 5 * P)), vocab=3)
        try:
            s = c.acquire(base)
        except sg.State:
            assert live, "an empty cache can always serve one short sequence"
            s0, _ = live.pop(0)
            c.release(s0)
            continue
        m = c.lookup(base)
        assert m >= s.reused_tokens
        c.commit(s, base)
        live.append((s, base))
        if len(live) > 5:
            s0, _ = live.pop(int(rng.integers(len(live))))
            c.release(s0)
        owner = {}
        held = set()
        for s1, t1 in live:
            for i, phys in enumerate(s1.table):
                key = tuple(t1[: (i + 1) * P]) if (i + 1) * P <= len(t1) else ("private", s1.handle, i)
                assert owner.setdefault(int(phys), key) == key
                held.add(int(phys))
        st = c.stats()
        assert st["free_pages"] + st["reclaimable_pages"] + len(held) <= pool
        assert max(held, default=0) < pool
    c.close()
