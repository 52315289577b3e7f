"""GPU test of the cache2 page tables end to end: two sequences that share a prompt prefix append
through kv_append_paged_q8_d128 into one pool, the second one writing only what the cache did not
already hold, and both decode through attn_decode_paged_q8kv_d128 to the oracle's answer."""
import numpy as np
import pytest

from cases import D, G, SCALE, assert_close, bind, normal_f16
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu

N_KV, PAGE, POOL = 4, 64, 12
ROW = N_KV * D


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


class Pool:
    def __init__(self, ctx):
        self.ctx = ctx
        rows = POOL * PAGE
        # not zeros: a page that is read without having been written must show up as a mismatch
        rng = np.random.default_rng(5)
        mk = lambda: (ctx.buffer_from_iter(rng.integers(-127, 128, rows * ROW, dtype=np.int8)),
                      ctx.buffer_from_iter((rng.random(rows * ROW // 32, dtype=np.float32) * 0.05).astype(np.float16).view(np.uint16)))
        self.kq, self.ks = mk()
        self.vq, self.vs = mk()
        self.step = ctx.new_step_buffer()

    def append(self, table, k16, v16, first):
        """Append logical tokens first.. of a sequence (rows of k16/v16 from `first` on)."""
        import super_gemma_b200 as sg

        n = len(k16) - first
        if n == 0:
            return
        kern = self.ctx.load_kernel("kv_append_paged_q8_d128")
        sg.StepState(pos=first).write_to(self.step)
        for x16, scales, quants in ((k16, self.ks, self.kq), (v16, self.vs, self.vq)):
            src = self.ctx.buffer_from_iter(np.ascontiguousarray(x16[first:]).view(np.uint16).reshape(-1))
            self.ctx.dispatch_blocking(kern, bind(src, scales, quants, table, self.step), (ROW, PAGE), kern.groups_for(n * ROW // 32))

    def decode(self, table, q16, kv_len, n_splits=3):
        import super_gemma_b200 as sg

        rows = N_KV * G
        sg.StepState(kv_len_global=kv_len).write_to(self.step)
        part = self.ctx.new_buffer(rows * n_splits * (D + 2), np.float32)
        out = self.ctx.new_buffer(rows * D, np.float32)
        self.ctx.dispatch(self.ctx.load_kernel("attn_decode_paged_q8kv_d128"),
                          bind(self.ctx.buffer_from_iter(q16), self.kq, self.ks, self.vq, self.vs, table, part, self.step),
                          (n_splits, SCALE, PAGE), [N_KV, n_splits, 1])
        self.ctx.dispatch_blocking(self.ctx.load_kernel("attn_reduce_f32_d128"), bind(part, out), n_splits, [rows, 1, 1])
        return out.read().reshape(1, rows, D)


def want(q16, k16, v16):
    def deq(x16):
        s, q = O.quant_q8_0(x16.astype(np.float32))
        return O.dequant_q8_0_f32(s, q).reshape(x16.shape)

    n = len(k16)
    return O.attention_f64(q16.astype(np.float32), deq(k16), deq(v16), 1, n - 1, N_KV * G, N_KV, D, SCALE)


def test_two_sequences_share_prefix_pages(ctx):
    from super_gemma_b200 import cache2

    cache = cache2.PageCache(POOL, PAGE)
    pool = Pool(ctx)
    rng = np.random.default_rng(21)
    tok_a = rng.integers(0, 50000, 200).astype(np.int32)
    tok_b = np.concatenate([tok_a[:150], rng.integers(0, 50000, 60).astype(np.int32)])
    # K/V rows are a function of the token prefix: equal prefixes give equal rows
    ka, va = normal_f16(31, 200, N_KV, D), normal_f16(32, 200, N_KV, D)
    kb = np.concatenate([ka[:150], normal_f16(33, 60, N_KV, D)])
    vb = np.concatenate([va[:150], normal_f16(34, 60, N_KV, D)])
    qa, qb = normal_f16(35, 1, N_KV * G, D), normal_f16(36, 1, N_KV * G, D)

    sa = cache.acquire(tok_a, capacity_tokens=256)
    assert sa.reused_tokens == 0
    ta = ctx.buffer_from_iter(sa.table)
    pool.append(ta, ka, va, 0)
    cache.commit(sa, tok_a)
    got_a = pool.decode(ta, qa, 200)
    assert_close(got_a, want(qa, ka, va), what="sequence A")

    sb = cache.acquire(tok_b, capacity_tokens=256)
    assert sb.reused_tokens == 128 and list(sb.table[:2]) == list(sa.table[:2]) and not set(sb.table[2:]) & set(sa.table)
    tb = ctx.buffer_from_iter(sb.table)
    pool.append(tb, kb, vb, sb.reused_tokens)  # only the 82 tokens the cache does not hold
    cache.commit(sb, tok_b)
    got_b = pool.decode(tb, qb, 210)
    assert_close(got_b, want(qb, kb, vb), what="sequence B over A's prefix pages")
    # A is untouched by B's appends
    assert np.array_equal(pool.decode(ta, qa, 200).view(np.uint32), got_a.view(np.uint32))

    # A ends; a third, unrelated sequence takes what is free and reclaims A's now idle third page,
    # but never a page B holds
    cache.release(sa)
    tok_c = rng.integers(0, 50000, 8 * PAGE).astype(np.int32)
    sc = cache.acquire(tok_c)
    assert cache.stats()["evictions"] == 1
    assert not set(sc.table) & set(sb.table)
    kc, vc = normal_f16(37, 8 * PAGE, N_KV, D), normal_f16(38, 8 * PAGE, N_KV, D)
    tc = ctx.buffer_from_iter(sc.table)
    pool.append(tc, kc, vc, 0)
    qc = normal_f16(39, 1, N_KV * G, D)
    assert_close(pool.decode(tc, qc, 8 * PAGE), want(qc, kc, vc), what="sequence C")
    assert np.array_equal(pool.decode(tb, qb, 210).view(np.uint32), got_b.view(np.uint32))
    cache.close()
