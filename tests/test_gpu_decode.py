"""GPU parity for split-K decode, the LSE combine and the speculative-verify extension, through the
C ABI.  Reference-shaped kernels replay the reference's own seeded cases at its own tolerance
(crates/sg-gpu/tests/parity_attn.rs:61,157,1002); the head_dim-128 paged Q8_0 kernel is held to
max-abs 2e-3 / relative 1e-2 against the f64 oracle on dequantised inputs, and to bit-exactness
for page-table indexing and determinism."""
import numpy as np
import pytest

from cases import ATOL, D, G, H, KV, PAGE, RTOL, SCALE, assert_close, bind, normal_f16, page_table, q8_pool
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu

N_Q = 32


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


def _reference_case(ctx, rng, part_name, red_name, n_kv, hd, scale, kv_len, n_splits, quant_k, slot):
    import super_gemma_b200 as sg

    q = O.through_f16(rng.f32_vec(N_Q * hd))
    k = O.through_f16(rng.f32_vec(kv_len * n_kv * hd))
    v = O.through_f16(rng.f32_vec(kv_len * n_kv * hd))
    bufs = [ctx.buffer_from_iter(O.f32_to_f16_bits(q))]
    if quant_k:
        ks, kq, k_ref = O.q8_quant_div(k)  # parity_attn.rs:1016
        bufs += [ctx.buffer_from_iter(kq), ctx.buffer_from_iter(ks)]
    else:
        bufs.append(ctx.buffer_from_iter(O.f32_to_f16_bits(k)))
        k_ref = k
    bufs.append(ctx.buffer_from_iter(O.f32_to_f16_bits(v)))
    part = ctx.new_buffer(N_Q * n_splits * (hd + 2), np.float32)
    out = ctx.new_buffer(N_Q * hd, np.uint16)
    step = ctx.new_step_buffer()
    sg.StepState(**{slot: kv_len}).write_to(step)
    ctx.dispatch_blocking(ctx.load_kernel(part_name), bind(*bufs, part, step), (n_splits, float(scale)), [n_kv, n_splits, 1])
    ctx.dispatch_blocking(ctx.load_kernel(red_name), bind(part, out), n_splits, [N_Q, 1, 1])
    got = O.f16_bits_to_f32(out.read()).reshape(N_Q, hd)
    want = O.attention_f64(q.reshape(1, N_Q, hd), k_ref.reshape(kv_len, n_kv, hd), v.reshape(kv_len, n_kv, hd), 1, kv_len - 1,
                           N_Q, n_kv, hd, scale)[0]
    assert_close(got, want, 1e-2, 1e-2, f"{part_name} kv_len={kv_len} splits={n_splits}")
    return part.read().reshape(N_Q, n_splits, hd + 2)


def test_attn_decode_sliding_matches_reference(ctx):  # parity_attn.rs:61
    rng = O.Rng(0xA77)
    for kv_len, n_splits in [(17, 1), (17, 4), (1024, 8)]:
        _reference_case(ctx, rng, "attn_decode_sliding", "attn_reduce_d256", 16, 256, 0.0625, kv_len, n_splits, False,
                        "kv_len_sliding")


def test_attn_decode_global_matches_reference(ctx):  # parity_attn.rs:157
    rng = O.Rng(0xA78)
    for kv_len, n_splits in [(333, 1), (333, 5), (3, 8), (4096, 4)]:
        _reference_case(ctx, rng, "attn_decode_global", "attn_reduce_d512", 4, 512, 0.044194174, kv_len, n_splits, False,
                        "kv_len_global")


def test_attn_decode_global_q8k_matches_reference(ctx):  # parity_attn.rs:1002
    rng = O.Rng(0xA79)
    for kv_len, n_splits in [(333, 1), (333, 5), (3, 8), (4096, 4)]:
        part = _reference_case(ctx, rng, "attn_decode_global_q8k", "attn_reduce_d512", 4, 512, 0.044194174, kv_len, n_splits,
                               True, "kv_len_global")
        if kv_len == 3:  # empty splits keep the sentinel
            assert np.all(part[:, 3:, 512] == np.float32(-3.0e38)) and np.all(part[:, 3:, 513] == 0)


# ---- head_dim 128, paged Q8_0 K and V ------------------------------------------------------------------
class PagedCase:
    def __init__(self, ctx, seed, kv_len, m_q=1, n_kv=KV, page=PAGE, identity=False, extra_pages=1):
        import super_gemma_b200 as sg

        self.ctx, self.kv_len, self.m_q, self.n_kv, self.page = ctx, kv_len, m_q, n_kv, page
        n_pages = -(-kv_len // page)
        self.table = page_table(seed + 0x100, n_pages + extra_pages, identity)[:n_pages]
        self.q16 = normal_f16(seed, m_q, n_kv * G, D)
        self.k = q8_pool(normal_f16(seed + 1, kv_len, n_kv, D), self.table, page, n_pages + extra_pages, seed + 2)
        self.v = q8_pool(normal_f16(seed + 3, kv_len, n_kv, D), self.table, page, n_pages + extra_pages, seed + 4)
        up = ctx.buffer_from_iter
        self.bufs = [up(self.q16), up(self.k.quants), up(self.k.scales), up(self.v.quants), up(self.v.scales), up(self.table)]
        self.step = ctx.new_step_buffer()
        sg.StepState(kv_len_global=kv_len).write_to(self.step)

    def want(self):
        return O.attention_f64(self.q16.astype(np.float32), self.k.deq, self.v.deq, self.m_q, self.kv_len - self.m_q,
                               self.n_kv * G, self.n_kv, D, SCALE)

    def run(self, n_splits, kernel="attn_decode_paged_q8kv_d128"):
        rows = self.m_q * self.n_kv * G
        part = self.ctx.new_buffer(rows * n_splits * (D + 2), np.float32)
        out = self.ctx.new_buffer(rows * D, np.float32)
        self.ctx.dispatch(self.ctx.load_kernel(kernel), bind(*self.bufs, part, self.step), (n_splits, SCALE, self.page),
                          [self.n_kv, n_splits, self.m_q])
        self.ctx.dispatch_blocking(self.ctx.load_kernel("attn_reduce_f32_d128"), bind(part, out), n_splits, [rows, 1, 1])
        return part.read().reshape(rows, n_splits, D + 2), out.read().reshape(self.m_q, self.n_kv * G, D)


@pytest.mark.parametrize("kv_len,n_splits", [(1, 1), (17, 4), (63, 2), (64, 1), (65, 3), (300, 5), (3, 8), (1000, 7), (4096, 16)])
def test_paged_decode_small_and_ragged(ctx, kv_len, n_splits):
    c = PagedCase(ctx, 0x5603 + kv_len, kv_len, page=64 if kv_len < 1000 else 256)
    want = c.want()
    part, got = c.run(n_splits)
    assert_close(got, want, what=f"paged decode kv_len={kv_len} splits={n_splits}")
    _, got_s = c.run(n_splits, "attn_decode_paged_q8kv_scalar_d128")
    assert_close(got_s, want, what=f"scalar paged decode kv_len={kv_len} splits={n_splits}")
    chunk = -(-kv_len // n_splits)
    for s in range(n_splits):  # empty splits: m = -3e38, l = 0, acc = 0
        if s * chunk >= kv_len:
            assert np.all(part[:, s, D] == np.float32(-3.0e38)) and np.all(part[:, s, :D] == 0) and np.all(part[:, s, D + 1] == 0)


@pytest.mark.parametrize("n_splits", [16, 32, 64])
def test_paged_decode_32k_random_table(ctx, n_splits):
    """benchmark config 3: 1 query x 32768 Q8_0 tokens, 128 pages, seeded random page table."""
    c = PagedCase(ctx, 0x5603, 32768)
    _, got = c.run(n_splits)
    assert_close(got, c.want(), what=f"cfg3 splits={n_splits}")
    _, again = c.run(n_splits)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))  # bit-deterministic (parity_attn.rs:1103)


def test_paged_equals_linear_bit_for_bit(ctx):
    """Page-table indexing: the same logical KV behind a random table and behind the identity table
    (rows gathered into logical order) must give identical partials."""
    a = PagedCase(ctx, 0x5703, 2000, extra_pages=3)
    b = PagedCase(ctx, 0x5703, 2000, identity=True, extra_pages=0)
    pa, _ = a.run(8)
    pb, _ = b.run(8)
    assert np.array_equal(pa.view(np.uint32), pb.view(np.uint32))


@pytest.mark.parametrize("kv_len,m_q,n_splits", [(7, 4, 2), (260, 2, 3), (65540, 4, 32)])
def test_speculative_verify_is_causal_among_the_draft(ctx, kv_len, m_q, n_splits):
    """benchmark config 4, global part: the draft tokens are appended first, then query i sees
    keys t <= kv_len - m_q + i.  There is no reference kernel for this step; the oracle is the f64
    attention at q0 = kv_len - m_q, i.e. the prefill kernels' semantics at M = m_q."""
    c = PagedCase(ctx, 0x5604, kv_len, m_q=m_q)
    want = c.want()
    _, got = c.run(n_splits, "attn_verify_paged_q8kv_d128")
    assert_close(got, want, what=f"verify kv_len={kv_len} m_q={m_q}")
    if kv_len < 1000:
        _, got_s = c.run(n_splits, "attn_decode_paged_q8kv_scalar_d128")
        assert_close(got_s, want, what="scalar verify")


def test_kv_head_slice_is_the_same_kernel(ctx):
    """A rank that owns 4 of the 16 kv heads dispatches grid [4, n_splits]."""
    c = PagedCase(ctx, 0x5605, 3000, n_kv=4)
    _, got = c.run(8)
    assert_close(got, c.want(), what="4 kv heads")


def test_rank_partials_combine_in_rank_order(ctx):
    """Sequence-split decode: each 'rank' merges its own splits to (acc, m, l); the combine kernel
    merges the gathered per-rank partials in rank order.  Emulated here on one GPU by giving each
    rank a slice of one partials buffer."""
    c = PagedCase(ctx, 0x5606, 5000)
    n_splits, ranks, rows = 8, 4, H
    part, got = c.run(n_splits)
    gathered = ctx.new_buffer(ranks * rows * (D + 2), np.float32)
    per = n_splits // ranks
    k = ctx.load_kernel("attn_reduce_partial_d128")
    for r in range(ranks):
        mine = ctx.buffer_from_iter(np.ascontiguousarray(part[:, r * per:(r + 1) * per]))
        ctx.dispatch(k, bind(mine, gathered.slice(r * rows * (D + 2), (r + 1) * rows * (D + 2))), per, [rows, 1, 1])
    out = ctx.new_buffer(rows * D, np.float32)
    ctx.dispatch_blocking(ctx.load_kernel("attn_combine_ranks_d128"), bind(gathered, out), ranks, [rows, 1, 1])
    assert np.allclose(out.read().reshape(1, rows, D), got, rtol=1e-5, atol=1e-6)
    assert_close(out.read().reshape(1, rows, D), c.want(), what="rank combine")


def test_sliding_decode_d128(ctx):
    """benchmark config 4, sliding part at decode: full wrapped ring in physical order."""
    import super_gemma_b200 as sg

    kv_len, n_splits = 1024, 16
    q16, k16, v16 = normal_f16(1, 1, H, D), normal_f16(2, kv_len, KV, D), normal_f16(3, kv_len, KV, D)
    part = ctx.new_buffer(H * n_splits * (D + 2), np.float32)
    out = ctx.new_buffer(H * D, np.float32)
    step = ctx.new_step_buffer()
    sg.StepState(kv_len_sliding=kv_len).write_to(step)
    ctx.dispatch(ctx.load_kernel("attn_decode_sliding_d128"),
                 bind(ctx.buffer_from_iter(q16), ctx.buffer_from_iter(k16), ctx.buffer_from_iter(v16), part, step),
                 (n_splits, SCALE), [KV, n_splits, 1])
    ctx.dispatch_blocking(ctx.load_kernel("attn_reduce_f32_d128"), bind(part, out), n_splits, [H, 1, 1])
    want = O.attention_f64(q16.astype(np.float32), k16.astype(np.float32), v16.astype(np.float32), 1, kv_len - 1, H, KV, D, SCALE)
    assert_close(out.read().reshape(1, H, D), want, what="sliding decode d128")


def test_bad_page_id_is_reported_not_followed(ctx):
    import super_gemma_b200 as sg

    c = PagedCase(ctx, 0x5607, 600)
    bad = c.table.copy()
    bad[1] = 1000  # far outside the pool
    c.bufs[5] = ctx.buffer_from_iter(bad)
    with pytest.raises(sg.Bounds):
        c.run(4)
    c.bufs[5] = ctx.buffer_from_iter(c.table)
    _, got = c.run(4)  # the context is still usable
    assert_close(got, c.want(), what="after a reported bounds error")
