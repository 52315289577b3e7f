"""Exhaustive small-shape sweeps with poisoned memory, the stand-in for a memory checker on this path.

Every length from 1 to 300 (decode) and every chunk size from 1 to 130 (prefill) is run against the f64 oracle
with the device status word required to stay zero (a reported out-of-range page or row, or a wait that ran out,
raises at the blocking dispatch).  Every pool or K/V row that the launch must not use -- rows past the sequence
end, unmapped pool pages, query rows past the chunk -- holds poison (NaN scales with +-127 quants, or NaN f16):
a kernel that lets such a row reach its result produces a non-finite output and fails.  Ragged last pages, ragged
last tiles, empty splits and every split count of the list are covered this way."""
import numpy as np
import pytest

from cases import D, G, H, KV, SCALE, assert_close, bind, normal_f16, page_table, q8_pool
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu

NAN16 = np.uint16(0x7E00)


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


def _poison_quants(shape, seed):
    return np.where(np.random.default_rng(seed).integers(0, 2, size=shape, dtype=np.int8) == 1, 127, -127).astype(np.int8)


@pytest.mark.parametrize("page,m_q", [(16, 1), (64, 1), (256, 1), (16, 4), (64, 4), (256, 4)])
def test_paged_decode_every_length_to_300(ctx, page, m_q):
    import super_gemma_b200 as sg

    L_MAX, splits = 300, (1, 2, 3, 5, 8, 16)
    n_pages = -(-L_MAX // page)
    pool_pages = n_pages + 2
    table = page_table(0x7000 + page, pool_pages)[:n_pages]
    seed = 0x7100 + page + m_q
    q16 = normal_f16(seed, m_q, H, D)
    k = q8_pool(normal_f16(seed + 1, L_MAX, KV, D), table, page, pool_pages, seed + 2)
    v = q8_pool(normal_f16(seed + 3, L_MAX, KV, D), table, page, pool_pages, seed + 4)
    t = np.arange(L_MAX)
    phys = table[t // page].astype(np.int64) * page + t % page
    used = np.zeros(pool_pages * page, bool)
    used[phys] = True
    for pool in (k, v):  # every row no token lives in: poison
        pool.quants[~used] = _poison_quants(pool.quants[~used].shape, seed + 9)
        pool.scales[~used] = NAN16
    up = ctx.buffer_from_iter
    b_q, b_kq, b_ks, b_vq, b_vs, b_tab = up(q16), up(k.quants), up(k.scales), up(v.quants), up(v.scales), up(table)
    row_q, row_s = KV * D, KV * D // 32
    pq, ps = _poison_quants((row_q,), seed + 10), np.full(row_s, NAN16)
    step = ctx.new_step_buffer()
    dec, red = ctx.load_kernel("attn_verify_paged_q8kv_d128" if m_q > 1 else "attn_decode_paged_q8kv_d128"), ctx.load_kernel("attn_reduce_f32_d128")
    rows = m_q * H
    out = ctx.new_buffer(rows * D, np.float32)
    parts = {n: ctx.new_buffer(rows * n * (D + 2), np.float32) for n in splits}
    q32 = q16.astype(np.float32)
    for kv_len in range(L_MAX, m_q - 1, -1):
        if kv_len < L_MAX:  # the token that just left the sequence becomes poison too
            r = int(phys[kv_len])
            for buf, val, n in ((b_kq, pq, row_q), (b_vq, pq, row_q), (b_ks, ps, row_s), (b_vs, ps, row_s)):
                buf.write(val, r * n)
        sg.StepState(kv_len_global=kv_len).write_to(step)
        want = O.attention_f64(q32, k.deq[:kv_len], v.deq[:kv_len], m_q, kv_len - m_q, H, KV, D, SCALE)
        for n in splits:
            ctx.dispatch(dec, bind(b_q, b_kq, b_ks, b_vq, b_vs, b_tab, parts[n], step), (n, SCALE, page), [KV, n, m_q])
            ctx.dispatch_blocking(red, bind(parts[n], out), n, [rows, 1, 1])  # raises if the status word is not zero
            assert_close(out.read().reshape(m_q, H, D), want, what=f"decode kv_len={kv_len} page={page} m_q={m_q} splits={n}")


@pytest.mark.parametrize("q0", [0, 63, 64, 1000])
def test_flash_prefill_every_chunk_size_to_130(ctx, q0):
    import super_gemma_b200 as sg

    M_MAX, windows, heads = 130, (0, 48, 1024), [0, 1, 13, 30, 31]
    L_MAX = q0 + M_MAX
    seed = 0x7200 + q0
    q16, k16, v16 = normal_f16(seed, M_MAX, H, D), normal_f16(seed + 1, L_MAX, KV, D), normal_f16(seed + 2, L_MAX, KV, D)
    pad = 160  # rows past the sequence end that a whole-tile load may touch: poison
    poison_rows = np.full((pad, KV, D), NAN16)
    b_q = ctx.buffer_from_iter(q16)
    b_k = ctx.buffer_from_iter(np.concatenate([k16.view(np.uint16), poison_rows]))
    b_v = ctx.buffer_from_iter(np.concatenate([v16.view(np.uint16), poison_rows]))
    step = ctx.new_step_buffer()
    sg.StepState(q0=q0).write_to(step)
    flash = ctx.load_kernel("attn_prefill_flash_f16_d128")
    q32, k32, v32 = q16.astype(np.float32), k16.astype(np.float32), v16.astype(np.float32)
    for m in range(M_MAX, 0, -1):
        if m < M_MAX:  # the chunk shrank by one token: its query row and its K/V row become poison
            b_q.write(np.full(H * D, NAN16), m * H * D)
            b_k.write(np.full(KV * D, NAN16), (q0 + m) * KV * D)
            b_v.write(np.full(KV * D, NAN16), (q0 + m) * KV * D)
        out = ctx.new_buffer(m * H * D, np.float32)
        for window in windows:
            ctx.dispatch_blocking(flash, bind(b_q, b_k, b_v, out, step), (SCALE, window), [KV, m, 1])
            want = O.attention_f64(q32[:m], k32[:q0 + m], v32[:q0 + m], m, q0, H, KV, D, SCALE, window=window, heads=heads)
            assert_close(out.read().reshape(m, H, D)[:, heads], want, what=f"flash m={m} q0={q0} window={window}")
