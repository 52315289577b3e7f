"""Parity at the shapes the throughput numbers are quoted on (benchmark config 5): a 4096-token query chunk at
q0 = 126 976 over 131 072 cached Q8_0 tokens behind a seeded RANDOM page table (5a), and a one-token decode over
the same 131 072-token cache (5b).  Nothing is overridden: the prefill launcher cuts the key range into the number
of pieces it chooses for this grid, the decode uses the library's split-count hint.  The f64 oracle runs on
dequantised inputs; tolerance max-abs 2e-3 + relative 1e-2 (form of crates/sg-gpu/tests/reference/mod.rs:137-153).
One 131 072-token pool (16 kv heads, K and V) is built once for both tests."""
import numpy as np
import pytest

from cases import D, G, H, KV, PAGE, SCALE, assert_close, bind, normal_f16, page_table, q8_pool
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu

CTX_LEN, CHUNK = 131072, 4096


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


@pytest.fixture(scope="module")
def cache(ctx):
    n_pages = CTX_LEN // PAGE
    table = page_table(0x5605 + 0x100, n_pages + 3)[:n_pages]  # 512 of 515 pool pages, shuffled
    k = q8_pool(normal_f16(0x5605 + 1, CTX_LEN, KV, D), table, PAGE, n_pages + 3, 0x5605 + 2)
    v = q8_pool(normal_f16(0x5605 + 3, CTX_LEN, KV, D), table, PAGE, n_pages + 3, 0x5605 + 4)
    up = ctx.buffer_from_iter
    bufs = [up(k.quants), up(k.scales), up(v.quants), up(v.scales), up(table)]
    return k, v, bufs


def test_cfg5a_chunked_prefill_random_table_default_pieces(ctx, cache, monkeypatch):
    import super_gemma_b200 as sg

    monkeypatch.delenv("SGB_FLASH_PIECES", raising=False)
    k, v, bufs = cache
    m, q0 = CHUNK, CTX_LEN - CHUNK
    q16 = normal_f16(0x5605, m, H, D)
    k_lin, v_lin = ctx.new_buffer(CTX_LEN * KV * D, np.uint16), ctx.new_buffer(CTX_LEN * KV * D, np.uint16)
    out = ctx.new_buffer(m * H * D, np.float32)
    step = ctx.new_step_buffer()
    sg.StepState(pos=q0, kv_len_global=CTX_LEN, q0=q0).write_to(step)
    ctx.dispatch_blocking(ctx.load_kernel("attn_prefill_paged_q8kv_flash_d128"),
                          bind(ctx.buffer_from_iter(q16), *bufs, k_lin, v_lin, out, step), (SCALE, PAGE), [KV, m, 1])
    got = out.read().reshape(m, H, D)
    assert np.all(np.isfinite(got))
    # first / last rows, both sides of every 64-token query tile edge near the ends, and a seeded sample
    tokens = np.unique(np.concatenate([[0, 1, 63, 64, 65, 127, 128, 2047, 2048, 4031, 4032, 4094, 4095],
                                       np.random.default_rng(5).integers(0, m, 28)])).astype(np.uint32)
    want = O.attention_f64(q16.astype(np.float32), k.deq16, v.deq16, m, q0, H, KV, D, SCALE, tokens=tokens)
    assert_close(got[tokens], want, what="cfg5a sampled rows")
    # bit-exact Q8_0 dequantisation and page-table indexing at this size: the gathered scratch is f16(scale * q)
    rows = np.random.default_rng(6).integers(0, CTX_LEN, 512)
    lin = k_lin.read().reshape(CTX_LEN, KV, D)
    assert np.array_equal(O.f16_bits_to_f32(lin[rows]), k.deq16[rows])


def test_cfg5b_decode_128k_hint_splits(ctx, cache):
    import super_gemma_b200 as sg

    k, v, bufs = cache
    n_splits = ctx.decode_splits_hint(KV, CTX_LEN)
    q16 = normal_f16(0x5615, 1, H, D)
    part, out = ctx.new_buffer(H * n_splits * (D + 2), np.float32), ctx.new_buffer(H * D, np.float32)
    step = ctx.new_step_buffer()
    sg.StepState(kv_len_global=CTX_LEN).write_to(step)
    dec, red = ctx.load_kernel("attn_decode_paged_q8kv_d128"), ctx.load_kernel("attn_reduce_f32_d128")
    runs = []
    for _ in range(2):
        ctx.dispatch(dec, bind(ctx.buffer_from_iter(q16), *bufs, part, step), (n_splits, SCALE, PAGE), [KV, n_splits, 1])
        ctx.dispatch_blocking(red, bind(part, out), n_splits, [H, 1, 1])
        runs.append(out.read().reshape(1, H, D))
    want = O.attention_f64(q16.astype(np.float32), k.deq, v.deq, 1, CTX_LEN - 1, H, KV, D, SCALE)
    assert_close(runs[0], want, what=f"cfg5b decode, {n_splits} splits")
    assert np.array_equal(runs[0].view(np.uint32), runs[1].view(np.uint32))
