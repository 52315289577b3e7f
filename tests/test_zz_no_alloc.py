"""The allocation-free decode entry point, called through the C ABI with raw device pointers.

Callers that cannot allocate device memory (all of HBM already belongs to their KV pool, or they
sit in a phase where cudaMalloc is not allowed) use sgb_decode_paged_q8kv_d128_noalloc; its
split-K scratch is a static device array inside the library.  The check: its output equals what the
ordinary dispatch path (attn_decode_paged_q8kv_d128 + attn_reduce_f32_d128, caller-allocated
partials) produces on the same inputs, on two calls in a row that share the static array, and both
match the f64 oracle.  Collected last so that a -x run has finished every other test first."""
import ctypes as C

import numpy as np
import pytest

from cases import D, G, H, KV, PAGE, SCALE, assert_close, bind, normal_f16, page_table, q8_pool
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu


def _case(ctx, seed, kv_len, m_q):
    n_pages = -(-kv_len // PAGE)
    table = page_table(seed + 0x100, n_pages + 1)[:n_pages]
    q16 = normal_f16(seed, m_q, H, D)
    k = q8_pool(normal_f16(seed + 1, kv_len, KV, D), table, PAGE, n_pages + 1, seed + 2)
    v = q8_pool(normal_f16(seed + 3, kv_len, KV, D), table, PAGE, n_pages + 1, seed + 4)
    up = ctx.buffer_from_iter
    return q16, k, v, [up(q16), up(k.quants), up(k.scales), up(v.quants), up(v.scales), up(table)], (n_pages + 1) * PAGE, n_pages


def test_noalloc_decode_matches_the_dispatch_path_twice_in_a_row():
    import super_gemma_b200 as sg

    ctx = sg.GpuContext(0)
    L = sg.lib()
    # two different problems back to back: the second call reuses the static scratch the first one left behind
    for seed, kv_len, m_q, n_splits in [(0x6601, 5000, 1, 64), (0x6602, 1300, 4, 16)]:
        q16, k, v, bufs, pool_rows, n_pages = _case(ctx, seed, kv_len, m_q)
        rows = m_q * H
        # the existing entry point: caller-allocated partials
        import super_gemma_b200 as sg2

        step = ctx.new_step_buffer()
        sg2.StepState(kv_len_global=kv_len).write_to(step)
        part, want_buf = ctx.new_buffer(rows * n_splits * (D + 2), np.float32), ctx.new_buffer(rows * D, np.float32)
        ctx.dispatch(ctx.load_kernel("attn_decode_paged_q8kv_d128"), bind(*bufs, part, step), (n_splits, SCALE, PAGE), [KV, n_splits, m_q])
        ctx.dispatch_blocking(ctx.load_kernel("attn_reduce_f32_d128"), bind(part, want_buf), n_splits, [rows, 1, 1])
        want = want_buf.read()
        # the allocation-free entry point: raw device pointers, its own static scratch
        out = ctx.new_buffer(rows * D, np.float32)
        status = ctx.new_buffer(4, np.uint32)
        p = [C.c_void_p(b.device_ptr) for b in bufs]
        rc = L.sgb_decode_paged_q8kv_d128_noalloc(0, C.c_void_p(ctx.stream), p[0], p[1], p[2], p[3], p[4], p[5], n_pages, pool_rows,
                                                  C.c_void_p(out.device_ptr), C.c_void_p(status.device_ptr), KV, m_q, kv_len,
                                                  n_splits, PAGE, C.c_float(SCALE))
        assert rc == 0, L.sgb_last_error().decode()
        ctx.sync()
        assert not status.read().any()
        got = out.read()
        # same partials, same combine arithmetic: the two entry points agree bit for bit
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"max diff {np.abs(got - want).max()}"
        oracle = O.attention_f64(q16.astype(np.float32), k.deq, v.deq, m_q, kv_len - m_q, H, KV, D, SCALE)
        assert_close(got.reshape(m_q, H, D), oracle, what=f"noalloc decode kv_len={kv_len} m_q={m_q}")

    # The property in the name: once the first call on the device is behind us, a call neither takes nor returns
    # device memory (cudaMemGetInfo reports the same free bytes before and after).
    import torch

    ctx.sync()
    free0 = torch.cuda.mem_get_info(0)[0]
    rc = L.sgb_decode_paged_q8kv_d128_noalloc(0, C.c_void_p(ctx.stream), p[0], p[1], p[2], p[3], p[4], p[5], n_pages, pool_rows,
                                              C.c_void_p(out.device_ptr), C.c_void_p(status.device_ptr), KV, m_q, kv_len,
                                              n_splits, PAGE, C.c_float(SCALE))
    assert rc == 0, L.sgb_last_error().decode()
    ctx.sync()
    free1 = torch.cuda.mem_get_info(0)[0]
    assert free1 == free0, f"free device memory moved by {free0 - free1} bytes across a call"
    assert np.array_equal(out.read().view(np.uint32), want.view(np.uint32))

    # kv_len smaller than the number of query tokens: rejected (such rows would see no key at all)
    rc = L.sgb_decode_paged_q8kv_d128_noalloc(0, C.c_void_p(ctx.stream), p[0], p[1], p[2], p[3], p[4], p[5], n_pages, pool_rows,
                                              C.c_void_p(out.device_ptr), None, KV, 4, 3, 1, PAGE, C.c_float(SCALE))
    assert rc == sg.gpu.SGB_ERR_VALIDATION and "m_q" in L.sgb_last_error().decode()

    # beyond the stated maximum: rejected with a clear error, nothing launched
    rc = L.sgb_decode_paged_q8kv_d128_noalloc(0, C.c_void_p(ctx.stream), p[0], p[1], p[2], p[3], p[4], p[5], n_pages, pool_rows,
                                              C.c_void_p(out.device_ptr), None, KV, 4, kv_len, 64, PAGE, C.c_float(SCALE))
    assert rc == sg.gpu.SGB_ERR_VALIDATION and "2048" in L.sgb_last_error().decode()
