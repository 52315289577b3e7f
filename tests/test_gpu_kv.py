"""GPU parity for the Q8_0 codec and KV placement kernels, through the C ABI.  Bit-exact against the
oracle; cases follow crates/sg-gpu/tests/parity_kv.rs (ring wrap at 1022, linear append at 7, an
all-zero block, determinism) and add the page-table placement this build defines."""
import numpy as np
import pytest

from cases import bind
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


def test_kv_quant_q8_bit_exact_and_deterministic(ctx):  # parity_kv.rs:131, :215
    x = O.through_f16(O.Rng(0xB2).f32_vec(4352))
    x[64:96] = 0.0
    src = ctx.buffer_from_iter(O.f32_to_f16_bits(x))
    scales, quants = ctx.new_buffer(4352 // 32, np.uint16), ctx.new_buffer(4352, np.int8)
    k = ctx.load_kernel("kv_quant_q8")
    ctx.dispatch_blocking(k, bind(src, scales, quants), None, k.groups_for(4352 // 32))
    want_s, want_q = O.quant_q8_0(x)
    got_s, got_q = scales.read(), quants.read()
    assert np.array_equal(got_s, want_s)  # scales: bit-exact
    assert np.array_equal(got_q, want_q)  # quants: IEEE division on both sides, so exact here too
    assert got_s[2] == 0 and not got_q[64:96].any()
    # dequant exact on GPU-produced data
    dst = ctx.new_buffer(4352, np.uint16)
    kd = ctx.load_kernel("kv_dequant_q8")
    ctx.dispatch_blocking(kd, bind(scales, quants, dst), None, kd.groups_for(4352 // 32))
    assert np.array_equal(dst.read(), O.dequant_q8_0_f16(got_s, got_q))
    # run twice -> bit-identical
    s2, q2 = ctx.new_buffer(4352 // 32, np.uint16), ctx.new_buffer(4352, np.int8)
    ctx.dispatch_blocking(k, bind(src, s2, q2), None, k.groups_for(4352 // 32))
    assert np.array_equal(s2.read(), got_s) and np.array_equal(q2.read(), got_q)


def test_kv_quant_q8_large_random(ctx):
    x = np.random.default_rng(3).standard_normal(1 << 20, dtype=np.float32).astype(np.float16)
    src = ctx.buffer_from_iter(x)
    scales, quants = ctx.new_buffer(x.size // 32, np.uint16), ctx.new_buffer(x.size, np.int8)
    k = ctx.load_kernel("kv_quant_q8")
    ctx.dispatch_blocking(k, bind(src, scales, quants), None, k.groups_for(x.size // 32))
    want_s, want_q = O.quant_q8_0(x.astype(np.float32))
    assert np.array_equal(scales.read(), want_s) and np.array_equal(quants.read(), want_q)


def test_kv_append_ring_wrap(ctx):  # parity_kv.rs:36
    import super_gemma_b200 as sg

    for name, row in (("kv_append_sliding", 4096), ("kv_append_sliding_d128", 2048)):
        src_h = O.f32_to_f16_bits(O.Rng(0xB0).f32_vec(5 * row))
        src = ctx.buffer_from_iter(src_h)
        dst = ctx.buffer_from_iter(np.full(1024 * row, 0x7E00, np.uint16))
        step = ctx.new_step_buffer()
        sg.StepState(pos=1022).write_to(step)
        k = ctx.load_kernel(name)
        ctx.dispatch_blocking(k, bind(src, dst, step), None, k.groups_for(5 * row))
        want = np.full(1024 * row, 0x7E00, np.uint16)
        O.kv_append(src_h, want, row, 1022, ring=1024)
        assert np.array_equal(dst.read(), want)


def test_kv_append_linear_and_out_of_range_is_reported(ctx):  # parity_kv.rs:85
    import super_gemma_b200 as sg

    row = 2048
    src_h = O.f32_to_f16_bits(O.Rng(0xB1).f32_vec(3 * row))
    src = ctx.buffer_from_iter(src_h)
    dst = ctx.buffer_from_iter(np.full(16 * row, 0x7E00, np.uint16))
    step = ctx.new_step_buffer()
    sg.StepState(pos=7).write_to(step)
    k = ctx.load_kernel("kv_append_global")
    ctx.dispatch_blocking(k, bind(src, dst, step), None, k.groups_for(3 * row))
    want = np.full(16 * row, 0x7E00, np.uint16)
    O.kv_append(src_h, want, row, 7)
    assert np.array_equal(dst.read(), want)
    # a slot past the end of dst is skipped and reported, not written
    sg.StepState(pos=15).write_to(step)
    with pytest.raises(sg.Bounds):
        ctx.dispatch_blocking(k, bind(src, dst, step), None, k.groups_for(3 * row))
    ctx.sync()  # the status word was cleared; the context stays usable


def test_kv_append_global_q8_and_paged(ctx):
    import super_gemma_b200 as sg

    row, n, slots = 2048, 6, 600
    src_h = O.f32_to_f16_bits(O.Rng(0xB3).f32_vec(n * row))
    src = ctx.buffer_from_iter(src_h)
    step = ctx.new_step_buffer()
    sg.StepState(pos=254).write_to(step)
    for paged in (False, True):
        scales, quants = ctx.new_buffer(slots * row // 32, np.uint16), ctx.new_buffer(slots * row, np.int8)
        ws, wq = np.zeros(slots * row // 32, np.uint16), np.zeros(slots * row, np.int8)
        if paged:
            table_h = np.array([1, 0], np.uint32)
            table = ctx.buffer_from_iter(table_h)
            k = ctx.load_kernel("kv_append_paged_q8_d128")
            ctx.dispatch_blocking(k, bind(src, scales, quants, table, step), (row, 256), k.groups_for(n * row // 32))
            O.kv_append_q8(src_h, ws, wq, row, 254, page_table=table_h, page=256)
        else:
            k = ctx.load_kernel("kv_append_global_q8")
            ctx.dispatch_blocking(k, bind(src, scales, quants, step), None, k.groups_for(n * row // 32))
            O.kv_append_q8(src_h, ws, wq, row, 254)
        assert np.array_equal(scales.read(), ws) and np.array_equal(quants.read(), wq)


def test_kv_dequant_paged_gathers_to_linear(ctx):
    import super_gemma_b200 as sg
    from cases import normal_f16, page_table, q8_pool

    n_kv, page, n_tokens = 4, 64, 300
    table_h = page_table(5, 7)[:5]
    pool = q8_pool(normal_f16(6, n_tokens, n_kv, 128), table_h, page, pool_pages=7)
    scales, quants = ctx.buffer_from_iter(pool.scales), ctx.buffer_from_iter(pool.quants)
    table = ctx.buffer_from_iter(table_h)
    dst = ctx.buffer_from_iter(np.full(400 * n_kv * 128, 0x7E00, np.uint16))
    step = ctx.new_step_buffer()
    sg.StepState(kv_len_global=n_tokens).write_to(step)
    k = ctx.load_kernel("kv_dequant_paged_q8_d128")
    ctx.dispatch_blocking(k, bind(scales, quants, table, dst, step), (n_kv * 128, page), [1, 1, 1])
    got = dst.read().reshape(400, n_kv, 128)
    assert np.array_equal(O.f16_bits_to_f32(got[:n_tokens]), pool.deq16)
    assert np.all(got[n_tokens:320] == 0)  # the rest of the last 64-key tile is zeroed: the flash kernel reads it under a mask
    assert np.all(got[320:] == 0x7E00)  # rows beyond that are left alone
