"""GPU parity for the steps before attention: per-head RMS norm, rotate-half RoPE and the fused
norm + RoPE + Q8_0 quantise + paged append, through the C ABI.  The reference-named kernels replay the
reference's own seeded cases at its own tolerance (crates/sg-gpu/tests/parity_elementwise.rs:20-135:
|got - want| <= 2e-3 + 1e-3 |want| against the f64 CPU reference); the fused head_dim-128 kernels are
held to the same tolerance against the f64 chain and to bit-exactness against their own unfused pieces."""
import numpy as np
import pytest

from cases import assert_close, bind
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-3  # parity_elementwise.rs:22-23


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


def test_rmsnorm_matches_reference_for_head_rows(ctx):  # parity_elementwise.rs:26
    rng = O.Rng(0xA11CE)
    rows = 7
    for variant, row_len, plus_one in [("rmsnorm_5376", 5376, False), ("rmsnorm_5376_plus1", 5376, True), ("rmsnorm_512", 512, False),
                                       ("rmsnorm_512_plus1", 512, True), ("rmsnorm_256", 256, False), ("rmsnorm_256_plus1", 256, True)]:
        x = O.through_f16(rng.f32_vec(rows * row_len))
        w = rng.f32_vec(row_len)
        if row_len == 5376:
            continue  # hidden-size rows are not on the attention path; the draws keep the seeded sequence
        y = ctx.new_buffer(rows * row_len, np.uint16)
        ctx.dispatch_blocking(ctx.load_kernel(variant), bind(ctx.buffer_from_iter(O.f32_to_f16_bits(x)), ctx.buffer_from_iter(w), y), None,
                              [rows, 1, 1])
        got = O.f16_bits_to_f32(y.read())
        assert_close(got, O.rmsnorm_f64(x, w, row_len, 1e-6, plus_one), ATOL, RTOL, variant)
        again = ctx.new_buffer(rows * row_len, np.uint16)
        ctx.dispatch_blocking(ctx.load_kernel(variant), bind(ctx.buffer_from_iter(O.f32_to_f16_bits(x)), ctx.buffer_from_iter(w), again),
                              None, [rows, 1, 1])
        assert np.array_equal(again.read(), y.read())  # parity_elementwise.rs:216


def test_rope_matches_reference_for_all_sites(ctx):  # parity_elementwise.rs:72
    rng = O.Rng(0x40FE)
    for variant, head_dim, rot_dims, n_heads, theta in [("rope_sliding_q", 256, 256, 32, 1e4), ("rope_sliding_k", 256, 256, 16, 1e4),
                                                         ("rope_global_q", 512, 128, 32, 1e6), ("rope_global_k", 512, 128, 4, 1e6)]:
        kernel = ctx.load_kernel(variant)
        inv_freq = O.inv_freqs(rot_dims, theta)
        for start_pos in (0, 1, 1023, 100_000):
            tokens = 3
            n = tokens * n_heads * head_dim
            x = O.through_f16(rng.f32_vec(n))
            cs = O.cos_sin_table(inv_freq, start_pos, tokens)
            buf = ctx.buffer_from_iter(O.f32_to_f16_bits(x))
            pairs = (n // head_dim) * (rot_dims // 2)
            ctx.dispatch_blocking(kernel, bind(buf, ctx.buffer_from_iter(cs)), None, kernel.groups_for(pairs))
            got = O.f16_bits_to_f32(buf.read())
            assert_close(got, O.rope_f64(x, head_dim, rot_dims, n_heads, cs), ATOL, RTOL, f"{variant}@{start_pos}")
            if rot_dims < head_dim:  # the frozen pairs pass through untouched
                live, half = rot_dims // 2, head_dim // 2
                g, xx = got.reshape(-1, head_dim), x.reshape(-1, head_dim)
                assert np.array_equal(g[:, live:half], xx[:, live:half]) and np.array_equal(g[:, half + live:], xx[:, half + live:])


def _chain_f64(x, w, n_heads, rot_dims, cs, plus_one=False):
    """The reference chain: rmsnorm -> f16 -> rope -> f16."""
    y = O.through_f16(O.rmsnorm_f64(x, w, 128, 1e-6, plus_one))
    if rot_dims:
        y = O.through_f16(O.rope_f64(y, 128, rot_dims, n_heads, cs))
    return y


@pytest.mark.parametrize("tokens,n_heads,rot_dims,plus_one,start", [(5, 32, 128, 0, 0), (3, 16, 128, 0, 100_000), (4, 16, 32, 1, 77), (2, 16, 0, 0, 0),
                                                                   (1, 1, 64, 0, 3)])
def test_fused_norm_rope_d128(ctx, tokens, n_heads, rot_dims, plus_one, start):
    rng = O.Rng(0xD128 + tokens + rot_dims)
    x = O.through_f16(rng.f32_vec(tokens * n_heads * 128))
    w = rng.f32_vec(128)
    cs = O.cos_sin_table(O.inv_freqs(max(rot_dims, 2), 1e6), start, tokens) if rot_dims else np.zeros(2, np.float32)
    y = ctx.new_buffer(x.size, np.uint16)
    ctx.dispatch_blocking(ctx.load_kernel("attn_norm_rope_d128"), bind(ctx.buffer_from_iter(O.f32_to_f16_bits(x)), ctx.buffer_from_iter(w),
                                                                       ctx.buffer_from_iter(cs), y), (n_heads, rot_dims, plus_one), [1, 1, 1])
    got = O.f16_bits_to_f32(y.read())
    assert_close(got, _chain_f64(x, w, n_heads, rot_dims, cs, bool(plus_one)), ATOL, RTOL, f"norm+rope rot={rot_dims}")
    if rot_dims and rot_dims < 128:  # dims outside the live pairs carry the norm only
        g = got.reshape(-1, 128)
        n_only = O.through_f16(O.rmsnorm_f64(x, w, 128, 1e-6, bool(plus_one))).reshape(-1, 128)
        live = rot_dims // 2
        assert_close(g[:, live:64], n_only[:, live:64], ATOL, RTOL, "frozen low half")
        assert_close(g[:, 64 + live:], n_only[:, 64 + live:], ATOL, RTOL, "frozen high half")


@pytest.mark.parametrize("tokens,pos,rot_dims", [(6, 254, 128), (1, 0, 128), (9, 700, 32)])
def test_fused_kv_append_equals_its_unfused_pieces(ctx, tokens, pos, rot_dims):
    """norm(k) + rope(k) + norm(v) + quantise + paged append in one launch gives the bits of
    attn_norm_rope_d128 followed by kv_append_paged_q8_d128, and the values of the f64 chain."""
    import super_gemma_b200 as sg

    n_kv, page, pool_pages = 4, 64, 16
    row = n_kv * 128
    rng = O.Rng(0xFA5E + tokens)
    k_raw, v_raw = O.through_f16(rng.f32_vec(tokens * row)), O.through_f16(rng.f32_vec(tokens * row))
    k_w = rng.f32_vec(128)
    cs = O.cos_sin_table(O.inv_freqs(rot_dims, 1e6), pos, tokens)
    table_h = np.random.default_rng(3).permutation(pool_pages).astype(np.uint32)
    up = ctx.buffer_from_iter
    kr, vr, kw, csb, table = up(O.f32_to_f16_bits(k_raw)), up(O.f32_to_f16_bits(v_raw)), up(k_w), up(cs), up(table_h)
    step = ctx.new_step_buffer()
    sg.StepState(pos=pos).write_to(step)
    rows = pool_pages * page
    fill = np.random.default_rng(4)

    def pools():
        return (up(fill.integers(0, 2**15, rows * row // 32).astype(np.uint16)), up(fill.integers(-127, 128, rows * row, dtype=np.int8)))

    fill = np.random.default_rng(4)
    ks1, kq1 = pools()
    vs1, vq1 = pools()
    fill = np.random.default_rng(4)
    ks2, kq2 = pools()
    vs2, vq2 = pools()
    fused = ctx.load_kernel("kv_norm_rope_append_paged_q8_d128")
    ctx.dispatch_blocking(fused, bind(kr, vr, kw, csb, ks1, kq1, vs1, vq1, table, step), (row, page, rot_dims, 0), [1, 1, 1])
    # the unfused pieces
    nr, app = ctx.load_kernel("attn_norm_rope_d128"), ctx.load_kernel("kv_append_paged_q8_d128")
    k_f16, v_f16 = ctx.new_buffer(tokens * row, np.uint16), ctx.new_buffer(tokens * row, np.uint16)
    ones = up(np.ones(128, np.float32))
    ctx.dispatch_blocking(nr, bind(kr, kw, csb, k_f16), (n_kv, rot_dims, 0), [1, 1, 1])
    ctx.dispatch_blocking(nr, bind(vr, ones, csb, v_f16), (n_kv, 0, 0), [1, 1, 1])
    ctx.dispatch_blocking(app, bind(k_f16, ks2, kq2, table, step), (row, page), app.groups_for(tokens * row // 32))
    ctx.dispatch_blocking(app, bind(v_f16, vs2, vq2, table, step), (row, page), app.groups_for(tokens * row // 32))
    for a, b in ((ks1, ks2), (kq1, kq2), (vs1, vs2), (vq1, vq2)):
        assert np.array_equal(a.read(), b.read())
    # and the values: dequantised rows against the f64 chain, within half a quantisation step
    t = pos + np.arange(tokens)
    phys = table_h[t // page].astype(np.int64) * page + t % page
    for raw, w, rot, sc, qu in ((k_raw, k_w, rot_dims, ks1, kq1), (v_raw, np.ones(128, np.float32), 0, vs1, vq1)):
        want = _chain_f64(raw, w, n_kv, rot, cs).reshape(tokens, row)
        s = sc.read().reshape(rows, row // 32)[phys]
        q = qu.read().reshape(rows, row)[phys]
        d = O.f16_bits_to_f32(s)
        got = np.repeat(d, 32, axis=1) * q.astype(np.float32)
        assert np.all(np.abs(got - want) <= 0.57 * np.repeat(d, 32, axis=1) + ATOL)


def test_fused_kv_append_reports_a_short_table(ctx):
    import super_gemma_b200 as sg

    n_kv, page = 2, 64
    row = n_kv * 128
    up = ctx.buffer_from_iter
    z = np.zeros(row, np.uint16)
    step = ctx.new_step_buffer()
    sg.StepState(pos=64).write_to(step)  # page 1 of a one-entry table
    bufs = bind(up(z), up(z), up(np.ones(128, np.float32)), up(np.zeros(128, np.float32)), ctx.new_buffer(page * row // 32, np.uint16),
                ctx.new_buffer(page * row, np.int8), ctx.new_buffer(page * row // 32, np.uint16), ctx.new_buffer(page * row, np.int8),
                up(np.zeros(1, np.uint32)), step)
    with pytest.raises(sg.Bounds):
        ctx.dispatch_blocking(ctx.load_kernel("kv_norm_rope_append_paged_q8_d128"), bufs, (row, page, 128, 0), [1, 1, 1])
    ctx.sync()


@pytest.mark.parametrize("tokens,n_kv", [(1, 4), (5, 4), (3, 16), (2, 1)])
def test_one_launch_qkv_equals_the_two_kernels(ctx, tokens, n_kv):
    """qkv_norm_rope_append_paged_q8_d128 = attn_norm_rope_d128 on q + kv_norm_rope_append_paged_q8_d128, bit for bit
    (also when the K/V blocks do not end on a warp boundary: n_kv = 1 gives 8 blocks per token)."""
    import super_gemma_b200 as sg

    n_q, page, pool_pages, rot, pos = 2 * n_kv, 64, 4, 128, 70
    row = n_kv * 128
    rng = O.Rng(0x0DE + tokens + n_kv)
    q_raw, k_raw, v_raw = (O.through_f16(rng.f32_vec(tokens * h * 128)) for h in (n_q, n_kv, n_kv))
    q_w, k_w = rng.f32_vec(128), rng.f32_vec(128)
    cs = O.cos_sin_table(O.inv_freqs(rot, 1e6), pos, tokens)
    up = ctx.buffer_from_iter
    qr, kr, vr, qw, kw, csb = up(O.f32_to_f16_bits(q_raw)), up(O.f32_to_f16_bits(k_raw)), up(O.f32_to_f16_bits(v_raw)), up(q_w), up(k_w), up(cs)
    table = up(np.array([2, 0, 3, 1], np.uint32))
    step = ctx.new_step_buffer()
    sg.StepState(pos=pos).write_to(step)
    rows = pool_pages * page
    mk = lambda dt, n: ctx.new_buffer(n, dt)
    a = [mk(np.uint16, rows * row // 32), mk(np.int8, rows * row), mk(np.uint16, rows * row // 32), mk(np.int8, rows * row)]
    b = [mk(np.uint16, rows * row // 32), mk(np.int8, rows * row), mk(np.uint16, rows * row // 32), mk(np.int8, rows * row)]
    q1, q2 = mk(np.uint16, tokens * n_q * 128), mk(np.uint16, tokens * n_q * 128)
    ctx.dispatch_blocking(ctx.load_kernel("qkv_norm_rope_append_paged_q8_d128"), bind(qr, qw, q1, kr, vr, kw, csb, *a, table, step),
                          (n_q, row, page, rot, 0), [1, 1, 1])
    ctx.dispatch_blocking(ctx.load_kernel("attn_norm_rope_d128"), bind(qr, qw, csb, q2), (n_q, rot, 0), [1, 1, 1])
    ctx.dispatch_blocking(ctx.load_kernel("kv_norm_rope_append_paged_q8_d128"), bind(kr, vr, kw, csb, *b, table, step), (row, page, rot, 0),
                          [1, 1, 1])
    assert np.array_equal(q1.read(), q2.read())
    assert np.any(q1.read() != 0)
    for x, y in zip(a, b):
        assert np.array_equal(x.read(), y.read())
    assert np.any(a[1].read() != 0)
