"""GPU tests of the dispatch surface itself: record once / replay with step-buffer updates
(crates/sg-gpu/tests/graph.rs:32), error variants, slices, timers."""
import numpy as np
import pytest

from cases import D, H, KV, SCALE, assert_close, bind, normal_f16
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


def test_recorded_graph_follows_step_updates(ctx):
    """Record (append K, append V, split-K decode, reduce) once; drive three steps by rewriting
    only the step buffer and the source rows; every step matches the oracle, and re-driving the
    same state gives the same bits."""
    import super_gemma_b200 as sg

    n_splits, ring = 4, 1024
    row = KV * D
    q = ctx.new_buffer(H * D, np.uint16)
    k_src, v_src = ctx.new_buffer(row, np.uint16), ctx.new_buffer(row, np.uint16)
    k_ring, v_ring = ctx.new_buffer(ring * row, np.uint16), ctx.new_buffer(ring * row, np.uint16)
    part = ctx.new_buffer(H * n_splits * (D + 2), np.float32)
    out = ctx.new_buffer(H * D, np.float32)
    step = ctx.new_step_buffer()
    timer = ctx.new_timer(2)
    app, dec, red = (ctx.load_kernel(n) for n in ("kv_append_sliding_d128", "attn_decode_sliding_d128", "attn_reduce_f32_d128"))

    def record(c):
        timer.stamp(0)
        c.dispatch(app, bind(k_src, k_ring, step), None, app.groups_for(row))
        c.dispatch(app, bind(v_src, v_ring, step), None, app.groups_for(row))
        c.dispatch(dec, bind(q, k_ring, v_ring, part, step), (n_splits, SCALE), [KV, n_splits, 1])
        c.dispatch(red, bind(part, out), n_splits, [H, 1, 1])
        timer.stamp(1)

    graph = ctx.record_graph(record)
    before = ctx.launch_count
    ks, vs, outs = [], [], []
    for pos in range(3):
        q16, k16, v16 = normal_f16(10 + pos, 1, H, D), normal_f16(20 + pos, 1, KV, D), normal_f16(30 + pos, 1, KV, D)
        ks.append(k16)
        vs.append(v16)
        q.write(q16)
        k_src.write(k16)
        v_src.write(v16)
        sg.StepState(pos=pos, kv_len_sliding=pos + 1).write_to(step)
        ctx.submit_blocking(graph)
        got = out.read().reshape(1, H, D)
        want = O.attention_f64(q16.astype(np.float32), np.concatenate(ks).astype(np.float32), np.concatenate(vs).astype(np.float32),
                               1, pos, H, KV, D, SCALE)
        assert_close(got, want, what=f"graph step {pos}")
        outs.append(got.copy())
    assert ctx.launch_count - before == 3 * 4 + 3  # four kernels per replay + one step write per step
    ctx.submit_blocking(graph)  # same state again -> same bits
    assert np.array_equal(out.read().reshape(1, H, D).view(np.uint32), outs[-1].view(np.uint32))
    ns = timer.read_ns()
    assert ns[0] == 0 and ns[1] > 0


def test_error_variants(ctx):
    import super_gemma_b200 as sg

    with pytest.raises(sg.UnknownKernel):
        ctx.load_kernel("attn_decode_nonexistent")
    red = ctx.load_kernel("attn_reduce_f32_d128")
    part, out = ctx.new_buffer(H * 4 * (D + 2), np.float32), ctx.new_buffer(H * D, np.float32)
    with pytest.raises(sg.Validation):  # binding count
        ctx.dispatch(red, bind(part), 4, [H, 1, 1])
    with pytest.raises(sg.Validation):  # push size
        ctx.dispatch(red, bind(part, out), (4, 1.0), [H, 1, 1])
    with pytest.raises(sg.Validation):  # part too small for 8 splits
        ctx.dispatch(red, bind(part, out), 8, [H, 1, 1])
    with pytest.raises(sg.Validation):  # same index twice
        ctx.dispatch(red, [sg.BufferBinding.buffer(0, part), sg.BufferBinding.buffer(0, out)], 4, [H, 1, 1])
    with pytest.raises(sg.Validation):  # slice outside the parent
        part.slice(0, len(part) + 1)
    dec = ctx.load_kernel("attn_decode_paged_q8kv_d128")
    bufs = [ctx.new_buffer(64, np.uint8) for _ in range(8)]
    with pytest.raises(sg.Validation):  # odd number of kv heads
        ctx.dispatch(dec, bind(*bufs), (4, SCALE, 256), [3, 4, 1])
    with pytest.raises(sg.Validation):  # page not a power of two
        ctx.dispatch(dec, bind(*bufs), (4, SCALE, 100), [16, 4, 1])
    with pytest.raises(sg.State):
        import ctypes as C

        out_g = C.c_void_p()
        sg.gpu._check(sg.lib().sgb_graph_end(ctx._h, C.byref(out_g)))
    ctx.sync()


def test_buffers_are_zeroed_and_slices_share_memory(ctx):
    b = ctx.new_buffer(1024, np.float32)
    assert not b.read().any()
    s = b.slice(256, 512)
    s.write(np.arange(256, dtype=np.float32))
    full = b.read()
    assert np.array_equal(full[256:512], np.arange(256, dtype=np.float32)) and not full[:256].any() and not full[512:].any()


def test_decode_splits_hint_fills_the_sms():
    import super_gemma_b200 as sg

    ctx = sg.GpuContext(0)
    sms = sg.lib().sgb_ctx_sm_count(ctx._h)
    n = ctx.decode_splits_hint(16, 1 << 20)
    assert n == sms * 16 // 32 and (16 * n * 2) % 4 == 0  # two warps per (kv head, split), 16 warps per SM
    assert ctx.decode_splits_hint(16, 2048) == 4           # at least 512 tokens per split
    assert ctx.decode_splits_hint(16, 10) == 1
