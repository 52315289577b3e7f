"""GPU tests of the whole attention block of a decode step, driven the way the reference's caller drives
sg-gpu: record once, then per token only write the step words and the token's inputs and replay
(crates/sg-gpu/src/graph.rs:29-61,523-528; crates/sg-model/src/graph.rs:552-640).  The block is
one launch for norm + RoPE of q and norm + RoPE + quantise + paged append of k and v, split-K decode over
the paged Q8_0 cache, and the combine.  Page tables come from the cache2 manager.  The second test is the
speculative step of docs/plans/07-mtp-speculative-decoding.md:23-27,58-59: append K draft tokens, verify
them in one launch, accept a prefix, and roll back by truncating the lengths."""
import numpy as np
import pytest

from cases import ATOL, D, G, RTOL, SCALE, assert_close, bind
from oracle import sg_oracle as O

pytestmark = pytest.mark.gpu

N_KV, PAGE, POOL, ROT, THETA = 4, 64, 16, 128, 1e6
N_Q = N_KV * G
ROW = N_KV * D


@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


class Block:
    """Device state of one attention layer plus the f64 mirror of what it should hold."""

    def __init__(self, ctx, capacity, seed):
        from super_gemma_b200 import cache2

        self.ctx, self.rng = ctx, O.Rng(seed)
        up = ctx.buffer_from_iter
        rows = POOL * PAGE
        fill = np.random.default_rng(seed)
        mk_s = lambda: up(fill.integers(0, 2**15, rows * ROW // 32).astype(np.uint16))
        mk_q = lambda: up(fill.integers(-127, 128, rows * ROW, dtype=np.int8))
        self.ks, self.kq, self.vs, self.vq = mk_s(), mk_q(), mk_s(), mk_q()
        self.q_w, self.k_w = self.rng.f32_vec(D) + 1.0, self.rng.f32_vec(D) + 1.0
        self.q_w_d, self.k_w_d = up(self.q_w), up(self.k_w)
        self.cache = cache2.PageCache(POOL, PAGE)
        self.tokens = np.arange(capacity, dtype=np.int32) + seed
        self.seq = self.cache.acquire(self.tokens[:0], capacity_tokens=capacity)
        self.table = up(self.seq.table)
        self.step = ctx.new_step_buffer()
        self.inv_freq = O.inv_freqs(ROT, THETA)
        self.k_ref = np.zeros((0, N_KV, D), np.float32)  # what the cache should dequantise to
        self.v_ref = np.zeros((0, N_KV, D), np.float32)

    def _deq(self, x):
        s, q = O.quant_q8_0(x)
        return O.dequant_q8_0_f32(s, q).reshape(-1, N_KV, D)

    def draw(self, n):
        """Raw q, k, v rows of n new tokens (as the QKV projections would leave them, f16)."""
        return tuple(O.through_f16(self.rng.f32_vec(n * h * D)) for h in (N_Q, N_KV, N_KV))

    def mirror_append(self, k_raw, v_raw, pos):
        n = len(k_raw) // ROW
        cs = O.cos_sin_table(self.inv_freq, pos, n)
        k = O.through_f16(O.rope_f64(O.through_f16(O.rmsnorm_f64(k_raw, self.k_w, D)), D, ROT, N_KV, cs))
        v = O.through_f16(O.rmsnorm_f64(v_raw, np.ones(D, np.float32), D))
        self.k_ref = np.concatenate([self.k_ref[:pos], self._deq(k)])
        self.v_ref = np.concatenate([self.v_ref[:pos], self._deq(v)])
        return cs

    def mirror_q(self, q_raw, cs):
        n = len(q_raw) // (N_Q * D)
        return O.through_f16(O.rope_f64(O.through_f16(O.rmsnorm_f64(q_raw, self.q_w, D)), D, ROT, N_Q, cs)).reshape(n, N_Q, D)

    def want(self, q, kv_len):
        m = len(q)
        return O.attention_f64(q, self.k_ref[:kv_len], self.v_ref[:kv_len], m, kv_len - m, N_Q, N_KV, D, SCALE)


def test_recorded_decode_block_replays_across_a_page_boundary(ctx):
    import super_gemma_b200 as sg

    b = Block(ctx, 256, 0x10C)
    up = ctx.buffer_from_iter
    # history: 125 tokens in one fused append
    _, k_raw, v_raw = b.draw(125)
    cs = b.mirror_append(k_raw, v_raw, 0)
    fused = ctx.load_kernel("kv_norm_rope_append_paged_q8_d128")
    sg.StepState(pos=0).write_to(b.step)
    ctx.dispatch_blocking(fused, bind(up(O.f32_to_f16_bits(k_raw)), up(O.f32_to_f16_bits(v_raw)), b.k_w_d, up(cs), b.ks, b.kq, b.vs, b.vq,
                                      b.table, b.step), (ROW, PAGE, ROT, 0), [1, 1, 1])
    # the per-token block, recorded once
    n_splits = 3
    q_raw_d, k_raw_d, v_raw_d = ctx.new_buffer(N_Q * D, np.uint16), ctx.new_buffer(ROW, np.uint16), ctx.new_buffer(ROW, np.uint16)
    cs_d = ctx.new_buffer(ROT, np.float32)
    q_d = ctx.new_buffer(N_Q * D, np.uint16)
    part = ctx.new_buffer(N_Q * n_splits * (D + 2), np.float32)
    out = ctx.new_buffer(N_Q * D, np.float32)
    kernels = [ctx.load_kernel(n) for n in ("qkv_norm_rope_append_paged_q8_d128", "attn_decode_paged_q8kv_d128", "attn_reduce_f32_d128")]

    def record(c):
        c.dispatch(kernels[0], bind(q_raw_d, b.q_w_d, q_d, k_raw_d, v_raw_d, b.k_w_d, cs_d, b.ks, b.kq, b.vs, b.vq, b.table, b.step),
                   (N_Q, ROW, PAGE, ROT, 0), [1, 1, 1])
        c.dispatch(kernels[1], bind(q_d, b.kq, b.ks, b.vq, b.vs, b.table, part, b.step), (n_splits, SCALE, PAGE), [N_KV, n_splits, 1])
        c.dispatch(kernels[2], bind(part, out), n_splits, [N_Q, 1, 1])

    graph = ctx.record_graph(record)
    for pos in range(125, 131):  # 127 -> 128 crosses into the third page
        q_raw, k_raw, v_raw = b.draw(1)
        cs = b.mirror_append(k_raw, v_raw, pos)
        for buf, val in ((q_raw_d, O.f32_to_f16_bits(q_raw)), (k_raw_d, O.f32_to_f16_bits(k_raw)), (v_raw_d, O.f32_to_f16_bits(v_raw)),
                         (cs_d, cs)):
            buf.write(val)
        sg.StepState(pos=pos, kv_len_global=pos + 1).write_to(b.step)  # the only per-step state (graph.rs:29-48)
        ctx.submit_blocking(graph)
        got = out.read().reshape(1, N_Q, D)
        assert_close(got, b.want(b.mirror_q(q_raw, cs), pos + 1), ATOL, RTOL, f"decode step at pos {pos}")


def test_speculative_verify_then_rollback(ctx):
    import super_gemma_b200 as sg

    b = Block(ctx, 256, 0x5BEC)
    up = ctx.buffer_from_iter
    fused = ctx.load_kernel("kv_norm_rope_append_paged_q8_d128")
    norm_q = ctx.load_kernel("attn_norm_rope_d128")
    reduce = ctx.load_kernel("attn_reduce_f32_d128")

    def append(k_raw, v_raw, pos):
        cs = b.mirror_append(k_raw, v_raw, pos)
        sg.StepState(pos=pos).write_to(b.step)
        ctx.dispatch_blocking(fused, bind(up(O.f32_to_f16_bits(k_raw)), up(O.f32_to_f16_bits(v_raw)), b.k_w_d, up(cs), b.ks, b.kq, b.vs,
                                          b.vq, b.table, b.step), (ROW, PAGE, ROT, 0), [1, 1, 1])
        return cs

    def attend(q_raw, cs, kv_len, kernel, n_splits=2):
        m = len(q_raw) // (N_Q * D)
        q_d = ctx.new_buffer(m * N_Q * D, np.uint16)
        ctx.dispatch_blocking(norm_q, bind(up(O.f32_to_f16_bits(q_raw)), b.q_w_d, up(cs), q_d), (N_Q, ROT, 0), [1, 1, 1])
        part = ctx.new_buffer(m * N_Q * n_splits * (D + 2), np.float32)
        out = ctx.new_buffer(m * N_Q * D, np.float32)
        sg.StepState(kv_len_global=kv_len).write_to(b.step)
        ctx.dispatch(ctx.load_kernel(kernel), bind(q_d, b.kq, b.ks, b.vq, b.vs, b.table, part, b.step), (n_splits, SCALE, PAGE),
                     [N_KV, n_splits, m])
        ctx.dispatch_blocking(reduce, bind(part, out), n_splits, [m * N_Q, 1, 1])
        return out.read().reshape(m, N_Q, D)

    _, k_raw, v_raw = b.draw(190)
    append(k_raw, v_raw, 0)
    # four draft tokens: appended first, then verified together; query i sees keys <= 190 + i
    q_raw, k_raw, v_raw = b.draw(4)
    cs = append(k_raw, v_raw, 190)
    got = attend(q_raw, cs, 194, "attn_verify_paged_q8kv_d128")
    assert_close(got, b.want(b.mirror_q(q_raw, cs), 194), ATOL, RTOL, "verify of 4 drafts")
    # two are accepted: the lengths go back to 192, the next token overwrites the rejected rows
    q_raw, k_raw, v_raw = b.draw(1)
    cs = append(k_raw, v_raw, 192)
    assert len(b.k_ref) == 193
    got = attend(q_raw, cs, 193, "attn_decode_paged_q8kv_d128")
    assert_close(got, b.want(b.mirror_q(q_raw, cs), 193), ATOL, RTOL, "decode after rollback")
