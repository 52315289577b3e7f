"""The committed golden vectors (tests/golden/attn_golden.npz, made by tests/golden/make_golden.py
from the numpy-only restatement) against the C oracle on the CPU and against the CUDA kernels
through the C ABI on the GPU."""
import os

import numpy as np
import pytest

from cases import assert_close, bind
from oracle import sg_oracle as O

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_golden.npz"))
H, KV, D, PAGE, KV_LEN, M = (int(x) for x in GOLD["meta"])
SCALE = 0.08838834764831845


def _src(name, round_f16=False):
    return O.KvSrc(quants=GOLD[f"{name}_quants"], scales=GOLD[f"{name}_scales"], page_table=GOLD["page_table"], page=PAGE,
                   round_f16=round_f16)


# ---- CPU: the oracle reproduces the golden vectors ----------------------------------------------
def test_oracle_codec_matches_golden_bits():
    x = O.f16_bits_to_f32(GOLD["codec_x"])
    s, q = O.quant_q8_0(x)
    assert np.array_equal(s, GOLD["codec_scales"]) and np.array_equal(q, GOLD["codec_quants"])
    assert np.array_equal(O.dequant_q8_0_f16(s, q), GOLD["codec_deq16"])


def test_oracle_attention_matches_golden():
    k, v = O.kv_materialize(_src("k"), KV_LEN, KV, D), O.kv_materialize(_src("v"), KV_LEN, KV, D)
    q1 = O.f16_bits_to_f32(GOLD["decode_q"])
    assert np.allclose(O.attention_f64(q1, k, v, 1, KV_LEN - 1, H, KV, D, SCALE), GOLD["decode_out"], rtol=1e-5, atol=1e-6)
    q4 = O.f16_bits_to_f32(GOLD["verify_q"])
    assert np.allclose(O.attention_f64(q4, k, v, 4, KV_LEN - 4, H, KV, D, SCALE), GOLD["verify_out"], rtol=1e-5, atol=1e-6)
    part = O.decode_partials_f32(GOLD["verify_q"], _src("k"), _src("v"), H, KV, D, KV_LEN, 5, SCALE, m_q=4)
    assert_close(O.reduce_f32(part, D, 5).reshape(4, H, D), GOLD["verify_out"], what="oracle split-K verify")
    k16, v16 = O.kv_materialize(_src("k", True), KV_LEN, KV, D), O.kv_materialize(_src("v", True), KV_LEN, KV, D)
    qp = O.f16_bits_to_f32(GOLD["prefill_q"])
    for window, key in ((0, "prefill_out"), (48, "prefill_window48_out")):
        got = O.attention_f64(qp, k16, v16, M, KV_LEN - M, H, KV, D, SCALE, window=window)
        assert np.allclose(got, GOLD[key], rtol=1e-5, atol=1e-6)
        fl = O.prefill_flash_f32(GOLD["prefill_q"], _src("k", True), _src("v", True), M, KV_LEN - M, H, KV, D, window, SCALE)
        assert_close(fl, GOLD[key], what=f"oracle flash order, window {window}")


# ---- GPU: the kernels reproduce the golden vectors ------------------------------------------------
@pytest.fixture(scope="module")
def ctx():
    import super_gemma_b200 as sg

    return sg.GpuContext(0)


@pytest.mark.gpu
def test_gpu_codec_matches_golden_bits(ctx):
    src = ctx.buffer_from_iter(GOLD["codec_x"])
    n = GOLD["codec_x"].size
    scales, quants, deq = ctx.new_buffer(n // 32, np.uint16), ctx.new_buffer(n, np.int8), ctx.new_buffer(n, np.uint16)
    k = ctx.load_kernel("kv_quant_q8")
    ctx.dispatch(k, bind(src, scales, quants), None, k.groups_for(n // 32))
    kd = ctx.load_kernel("kv_dequant_q8")
    ctx.dispatch_blocking(kd, bind(scales, quants, deq), None, kd.groups_for(n // 32))
    assert np.array_equal(scales.read(), GOLD["codec_scales"]) and np.array_equal(quants.read(), GOLD["codec_quants"])
    assert np.array_equal(deq.read(), GOLD["codec_deq16"])


def _pool_bufs(ctx):
    up = ctx.buffer_from_iter
    return [up(GOLD["k_quants"]), up(GOLD["k_scales"]), up(GOLD["v_quants"]), up(GOLD["v_scales"]), up(GOLD["page_table"])]


@pytest.mark.gpu
@pytest.mark.parametrize("m_q,qkey,okey", [(1, "decode_q", "decode_out"), (4, "verify_q", "verify_out")])
def test_gpu_paged_decode_matches_golden(ctx, m_q, qkey, okey):
    import super_gemma_b200 as sg

    n_splits = 4
    part, out = ctx.new_buffer(m_q * H * n_splits * (D + 2), np.float32), ctx.new_buffer(m_q * H * D, np.float32)
    step = ctx.new_step_buffer()
    sg.StepState(kv_len_global=KV_LEN).write_to(step)
    ctx.dispatch(ctx.load_kernel("attn_decode_paged_q8kv_d128"), bind(ctx.buffer_from_iter(GOLD[qkey]), *_pool_bufs(ctx), part, step),
                 (n_splits, SCALE, PAGE), [KV, n_splits, m_q])
    ctx.dispatch_blocking(ctx.load_kernel("attn_reduce_f32_d128"), bind(part, out), n_splits, [m_q * H, 1, 1])
    assert_close(out.read().reshape(m_q, H, D), GOLD[okey], what=f"paged decode m_q={m_q} vs golden")


@pytest.mark.gpu
def test_gpu_paged_flash_prefill_matches_golden(ctx):
    import super_gemma_b200 as sg

    q0 = KV_LEN - M
    rows = -(-KV_LEN // 64) * 64
    k_lin, v_lin = ctx.new_buffer(rows * KV * D, np.uint16), ctx.new_buffer(rows * KV * D, np.uint16)
    out = ctx.new_buffer(M * H * D, np.float32)
    step = ctx.new_step_buffer()
    sg.StepState(pos=q0, kv_len_global=KV_LEN, q0=q0).write_to(step)
    qb = ctx.buffer_from_iter(GOLD["prefill_q"])
    ctx.dispatch_blocking(ctx.load_kernel("attn_prefill_paged_q8kv_flash_d128"), bind(qb, *_pool_bufs(ctx), k_lin, v_lin, out, step),
                          (SCALE, PAGE), [KV, M, 1])
    assert_close(out.read().reshape(M, H, D), GOLD["prefill_out"], what="paged flash prefill vs golden")
    # the dequantised scratch is now a linear f16 cache: the windowed flash kernel runs on it directly
    out_w = ctx.new_buffer(M * H * D, np.float32)
    ctx.dispatch_blocking(ctx.load_kernel("attn_prefill_flash_f16_d128"), bind(qb, k_lin, v_lin, out_w, step), (SCALE, 48), [KV, M, 1])
    assert_close(out_w.read().reshape(M, H, D), GOLD["prefill_window48_out"], what="windowed flash prefill vs golden")
