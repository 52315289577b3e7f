"""CPU tests that pin the oracle: bit-level codecs, the reference's closed-form cases, replays of
the reference's seeded kernel-test cases (f32 shader-order form against the f64 form, at the
reference's own tolerance), and the properties that stand in where the reference has no code
(page table, cross-rank combine)."""
import numpy as np
import pytest

import npref
from oracle import sg_oracle as O

ATOL = 1e-2  # crates/sg-gpu/tests/parity_attn.rs:33-34
RTOL = 1e-2


def assert_close(got, want, atol=ATOL, rtol=RTOL, what=""):
    """|got - want| <= atol + rtol*|want| (tests/reference/mod.rs:137-153)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, what
    excess = np.abs(got - want) - rtol * np.abs(want)
    i = int(np.argmax(excess))
    assert excess.flat[i] <= atol, f"{what}: element {i}: got {got.flat[i]} want {want.flat[i]}"


# ---- f16 -------------------------------------------------------------------------------------
def test_f16_to_f32_all_patterns():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = O.f16_bits_to_f32(bits)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    L = O.lib()
    for b in [0, 1, 0x3FF, 0x400, 0x3C00, 0x7BFF, 0x7C00, 0x8001, 0xFBFF, 0x6480]:
        assert np.float32(L.sgo_h2f_fast(b)).view(np.uint32) == want[b].view(np.uint32)


def test_f32_to_f16_rtne_matches_numpy():
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32),
        (rng.standard_normal(50000) * 1e-6).astype(np.float32),  # subnormal range
        (rng.standard_normal(20000) * 3e4).astype(np.float32),  # near overflow
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0**-24, 2.0**-25, 2.0**-25 * 1.0001,
                  1.0 + 2.0**-11, 1.0 + 3 * 2.0**-11, np.inf, -np.inf], np.float32),
        np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)[:0x7C00],
    ])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = O.f32_to_f16_bits(x)
    assert np.array_equal(got, want)
    L = O.lib()
    for v in x[:2000]:
        assert np.float32(L.sgo_round_through_f16_fast(float(v))) == np.float16(v).astype(np.float32)


# ---- generator -------------------------------------------------------------------------------
def test_rng_matches_independent_restatement():
    for seed in (0xA77, 0xA79, 0xB2, 0):
        r = O.Rng(seed)
        assert np.array_equal(r.f32_vec(257), npref.xorshift64star(seed, 257))
    v = O.Rng(0xA77).f32_vec(100000)
    assert v.min() >= -2.0 and v.max() < 2.0 and abs(float(v.mean())) < 0.02


# ---- Q8_0 codec (crates/sg-gpu/tests/parity_kv.rs:131-209) ---------------------------------
def test_quant_q8_0_against_numpy_and_zero_block():
    x = O.through_f16(O.Rng(0xB2).f32_vec(4352))
    x[64:96] = 0.0  # an all-zero block: d = 0 -> id = 0 -> q = 0
    scales, quants = O.quant_q8_0(x)
    s2, q2 = npref.quant_q8_0(x)
    assert np.array_equal(scales, s2)
    assert np.array_equal(quants, q2)
    assert scales[2] == 0 and not quants[64:96].any()
    deq16 = O.dequant_q8_0_f16(scales, quants)
    want16 = npref.dequant_f32(scales, quants).astype(np.float16).view(np.uint16)
    assert np.array_equal(deq16, want16)
    assert np.array_equal(O.dequant_q8_0_f32(scales, quants), npref.dequant_f32(scales, quants))
    # half a step from rounding q, plus up to 127 * 2^-11 of a step from rounding the scale to f16
    d = np.repeat(scales.view(np.float16).astype(np.float32), 32)
    assert np.all(np.abs(O.dequant_q8_0_f32(scales, quants) - x) <= 0.57 * d + 1e-7)


def test_q8_quant_division_form_is_close_to_multiply_form():
    x = O.through_f16(O.Rng(0xA79).f32_vec(8192))
    s1, q1 = O.quant_q8_0(x)
    s2, q2, deq = O.q8_quant_div(x)
    assert np.max(np.abs(q1.astype(int) - q2.astype(int))) <= 1
    assert np.max(np.abs(s1.astype(int) - s2.astype(int))) <= 1
    assert np.array_equal(deq, npref.dequant_f32(s2, q2))


# ---- KV placement (crates/sg-gpu/tests/parity_kv.rs:36-128) ----------------------------------
def test_kv_append_ring_wrap_and_linear():
    row = 16 * 256
    src = O.f32_to_f16_bits(O.Rng(0xB0).f32_vec(5 * row))
    dst = np.full(1024 * row, 0x7E00, np.uint16)
    O.kv_append(src, dst, row, pos=1022, ring=1024)
    d = dst.reshape(1024, row)
    for t, slot in enumerate([1022, 1023, 0, 1, 2]):
        assert np.array_equal(d[slot], src.reshape(5, row)[t])
    untouched = np.ones(1024, bool)
    untouched[[1022, 1023, 0, 1, 2]] = False
    assert np.all(d[untouched] == 0x7E00)

    src3 = src[: 3 * row]
    lin = np.full(16 * row, 0x7E00, np.uint16)
    O.kv_append(src3, lin, row, pos=7, ring=0)
    assert np.array_equal(lin.reshape(16, row)[7:10].reshape(-1), src3)
    assert np.all(lin.reshape(16, row)[:7] == 0x7E00) and np.all(lin.reshape(16, row)[10:] == 0x7E00)


def test_kv_append_q8_linear_and_paged():
    row = 16 * 128
    n = 6
    src = O.f32_to_f16_bits(O.Rng(0xB3).f32_vec(n * row))
    want_s, want_q = O.quant_q8_0(O.f16_bits_to_f32(src))
    scales = np.zeros(600 * (row // 32), np.uint16)
    quants = np.zeros(600 * row, np.int8)
    O.kv_append_q8(src, scales, quants, row, pos=254)  # linear rows 254..259
    assert np.array_equal(scales.reshape(600, -1)[254:260].reshape(-1), want_s)
    assert np.array_equal(quants.reshape(600, row)[254:260].reshape(-1), want_q)
    table = np.array([1, 0], np.uint32)  # logical page 0 -> physical 1, 1 -> 0
    scales[:] = 0
    quants[:] = 0
    O.kv_append_q8(src, scales, quants, row, pos=254, page_table=table, page=256)
    rows = [256 + 254, 256 + 255, 0, 1, 2, 3]
    assert np.array_equal(quants.reshape(600, row)[rows].reshape(-1), want_q)
    assert np.array_equal(scales.reshape(600, -1)[rows].reshape(-1), want_s)


# ---- closed-form cases of crates/sg-model/src/reference.rs:572-596 --------------------------
def test_uniform_keys_give_mean_of_values():
    hd = 2
    ck = np.ones((3, 2, hd), np.float32)
    cv = np.arange(3 * 2 * hd, dtype=np.float32).reshape(3, 2, hd)
    q = np.ones((1, 4, hd), np.float32)
    out = O.attention_f64(q, ck, cv, 1, 2, 4, 2, hd, 1.0)
    assert abs(out[0, 0, 0] - 4.0) < 1e-6  # kv head 0, dim 0: 0, 4, 8
    assert abs(out[0, 2, 0] - 6.0) < 1e-6  # q heads 2, 3 read kv head 1: 2, 6, 10


def test_window_two_masks_old_keys():
    ck = np.ones((3, 1, 1), np.float32)
    cv = np.array([10.0, 20.0, 30.0], np.float32).reshape(3, 1, 1)
    q = np.ones((1, 1, 1), np.float32)
    out = O.attention_f64(q, ck, cv, 1, 2, 1, 1, 1, 1.0, window=2)
    assert abs(out[0, 0, 0] - 25.0) < 1e-6


# ---- f64 form against the independent numpy restatement ---------------------------------------
def test_attention_f64_matches_numpy():
    rng = np.random.default_rng(7)
    m, q0, n_q, n_kv, hd = 9, 37, 8, 4, 32
    q = rng.standard_normal((m, n_q, hd)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((q0 + m, n_kv, hd)).astype(np.float16).astype(np.float32)
    v = rng.standard_normal((q0 + m, n_kv, hd)).astype(np.float16).astype(np.float32)
    for window in (0, 16):
        got = O.attention_f64(q, k, v, m, q0, n_q, n_kv, hd, 0.17, window=window)
        want = npref.attention(q, k, v, q0, n_q, n_kv, window, 0.17)
        assert np.allclose(got, want, rtol=1e-6, atol=1e-7)
    sel = O.attention_f64(q, k, v, m, q0, n_q, n_kv, hd, 0.17, tokens=[8, 2], heads=[5, 0, 7])
    full = O.attention_f64(q, k, v, m, q0, n_q, n_kv, hd, 0.17)
    assert np.array_equal(sel, full[[8, 2]][:, [5, 0, 7]])


# ---- replays of the reference's seeded decode cases ------------------------------------------
N_Q = 32


def _decode_case(rng, kv_len, n_splits, n_kv, hd, scale, quant_k):
    q = O.through_f16(rng.f32_vec(N_Q * hd))
    k = O.through_f16(rng.f32_vec(kv_len * n_kv * hd))
    v = O.through_f16(rng.f32_vec(kv_len * n_kv * hd))
    q16 = O.f32_to_f16_bits(q)
    if quant_k:
        ks_, kq_, k_deq = O.q8_quant_div(k)  # parity_attn.rs:1016 uses this helper
        ksrc = O.KvSrc(quants=kq_, scales=ks_)
        k_ref = k_deq
    else:
        ksrc = O.KvSrc(f16=O.f32_to_f16_bits(k))
        k_ref = k
    vsrc = O.KvSrc(f16=O.f32_to_f16_bits(v))
    part = O.decode_partials_f32(q16, ksrc, vsrc, N_Q, n_kv, hd, kv_len, n_splits, scale)
    got = O.f16_bits_to_f32(O.reduce_f32(part, hd, n_splits, f16_out=True))
    want = O.attention_f64(q.reshape(1, N_Q, hd), k_ref.reshape(kv_len, n_kv, hd), v.reshape(kv_len, n_kv, hd), 1,
                           kv_len - 1, N_Q, n_kv, hd, scale)[0]
    return part, got, want


def test_decode_sliding_cases():  # parity_attn.rs:61, seed 0xA77, head_dim 256, 16 kv heads
    rng = O.Rng(0xA77)
    for kv_len, n_splits in [(17, 1), (17, 4), (1024, 8)]:
        _, got, want = _decode_case(rng, kv_len, n_splits, 16, 256, 0.0625, False)
        assert_close(got, want, what=f"decode_sliding {kv_len}/{n_splits}")


def test_decode_global_q8k_cases_with_empty_splits():  # parity_attn.rs:1002, seed 0xA79, head_dim 512, 4 kv heads
    rng = O.Rng(0xA79)
    for kv_len, n_splits in [(333, 1), (333, 5), (3, 8), (1500, 4)]:
        part, got, want = _decode_case(rng, kv_len, n_splits, 4, 512, 0.044194174, True)
        assert_close(got, want, what=f"decode_global_q8k {kv_len}/{n_splits}")
        if kv_len == 3:  # splits 3..7 are empty: m stays at the sentinel, l = 0
            assert np.all(part[:, 3:, 512] == np.float32(-3.0e38)) and np.all(part[:, 3:, 513] == 0)


# ---- sliding prefill: ring + chunk (parity_attn.rs:342) ----------------------------------------
@pytest.mark.parametrize("q0", [0, 100, 1000, 1531])
def test_prefill_sliding_ring_cases(q0):
    n_kv, hd, m, W, R = 16, 64, 16, 1024, 1024  # head_dim reduced to keep the CPU suite short
    rng = O.Rng(0xA7C + q0)
    row = n_kv * hd
    L = q0 + m
    q = O.through_f16(rng.f32_vec(m * N_Q * hd))
    k_all = O.through_f16(rng.f32_vec(L * row)).reshape(L, row)
    v_all = O.through_f16(rng.f32_vec(L * row)).reshape(L, row)
    k_ring = np.zeros((R, row), np.float32)
    v_ring = np.zeros((R, row), np.float32)
    for t in range(max(0, q0 - R), q0):
        k_ring[t % R] = k_all[t]
        v_ring[t % R] = v_all[t]
    b = O.f32_to_f16_bits
    got = O.prefill_stream_f32(b(q), O.KvSrc(f16=b(k_ring)), O.KvSrc(f16=b(v_ring)), O.KvSrc(f16=b(k_all[q0:])),
                               O.KvSrc(f16=b(v_all[q0:])), m, q0, N_Q, n_kv, hd, W, R, 0.125)
    want = O.attention_f64(q.reshape(m, N_Q, hd), k_all.reshape(L, n_kv, hd), v_all.reshape(L, n_kv, hd), m, q0, N_Q, n_kv,
                           hd, 0.125, window=W)
    assert_close(got, want, what=f"prefill_sliding_ring q0={q0}")
    # the linear twin (attn_prefill_sliding.wgsl) over the same keys gives the same bits
    lin = O.prefill_stream_f32(b(q), O.KvSrc(f16=b(k_all)), O.KvSrc(f16=b(v_all)), None, None, m, q0, N_Q, n_kv, hd, W, 0,
                               0.125)
    assert np.array_equal(lin, got)


# ---- flash order (parity_attn.rs:604 / flash_sp_q8) -------------------------------------------
@pytest.mark.parametrize("q0", [0, 200])
def test_prefill_flash_q8_matches_f64_on_dequantised_inputs(q0):
    n_kv, hd, m = 4, 128, 24
    rng = O.Rng(0xB7A + q0)
    L = q0 + m
    q = O.through_f16(rng.f32_vec(m * N_Q * hd))
    k = O.through_f16(rng.f32_vec(L * n_kv * hd))
    v = O.through_f16(rng.f32_vec(L * n_kv * hd))
    ks_, kq_ = O.quant_q8_0(k)
    vs_, vq_ = O.quant_q8_0(v)
    ksrc = O.KvSrc(quants=kq_, scales=ks_, round_f16=True)
    vsrc = O.KvSrc(quants=vq_, scales=vs_, round_f16=True)
    got = O.prefill_flash_f32(O.f32_to_f16_bits(q), ksrc, vsrc, m, q0, N_Q, n_kv, hd, 0, 0.0884)
    k_deq = O.kv_materialize(ksrc, L, n_kv, hd)
    v_deq = O.kv_materialize(vsrc, L, n_kv, hd)
    assert np.array_equal(k_deq.reshape(-1), O.f16_bits_to_f32(O.dequant_q8_0_f16(ks_, kq_)))
    want = O.attention_f64(q.reshape(m, N_Q, hd), k_deq, v_deq, m, q0, N_Q, n_kv, hd, 0.0884)
    assert_close(got, want, atol=2e-3, what=f"flash q0={q0}")


# ---- page table: paged == linear over gathered rows (no reference code exists) ---------------
def test_paged_equals_linear_bit_for_bit():
    n_kv, hd, page, kv_len, n_pages = 2, 128, 64, 300, 7
    rng = np.random.default_rng(5)
    table = rng.permutation(n_pages).astype(np.uint32)[:5]
    x = rng.standard_normal((2, n_pages * page, n_kv * hd)).astype(np.float16).astype(np.float32)
    pools = [O.quant_q8_0(x[i]) for i in range(2)]
    q16 = O.f32_to_f16_bits(rng.standard_normal(N_Q * hd))
    rows = np.array([table[t // page] * page + t % page for t in range(kv_len)])

    def src(i, paged):
        s, qn = pools[i]
        s, qn = s.reshape(n_pages * page, -1), qn.reshape(n_pages * page, -1)
        if paged:
            return O.KvSrc(quants=qn, scales=s, page_table=table, page=page)
        return O.KvSrc(quants=np.ascontiguousarray(qn[rows]), scales=np.ascontiguousarray(s[rows]))

    a = O.decode_partials_f32(q16, src(0, True), src(1, True), N_Q, n_kv, hd, kv_len, 5, 0.0884)
    b = O.decode_partials_f32(q16, src(0, False), src(1, False), N_Q, n_kv, hd, kv_len, 5, 0.0884)
    assert np.array_equal(a, b)


# ---- multi-query decode and the cross-rank (m, l, O) combine ---------------------------------
def test_multi_query_decode_and_two_level_combine():
    n_kv, hd, kv_len, m_q = 4, 128, 700, 4
    rng = np.random.default_rng(11)
    q = rng.standard_normal((m_q, N_Q, hd)).astype(np.float16)
    k = rng.standard_normal((kv_len, n_kv, hd)).astype(np.float16)
    v = rng.standard_normal((kv_len, n_kv, hd)).astype(np.float16)
    ksrc, vsrc = O.KvSrc(f16=k.view(np.uint16)), O.KvSrc(f16=v.view(np.uint16))
    part = O.decode_partials_f32(q.view(np.uint16), ksrc, vsrc, N_Q, n_kv, hd, kv_len, 6, 0.0884, m_q=m_q)
    got = O.reduce_f32(part, hd, 6).reshape(m_q, N_Q, hd)
    want = O.attention_f64(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), m_q, kv_len - m_q, N_Q, n_kv,
                           hd, 0.0884)
    assert_close(got, want, atol=2e-3, what="multi-query decode")
    # two ranks each merge their own 3 splits to (acc, m, l); merging those equals merging all 6
    p = part.reshape(m_q * N_Q, 6, hd + 2)
    r0 = O.reduce_f32(np.ascontiguousarray(p[:, :3]), hd, 3, out_mode=1)
    r1 = O.reduce_f32(np.ascontiguousarray(p[:, 3:]), hd, 3, out_mode=1)
    two = O.reduce_f32(np.ascontiguousarray(np.stack([r0, r1], axis=1)), hd, 2).reshape(m_q, N_Q, hd)
    assert np.allclose(two, got, rtol=2e-6, atol=1e-7)


# ---- pre-attention steps: known answers for the f64 restatement of reference/mod.rs:156-216 ---------------
def test_rmsnorm_known_answers():
    w = np.arange(1, 257, dtype=np.float32)
    assert np.allclose(O.rmsnorm_f64(np.full(256, 3.0, np.float32), w, 256), w, rtol=1e-6)  # a constant row normalises to 1
    assert np.allclose(O.rmsnorm_f64(np.full(256, -2.0, np.float32), w, 256, plus_one=True), -(1 + w), rtol=1e-6)
    x = np.zeros(512, np.float32)
    x[5] = 4.0  # mean square 16/512 -> inv = sqrt(32)
    assert np.isclose(O.rmsnorm_f64(x, np.ones(512, np.float32), 512)[5], 4.0 * np.sqrt(32.0), rtol=1e-4)  # up to the 1e-6 epsilon
    assert np.all(O.rmsnorm_f64(np.zeros(256, np.float32), w, 256) == 0)  # eps keeps the zero row finite


def test_rope_known_answers():
    f = O.inv_freqs(128, 1e6)
    assert f[0] == 1.0 and np.isclose(f[-1], 1e6 ** (-126 / 128))
    cs0 = O.cos_sin_table(f, 0, 1).reshape(-1, 2)
    assert np.all(cs0[:, 0] == 1) and np.all(cs0[:, 1] == 0)
    x = O.Rng(5).f32_vec(2 * 4 * 512)
    assert np.array_equal(O.rope_f64(x, 512, 128, 4, O.cos_sin_table(f, 0, 2))[:4 * 512], x[:4 * 512])  # position 0 is the identity
    y = O.rope_f64(x, 512, 128, 4, O.cos_sin_table(f, 1000, 2)).reshape(-1, 512)
    xx = x.reshape(-1, 512)
    assert np.allclose((y ** 2).sum(1), (xx ** 2).sum(1), rtol=1e-5)  # a rotation keeps the norm
    assert np.array_equal(y[:, 64:256], xx[:, 64:256]) and np.array_equal(y[:, 320:], xx[:, 320:])  # frozen pairs
    # quarter turn on pair 0 (inv_freq 1): pos = pi/2 is not an integer, so build the table by hand
    cs = np.zeros((1, 64, 2), np.float32)
    cs[:, :, 0] = 1.0
    cs[0, 0] = (0.0, 1.0)
    r = O.rope_f64(np.arange(512, dtype=np.float32), 512, 128, 1, cs.reshape(-1))
    assert r[0] == -256.0 and r[256] == 0.0 and r[1] == 1.0
