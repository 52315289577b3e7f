"""Generates tests/golden/attn_golden.npz with the independent numpy restatement (tests/npref.py).

The reference keeps no stored vectors for its attention path (its tests are seeded generators
compared with an f64 oracle, crates/sg-gpu/tests/parity_attn.rs), and it cannot be run on this
project's machines, so these vectors come from a second, numpy-only statement of the same math
that shares no code with oracle/.  Both the C oracle (CPU tests) and the CUDA kernels (GPU tests)
are checked against them.  Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import npref  # noqa: E402

H, KV, D, PAGE, SCALE = 4, 2, 128, 32, 0.08838834764831845


def main():
    rng = np.random.default_rng(0x601D)
    out = {}
    # Q8_0 codec
    x = rng.standard_normal(512, dtype=np.float32).astype(np.float16)
    x[96:128] = 0
    s, q = npref.quant_q8_0(x.astype(np.float32))
    out.update(codec_x=x.view(np.uint16), codec_scales=s, codec_quants=q,
               codec_deq16=npref.dequant_f32(s, q).astype(np.float16).view(np.uint16))
    # paged Q8_0 decode / verify / prefill over one cache
    kv_len, n_pages = 150, 5
    table = rng.permutation(n_pages + 1).astype(np.uint32)[:n_pages]
    pools = {}
    for name in ("k", "v"):
        vals = rng.standard_normal((kv_len, KV * D), dtype=np.float32).astype(np.float16)
        sc, qu = npref.quant_q8_0(vals.astype(np.float32))
        sc, qu = sc.reshape(kv_len, KV * D // 32), qu.reshape(kv_len, KV * D)
        pq = rng.integers(-127, 128, size=((n_pages + 1) * PAGE, KV * D), dtype=np.int8)
        ps = (rng.random(((n_pages + 1) * PAGE, KV * D // 32), dtype=np.float32) * 0.05).astype(np.float16).view(np.uint16)
        t = np.arange(kv_len)
        rows = table[t // PAGE].astype(np.int64) * PAGE + t % PAGE
        pq[rows], ps[rows] = qu, sc
        pools[name] = (pq, ps, npref.dequant_f32(sc.reshape(-1), qu.reshape(-1)).reshape(kv_len, KV, D))
        out[f"{name}_quants"], out[f"{name}_scales"] = pq, ps
    out["page_table"] = table
    kd, vd = pools["k"][2], pools["v"][2]
    q1 = rng.standard_normal((1, H, D), dtype=np.float32).astype(np.float16)
    out["decode_q"] = q1.view(np.uint16)
    out["decode_out"] = npref.attention(q1.astype(np.float32), kd, vd, kv_len - 1, H, KV, 0, SCALE)
    q4 = rng.standard_normal((4, H, D), dtype=np.float32).astype(np.float16)
    out["verify_q"] = q4.view(np.uint16)
    out["verify_out"] = npref.attention(q4.astype(np.float32), kd, vd, kv_len - 4, H, KV, 0, SCALE)
    # prefill over the f16-rounded dequantised values (the flash path's contract)
    kd16, vd16 = kd.astype(np.float16).astype(np.float32), vd.astype(np.float16).astype(np.float32)
    m = 70
    qp = rng.standard_normal((m, H, D), dtype=np.float32).astype(np.float16)
    out["prefill_q"] = qp.view(np.uint16)
    out["prefill_out"] = npref.attention(qp.astype(np.float32), kd16, vd16, kv_len - m, H, KV, 0, SCALE)
    out["prefill_window48_out"] = npref.attention(qp.astype(np.float32), kd16, vd16, kv_len - m, H, KV, 48, SCALE)
    out["meta"] = np.array([H, KV, D, PAGE, kv_len, m], np.int64)
    np.savez_compressed(os.path.join(HERE, "attn_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "attn_golden.npz"))


if __name__ == "__main__":
    main()
