#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (CUDA, through the C ABI)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's math on the host cores

Headline workload (config 5a of the benchmark definition, the 128K-context case of the metric): a 4096-token query
chunk at q0 = 126976 attends causally to 131072 cached tokens held as Q8_0 in 256-token pages
behind a seeded random page table; 32 query / 16 kv heads, head_dim 128.  A step is one pass:
dequantise-and-gather K and V, then the tcgen05 flash kernel.  With N GPUs the kv heads are split
into N groups (strong scaling, no data-path collective).  The JSON line also carries the definition's
other configs under "extra": config 2 (8192 x 8192 prefill), config 3 (32K decode), config 4
(4-token verify at 64K), the recorded per-token decode block, and config 5b (128K decode, sequence-split
over the ranks; the combine and the exchange of the (acc, m, l) partials run as one kernel over peer
memory, with the reduce + NCCL all-gather + combine form timed beside it).

All inputs are synthetic: seeded N(0,1) rounded to f16, quantised on the device by this library's
own kv_append_paged_q8_d128 (bit-exact with the oracle's quantiser, see tests/test_gpu_kv.py).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, KV, D, G, PAGE = 32, 16, 128, 2, 256
SCALE = 1.0 / math.sqrt(D)
SEED = 0x5605


# dram__bytes_read.sum + dram__bytes_write.sum of one flash_prefill_kernel launch, from an ncu capture of this
# script (summarised under profiles/), keyed by (m, ctx, n_gpus).  Other shapes: not captured.
FLASH_DRAM_BYTES = {(4096, 131072, 1): 1358588672 + 123469312}


def peaks():
    """Measured denominators (driver-written MEASURED_PEAKS.json), else the pool's earlier measurement."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tf_burst": d["bf16_tflops"], "tf_sustained": d["bf16_tflops_sustained"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "kind": "fallback"}


def causal_pairs(m, q0):
    return m * q0 + m * (m + 1) // 2


# --------------------------------------------------------------------------------------------------
# clocks during the timed region
# --------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi polled every 20 ms while the headline workload runs.  The summary is taken over the samples that fall
    inside the device-timed window (host clock, see `timed`): the SM clock a kernel actually ran at differs from the
    clock of the idle or copy-bound phases around it by hundreds of MHz on a power-capped part."""

    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.path = device, None, None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.device)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, window=None):
        import datetime

        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        try:
            rows = [[c.strip() for c in r.split(",")] for r in open(self.path).read().strip().splitlines() if r.strip()]
            stamp = lambda r: datetime.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
            inside = [r for r in rows if window and window[0] - 0.01 <= stamp(r) <= window[1] + 0.01]
            use = inside if inside else rows
            out["sm_mhz"] = float(np.median([float(r[1]) for r in use]))
            out["sm_max_mhz"] = float(rows[0][2])
            out["power_w_max"] = max(float(r[3]) for r in use)
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            out["reasons"] = [n for i, n in enumerate(names) if any("Active" in r[5 + i] and "Not" not in r[5 + i] for r in use)]
            out["samples"] = len(use)
            out["window"] = "the device-timed steps" if inside else "the whole headline run (no sample fell inside the timed steps)"
            out["sm_mhz_whole_run"] = float(np.median([float(r[1]) for r in rows]))
            os.unlink(self.path)
        except Exception:
            pass
        return out


# --------------------------------------------------------------------------------------------------
# device-side workload construction
# --------------------------------------------------------------------------------------------------
class Dev:
    """One rank's device state: a context on a torch stream, and helpers to wrap torch tensors."""

    def __init__(self, local_rank):
        import torch

        import super_gemma_b200 as sg

        self.torch, self.sg = torch, sg
        torch.cuda.set_device(local_rank)
        self.device = torch.device("cuda", local_rank)
        self.stream = torch.cuda.Stream(self.device)
        self.ctx = sg.GpuContext(local_rank, stream=self.stream.cuda_stream)
        self.k = {}

    def kernel(self, name):
        if name not in self.k:
            self.k[name] = self.ctx.load_kernel(name)
        return self.k[name]

    def wrap(self, t):
        return self.ctx.adopt(t.data_ptr(), t.numel() * t.element_size(), np.uint8, keep=t)

    def randn_f16(self, seed, *shape):
        g = self.torch.Generator(device=self.device)
        g.manual_seed(seed)
        return self.torch.randn(*shape, generator=g, device=self.device, dtype=self.torch.float32).half()

    def bind(self, *bufs):
        return [self.sg.BufferBinding.buffer(i, b) for i, b in enumerate(bufs)]


def build_q(dev, seed, m, heads):
    """Q [m, len(heads), D]: each query head is seeded by its global index, so a rank that owns a
    slice of the heads holds exactly the rows the 1-GPU run holds."""
    t = dev.torch.empty(m, len(heads), D, dtype=dev.torch.float16, device=dev.device)
    for j, h in enumerate(heads):
        t[:, j] = dev.randn_f16(seed * 1000 + h, m, D)
    return t


def build_paged_kv(dev, seed, tokens, kv_heads, table, pool_pages):
    """K and V of `tokens` logical tokens for the given global kv heads, quantised to Q8_0 and
    scattered into paged pools through `table` by kv_append_paged_q8_d128."""
    torch = dev.torch
    n_kv = len(kv_heads)
    row = n_kv * D
    rows = pool_pages * PAGE
    table_t = torch.from_numpy(table.astype(np.int32)).to(dev.device)
    step = torch.zeros(4, dtype=torch.int32, device=dev.device)
    pools = []
    for which in range(2):
        quants = torch.zeros(rows * row, dtype=torch.int8, device=dev.device)
        scales = torch.zeros(rows * row // 32, dtype=torch.float16, device=dev.device)
        src = torch.empty(tokens, n_kv, D, dtype=torch.float16, device=dev.device)
        for j, h in enumerate(kv_heads):
            src[:, j] = dev.randn_f16(seed * 1000 + 100 * (which + 1) + h, tokens, D)
        torch.cuda.synchronize()
        k = dev.kernel("kv_append_paged_q8_d128")
        dev.ctx.dispatch_blocking(k, dev.bind(dev.wrap(src), dev.wrap(scales), dev.wrap(quants), dev.wrap(table_t), dev.wrap(step)),
                                  (row, PAGE), k.groups_for(tokens * row // 32))
        pools += [quants, scales]
        del src
    return pools[0], pools[1], pools[2], pools[3], table_t


def fisher_yates(seed, n):
    return np.random.default_rng(seed).permutation(n).astype(np.uint32)


def check_prefill_rows(dev, out, q, kq, ks, vq, vs, table, m, q0, ctx_len, local_kv, tokens):
    """After the timed region: sampled rows of the prefill output against the f64 oracle (test infrastructure,
    used here only as the checker).  For each of the given LOCAL kv heads the head's Q8_0 rows are brought to the
    host, put into logical order through the page table, dequantised to f16(scale * q) by the oracle's codec and
    attended to in f64.  Returns {"rows", "max_abs_err", "ok"}; tolerance 2e-3 + 1e-2 * |want|."""
    from oracle import sg_oracle as O

    torch = dev.torch
    n_kv = kq.numel() // (int(table.size) * PAGE * D)
    t = np.arange(ctx_len)
    phys = torch.from_numpy(table.astype(np.int64)[t // PAGE] * PAGE + t % PAGE).to(dev.device)
    worst, bad, rows = 0.0, 0, 0
    for j in local_kv:
        def head(quants, scales):
            qh = quants.view(-1, n_kv, D)[:, j][phys].contiguous().cpu().numpy()
            sh = scales.view(-1, n_kv, D // 32)[:, j][phys].contiguous().cpu().numpy().view(np.uint16)
            return O.f16_bits_to_f32(O.dequant_q8_0_f16(sh, qh)).reshape(ctx_len, 1, D)
        k32, v32 = head(kq, ks), head(vq, vs)
        q32 = q[:, j * G:(j + 1) * G].float().cpu().numpy()
        want = O.attention_f64(q32, k32, v32, m, q0, G, 1, D, SCALE, tokens=np.asarray(tokens, np.uint32))
        got = out[:, j * G:(j + 1) * G][torch.as_tensor(np.asarray(tokens, np.int64), device=dev.device)].cpu().numpy()
        err = np.abs(got.astype(np.float64) - want)
        worst = max(worst, float(err.max()))
        bad += int(np.sum((err > 2e-3 + 1e-2 * np.abs(want)) | ~np.isfinite(got)))
        rows += got.shape[0] * got.shape[1]
    return {"rows": rows, "max_abs_err": worst, "ok": bad == 0, "against": "f64 oracle on f16(scale*q) K/V, 2e-3 + 1e-2*|want|"}


def timed(dev, fn, steps, warmup, dist=None, stamps_per_step=1, graph=False):
    """W untimed steps, then K steps bracketed by barrier + synchronize; returns (max-over-ranks
    seconds for the K steps, per-step stamp deltas in ns as array [K, stamps_per_step], launches).
    graph=True records the K steps once and replays them as one CUDA graph, the way the reference
    drives its decode step (record_graph / submit_blocking): steps of a few tens of microseconds
    are otherwise bounded by the host's dispatch rate, not by the GPU.
    stamps_per_step = 0 puts no timestamp between the steps (one before the first, one after the last; the deltas
    are then None): an event record between two kernels of a few tens of microseconds costs microseconds of its
    own and keeps the second kernel from being scheduled behind the first."""
    torch = dev.torch
    for _ in range(warmup):
        fn(None, 0)
    dev.ctx.sync()
    ends_only = stamps_per_step == 0
    timer = dev.ctx.new_timer(2 if ends_only else steps * stamps_per_step + 1)

    def run_steps():
        if ends_only:
            timer.stamp(0)
            for i in range(steps):
                fn(None, i)
            timer.stamp(1)
        else:
            for i in range(steps):
                fn(timer, i * stamps_per_step)
            timer.stamp(steps * stamps_per_step)

    g = None
    if graph:
        g = dev.ctx.record_graph(lambda _ctx: run_steps())
        dev.ctx.submit_blocking(g)  # one untimed replay
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    before = dev.ctx.launch_count
    t_host0 = time.time()
    if g is not None:
        dev.ctx.submit(g)
    else:
        run_steps()
    dev.ctx.sync()
    torch.cuda.synchronize()
    dev.last_timed_window = (t_host0, time.time())
    launches = dev.ctx.launch_count - before
    ns = np.array(timer.read_ns(), dtype=np.float64)
    total_s = (ns[-1] - ns[0]) * 1e-9
    if dist is not None:
        t = torch.tensor([total_s], dtype=torch.float64, device=dev.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_s = float(t.item())
    return total_s, (None if ends_only else np.diff(ns).reshape(steps, stamps_per_step)), launches


# --------------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------------
def run_prefill(dev, rank, world, steps, warmup, dist, m, ctx_len, identity, seed, e2e=False, check=True):
    """Chunked prefill of m tokens at q0 = ctx_len - m over a ctx_len-token paged Q8_0 cache;
    kv heads split over the ranks.  Returns a dict of measurements."""
    torch = dev.torch
    q0 = ctx_len - m
    kvh = list(range(rank * KV // world, (rank + 1) * KV // world))
    qh = [h * G + g for h in kvh for g in range(G)]
    n_kv = len(kvh)
    n_pages = ctx_len // PAGE
    table = np.arange(n_pages, dtype=np.uint32) if identity else fisher_yates(seed + 0x100, n_pages)
    kq, ks, vq, vs, table_t = build_paged_kv(dev, seed, ctx_len, kvh, table, n_pages)
    q = build_q(dev, seed, m, qh)
    k_lin = torch.zeros(ctx_len * n_kv * D, dtype=torch.float16, device=dev.device)
    v_lin = torch.zeros_like(k_lin)
    out = torch.zeros(m, len(qh), D, dtype=torch.float32, device=dev.device)
    step_t = torch.tensor([q0, 0, ctx_len, q0], dtype=torch.int32, device=dev.device)
    torch.cuda.synchronize()
    W = dev.wrap
    b_q, b_kq, b_ks, b_vq, b_vs, b_tab, b_kl, b_vl, b_out, b_step = map(W, (q, kq, ks, vq, vs, table_t, k_lin, v_lin, out, step_t))
    deq, flash = dev.kernel("kv_dequant_paged_q8_d128"), dev.kernel("attn_prefill_flash_f16_d128")
    row = n_kv * D

    def step(timer, base):
        if timer is not None:
            timer.stamp(base)
        dev.ctx.dispatch(deq, dev.bind(b_ks, b_kq, b_tab, b_kl, b_step), (row, PAGE), [1, 1, 1])
        dev.ctx.dispatch(deq, dev.bind(b_vs, b_vq, b_tab, b_vl, b_step), (row, PAGE), [1, 1, 1])
        if timer is not None:
            timer.stamp(base + 1)
        dev.ctx.dispatch(flash, dev.bind(b_q, b_kl, b_vl, b_out, b_step), (SCALE, 0), [n_kv, m, 1])

    total_s, deltas, launches = timed(dev, step, steps, warmup, dist, stamps_per_step=2)
    timed_window = dev.last_timed_window
    flop_total = 4.0 * D * causal_pairs(m, q0) * H
    res = {"ms_per_step": total_s / steps * 1e3, "tflops": flop_total * steps / total_s / 1e12, "launches": launches,
           "flash_ms": float(np.mean(deltas[:, 1])) * 1e-6, "dequant_ms": float(np.mean(deltas[:, 0])) * 1e-6,
           "flop_per_rank": flop_total / world, "flop_total": flop_total, "timed_window": timed_window}
    if check and rank == 0:
        # run by the caller after the timed and clock-sampled region: it is CPU work
        tokens = sorted({0, 1, 63, 64, m // 2, m - 65, m - 64, m - 1} & set(range(m)))
        res["_check"] = lambda: check_prefill_rows(dev, out, q, kq, ks, vq, vs, table, m, q0, ctx_len, sorted({0, n_kv - 1}), tokens)

    if e2e:
        # The same pass through the C ABI with HOST buffers: pinned Q, K/V pools, page table and step words go up
        # every step, the f32 output comes back every step.  Uploads, compute and the read-back run on three
        # streams over two sets of device buffers, so step i + 1 is uploaded while step i computes (a server
        # streams the next chunk's inputs the same way); events order the reuse of each set.
        names = ("q", "kq", "ks", "vq", "vs", "tab")
        dev_sets = [dict(zip(names, (q, kq, ks, vq, vs, table_t)))]
        dev_sets.append({n: torch.empty_like(t) for n, t in dev_sets[0].items()})
        outs = [out, torch.empty_like(out)]
        host = {n: torch.empty(t.shape, dtype=t.dtype).pin_memory() for n, t in dev_sets[0].items()}
        for n, t in dev_sets[0].items():
            host[n].copy_(t)
        out_h = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
        up_stream, down_stream = torch.cuda.Stream(dev.device), torch.cuda.Stream(dev.device)
        up_ctx = dev.sg.GpuContext(dev.device.index, stream=up_stream.cuda_stream)
        down_ctx = dev.sg.GpuContext(dev.device.index, stream=down_stream.cuda_stream)
        adopt = lambda c, t: c.adopt(t.data_ptr(), t.numel() * t.element_size(), np.uint8, keep=t)
        up_bufs = [{n: adopt(up_ctx, t) for n, t in d.items()} for d in dev_sets]
        cmp_bufs = [{n: W(t) for n, t in d.items()} for d in dev_sets]
        cmp_out = [W(o) for o in outs]
        down_out = [adopt(down_ctx, o) for o in outs]
        L = dev.sg.lib()
        chk = dev.sg.gpu._check
        h2d = sum(t.numel() * t.element_size() for t in host.values()) + 16
        d2h = out.numel() * 4
        ev = lambda: [torch.cuda.Event() for _ in range(2)]
        uploaded, computed, downloaded = ev(), ev(), ev()

        def pipeline_step(i):
            s_ = i % 2
            if i >= 2:
                up_stream.wait_event(computed[s_])        # the set's previous contents have been consumed
            for n in names:
                t = host[n]
                chk(L.sgb_buffer_upload_async(up_bufs[s_][n]._h, 0, t.data_ptr(), t.numel() * t.element_size()))
            uploaded[s_].record(up_stream)
            dev.stream.wait_event(uploaded[s_])
            if i >= 2:
                dev.stream.wait_event(downloaded[s_])     # out[s_] has been read back
            c = cmp_bufs[s_]
            dev.sg.StepState(pos=q0, kv_len_global=ctx_len, q0=q0).write_to(b_step)
            dev.ctx.dispatch(deq, dev.bind(c["ks"], c["kq"], c["tab"], b_kl, b_step), (row, PAGE), [1, 1, 1])
            dev.ctx.dispatch(deq, dev.bind(c["vs"], c["vq"], c["tab"], b_vl, b_step), (row, PAGE), [1, 1, 1])
            dev.ctx.dispatch(flash, dev.bind(c["q"], b_kl, b_vl, cmp_out[s_], b_step), (SCALE, 0), [n_kv, m, 1])
            computed[s_].record(dev.stream)
            down_stream.wait_event(computed[s_])
            chk(L.sgb_buffer_download_async(down_out[s_]._h, 0, out_h[s_].data_ptr(), d2h))
            downloaded[s_].record(down_stream)

        e_steps = max(4, min(steps, 10))
        for i in range(2):
            pipeline_step(i)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(dev.stream)
        up_stream.wait_event(t0)                          # nothing of the timed steps starts before t0
        for i in range(e_steps):
            pipeline_step(i + 2)
        for e in downloaded:
            dev.stream.wait_event(e)                      # the last results are on the host before t1
        t1.record(dev.stream)
        torch.cuda.synchronize()
        total_e = t0.elapsed_time(t1) * 1e-3
        if dist is not None:
            tt = torch.tensor([total_e], dtype=torch.float64, device=dev.device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            total_e = float(tt.item())
        same = bool(torch.equal(out_h[0], out_h[1])) and bool(torch.equal(out_h[0].to(dev.device), outs[0]))
        res["e2e"] = {"value": flop_total * e_steps / total_e / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d * world),
                      "d2h_bytes_per_step": int(d2h * world), "ms_per_step": total_e / e_steps * 1e3, "steps": e_steps,
                      "pipelined": "uploads, compute and read-back on three streams over two buffer sets", "outputs_agree": same}
    return res


def prefill_output(dev, kvh, m, ctx_len, seed):
    """One untimed pass of the paged prefill over the given GLOBAL kv heads; returns the output tensor [m, 2*len(kvh), D]."""
    torch = dev.torch
    q0, n_kv, n_pages = ctx_len - m, len(kvh), ctx_len // PAGE
    kq, ks, vq, vs, table_t = build_paged_kv(dev, seed, ctx_len, kvh, fisher_yates(seed + 0x100, n_pages), n_pages)
    q = build_q(dev, seed, m, [h * G + g for h in kvh for g in range(G)])
    k_lin = torch.zeros(ctx_len * n_kv * D, dtype=torch.float16, device=dev.device)
    v_lin = torch.zeros_like(k_lin)
    out = torch.zeros(m, n_kv * G, D, dtype=torch.float32, device=dev.device)
    step_t = torch.tensor([q0, 0, ctx_len, q0], dtype=torch.int32, device=dev.device)
    torch.cuda.synchronize()
    W = dev.wrap
    dev.ctx.dispatch_blocking(dev.kernel("attn_prefill_paged_q8kv_flash_d128"),
                              dev.bind(*map(W, (q, kq, ks, vq, vs, table_t, k_lin, v_lin, out, step_t))), (SCALE, PAGE), [n_kv, m, 1])
    return out


def check_sharded_prefill(dev, rank, world, dist, m=512, ctx_len=8192, seed=0x5607):
    """Every rank computes its kv-head slice the way the sharded run does, and the same heads inside a launch over
    all 16 kv heads the way a 1-GPU run does; the two must agree within the parity tolerance (the launch geometry may
    cut the key range into a different number of pieces, each with its own running maximum, so P is rounded to f16 at
    different scales and the bits differ)."""
    torch = dev.torch
    mine = list(range(rank * KV // world, (rank + 1) * KV // world))
    a = prefill_output(dev, mine, m, ctx_len, seed)
    b = prefill_output(dev, list(range(KV)), m, ctx_len, seed)[:, mine[0] * G:(mine[-1] + 1) * G]
    diff = float((a - b).abs().max().item())
    within = bool(((a - b).abs() <= 2e-3 + 1e-2 * b.abs()).all()) and bool(torch.isfinite(a).all())
    ok = torch.tensor([1 if within else 0], device=dev.device)
    worst = torch.tensor([diff], dtype=torch.float64, device=dev.device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    return {"agrees": bool(ok.item() == 1), "max_abs_diff": float(worst.item()), "tolerance": "2e-3 + 1e-2*|x|",
            "shape": f"{m} queries over {ctx_len} tokens, every rank"}


def run_decode(dev, rank, world, steps, warmup, dist, ctx_len, m_q, n_splits, seed, copies=4):
    """Decode (m_q = 1) or verify (m_q = 4) over a ctx_len-token paged Q8_0 cache.  With world > 1
    the sequence is split into contiguous page ranges; each rank merges its own splits to
    (acc, m, l), the partials are all-gathered over NCCL and merged in rank order."""
    torch = dev.torch
    local_len = ctx_len // world
    n_pages = local_len // PAGE
    kvh = list(range(KV))
    # distinct pools per launch rotate through HBM so that a 143 MB stream is not served from L2
    pools = []
    for c in range(copies if local_len * KV * (D + 8) * 2 < 512e6 else 2):
        table = fisher_yates(seed + 0x100 + c, n_pages)
        pools.append(build_paged_kv(dev, seed + 17 * c + 31 * rank, local_len, kvh, table, n_pages))
    q = build_q(dev, seed, m_q, list(range(H)))
    rows = m_q * H
    part = torch.zeros(rows * n_splits * (D + 2), dtype=torch.float32, device=dev.device)
    out = torch.zeros(rows * D, dtype=torch.float32, device=dev.device)
    mine = torch.zeros(rows * (D + 2), dtype=torch.float32, device=dev.device)
    gathered = torch.zeros(world * rows * (D + 2), dtype=torch.float32, device=dev.device)
    step_t = torch.tensor([0, 0, local_len, 0], dtype=torch.int32, device=dev.device)
    torch.cuda.synchronize()
    W = dev.wrap
    b_q, b_part, b_out, b_mine, b_gath, b_step = map(W, (q, part, out, mine, gathered, step_t))
    b_pools = [tuple(W(t) for t in p) for p in pools]
    dec = dev.kernel("attn_decode_paged_q8kv_d128" if m_q == 1 else "attn_verify_paged_q8kv_d128")
    red, redp, comb = dev.kernel("attn_reduce_f32_d128"), dev.kernel("attn_reduce_partial_d128"), dev.kernel("attn_combine_ranks_d128")

    def make_step(mid_stamp, tail):
        def step(timer, base):
            kq, ks, vq, vs, tab = b_pools[base % len(b_pools)]
            if timer is not None:
                timer.stamp(base)
            dev.ctx.dispatch(dec, dev.bind(b_q, kq, ks, vq, vs, tab, b_part, b_step), (n_splits, SCALE, PAGE), [KV, n_splits, m_q])
            if timer is not None and mid_stamp:
                timer.stamp(base + 1)
            tail()
        return step

    def tail_local():
        dev.ctx.dispatch(red, dev.bind(b_part, b_out), n_splits, [rows, 1, 1])

    def tail_nccl():
        dev.ctx.dispatch(redp, dev.bind(b_part, b_mine), n_splits, [rows, 1, 1])
        with torch.cuda.stream(dev.stream):
            dist.all_gather_into_tensor(gathered, mine)
        dev.ctx.dispatch(comb, dev.bind(b_gath, b_out), world, [rows, 1, 1])

    tail0 = tail_local if world == 1 else tail_nccl
    kv_bytes = ctx_len * KV * (D + 8) * 2  # quants + scales, K and V
    algo = kv_bytes + m_q * H * D * 2 + m_q * H * D * 4 + (ctx_len // PAGE) * 4
    # the decode kernel alone (a stamp between the two kernels), then the whole step with nothing between its kernels
    _, deltas, _ = timed(dev, make_step(True, tail0), steps, warmup, dist, stamps_per_step=2, graph=(world == 1))
    total_s, _, launches = timed(dev, make_step(False, tail0), steps, warmup, dist, stamps_per_step=0, graph=(world == 1))
    kern_us = float(np.median(deltas[:, 0])) * 1e-3
    res = {"us_per_step": total_s / steps * 1e6, "gbs": algo * steps / total_s / 1e9, "kernel_us": kern_us,
           "kernel_gbs": (algo / world) / kern_us / 1e3, "algorithmic_bytes": algo, "n_splits": n_splits, "launches": launches,
           "step": "attn_decode_paged_q8kv_d128, then attn_reduce_f32_d128"}
    if world > 1:
        # The same step with the combine and the exchange in ONE kernel over peer memory (attn_reduce_exchange_d128)
        # instead of reduce + NCCL all-gather + combine; no collective call, so it replays as a CUDA graph.
        try:
            from super_gemma_b200 import sharding

            xbuf, peers, keep = sharding.alloc_exchange(dist, dev.device, world, rank, rows)
            b_x, b_peers = W(xbuf), W(peers)
            fx, fxt = dev.kernel("attn_reduce_exchange_d128"), dev.kernel("attn_reduce_exchange_timed_d128")

            def tail_fused():
                dev.ctx.dispatch(fx, dev.bind(b_part, b_x, b_peers, b_out), (n_splits, world, rank, 0), [rows, 1, 1])

            total_f, _, launches_f = timed(dev, make_step(False, tail_fused), steps, warmup, dist, stamps_per_step=0, graph=True)
            res.update({"nccl_us_per_step": res["us_per_step"], "nccl_gbs": res["gbs"], "us_per_step": total_f / steps * 1e6,
                        "gbs": algo * steps / total_f / 1e9, "launches": launches_f,
                        "step": f"attn_decode_paged_q8kv_d128, then attn_reduce_exchange_d128 (combine + exchange over NVLink peer stores, "
                                f"{keep[1]}); nccl_* = decode, reduce, NCCL all-gather, combine"})
            # Correctness of what was just timed: the same pool through both forms, compared bit for bit on every rank.
            outs = []
            for form in (make_step(False, tail_nccl), make_step(False, tail_fused)):
                out.zero_()
                form(None, 0)
                dev.ctx.sync()
                dist.barrier()
                outs.append(out.clone())
            same = bool(torch.equal(outs[0].view(torch.int32), outs[1].view(torch.int32))) and bool(torch.isfinite(outs[1]).all())
            flag = torch.tensor([1 if same else 0], device=dev.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            res["exchange_agrees"] = bool(flag.item() == 1)
            # Where the exchange kernel's time goes: global-timer stamps at its four phase boundaries, per row.
            stamps = torch.zeros(rows * 5, dtype=torch.int64, device=dev.device)
            b_st = W(stamps)
            phases = []
            tail_timed = lambda: dev.ctx.dispatch(fxt, dev.bind(b_part, b_x, b_peers, b_out, b_st), (n_splits, world, rank, 0), [rows, 1, 1])
            step_timed = make_step(False, tail_timed)
            # eight steps replayed as one graph keep the ranks in step with one another (through the exchange itself);
            # the stamps that survive a replay are those of its last step
            g8 = dev.ctx.record_graph(lambda _c: [step_timed(None, i) for i in range(8)])
            for i in range(12):
                dist.barrier()
                dev.ctx.submit_blocking(g8)
                if i >= 2:
                    phases.append(np.diff(stamps.cpu().numpy().reshape(rows, 5), axis=1))
            ph = np.stack(phases).astype(np.float64) * 1e-3  # [launch, row, phase] in us
            med = np.median(ph, axis=(0, 1))
            wait_max = torch.tensor([float(np.median(ph[:, :, 2].max(axis=1)))], dtype=torch.float64, device=dev.device)
            dist.all_reduce(wait_max, op=dist.ReduceOp.MAX)
            res["exchange_phases_us"] = {"local_merge": med[0], "peer_stores_and_flags": med[1], "wait": med[2], "rank_merge": med[3],
                                         "wait_max_over_rows_and_ranks": float(wait_max.item()),
                                         "note": "attn_reduce_exchange_timed_d128: rank 0's medians over rows and replays, last of eight graph-replayed steps"}
        except Exception as e:
            res["fused_exchange_error"] = repr(e)
    return res


def run_decode_block(dev, steps, warmup, ctx_len, n_splits, seed, chunk=4096):
    """The whole attention block of one decode token, recorded once and replayed: one launch for norm + RoPE
    of q and norm + RoPE + Q8_0 quantise + paged append of k and v, split-K decode over the ctx_len-token
    cache, combine.  Also times the fused append alone on a prefill chunk of `chunk` tokens."""
    torch = dev.torch
    n_pages = ctx_len // PAGE
    kq, ks, vq, vs, table = build_paged_kv(dev, seed, ctx_len, list(range(KV)), fisher_yates(seed + 0x100, n_pages), n_pages)
    g = torch.Generator(device=dev.device)
    g.manual_seed(seed)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=dev.device, dtype=torch.float32)
    q_raw, k_raw, v_raw = rnd(1, H, D).half(), rnd(chunk, KV, D).half(), rnd(chunk, KV, D).half()
    q_w, k_w = rnd(D) + 1.0, rnd(D) + 1.0
    pos = torch.arange(chunk, device=dev.device, dtype=torch.float64)[:, None] + float(ctx_len - 1)
    ang = pos * torch.pow(torch.tensor(1e6, dtype=torch.float64, device=dev.device),
                          -2.0 * torch.arange(D // 2, device=dev.device, dtype=torch.float64) / D)[None, :]
    cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous()  # host-filled in the reference; values only
    q = torch.zeros(H * D, dtype=torch.float16, device=dev.device)
    part = torch.zeros(H * n_splits * (D + 2), dtype=torch.float32, device=dev.device)
    out = torch.zeros(H * D, dtype=torch.float32, device=dev.device)
    step_t = torch.tensor([ctx_len - 1, 0, ctx_len, 0], dtype=torch.int32, device=dev.device)  # the token lands in the last row
    k1, v1 = k_raw[:1].contiguous(), v_raw[:1].contiguous()
    torch.cuda.synchronize()
    W = dev.wrap
    b = {n: W(t) for n, t in dict(q_raw=q_raw, k1=k1, v1=v1, q_w=q_w, k_w=k_w, cs=cos_sin, q=q, part=part, out=out, step=step_t, kq=kq, ks=ks,
                                  vq=vq, vs=vs, table=table).items()}
    qkv, fused = dev.kernel("qkv_norm_rope_append_paged_q8_d128"), dev.kernel("kv_norm_rope_append_paged_q8_d128")
    dec, red = dev.kernel("attn_decode_paged_q8kv_d128"), dev.kernel("attn_reduce_f32_d128")
    row = KV * D

    def step(timer, base):
        if timer is not None:
            timer.stamp(base)
        dev.ctx.dispatch(qkv, dev.bind(b["q_raw"], b["q_w"], b["q"], b["k1"], b["v1"], b["k_w"], b["cs"], b["ks"], b["kq"], b["vs"], b["vq"],
                                       b["table"], b["step"]), (H, row, PAGE, D, 0), [1, 1, 1])
        dev.ctx.dispatch(dec, dev.bind(b["q"], b["kq"], b["ks"], b["vq"], b["vs"], b["table"], b["part"], b["step"]), (n_splits, SCALE, PAGE),
                         [KV, n_splits, 1])
        dev.ctx.dispatch(red, dev.bind(b["part"], b["out"]), n_splits, [H, 1, 1])

    total_s, _, launches = timed(dev, step, steps, warmup, None, stamps_per_step=0, graph=True)
    res = {"us_per_token": total_s / steps * 1e6, "launches": launches, "kernels_per_token": 3, "ctx": ctx_len, "n_splits": n_splits,
           "note": "one cache copy: parts of the 143 MB stream may be served from the 126 MB L2"}
    # the fused append alone, on a prefill chunk written at positions 0..chunk-1
    step0 = torch.zeros(4, dtype=torch.int32, device=dev.device)
    b_k, b_v, b_s0 = W(k_raw), W(v_raw), W(step0)
    torch.cuda.synchronize()

    def step_app(timer, base):
        if timer is not None:
            timer.stamp(base)
        dev.ctx.dispatch(fused, dev.bind(b_k, b_v, b["k_w"], b["cs"], b["ks"], b["kq"], b["vs"], b["vq"], b["table"], b_s0), (row, PAGE, D, 0),
                         [1, 1, 1])

    total_s, _, _ = timed(dev, step_app, steps, warmup, None, stamps_per_step=0, graph=True)
    algo = chunk * KV * (2 * D * 2 + 2 * (D + 8))
    res["fused_append_chunk"] = {"tokens": chunk, "us": total_s / steps * 1e6, "algorithmic_bytes": algo,
                                 "gbs": algo * steps / total_s / 1e9, "note": "50 MB working set: L2-resident, not an HBM figure"}
    return res


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle's f32 shader-order flash prefill on a bounded sample of the headline workload
# --------------------------------------------------------------------------------------------------
def cpu_prefill_sample(m, ctx_len, target_s, seed=SEED):
    """Times oracle/sg_oracle.c:sgo_prefill_flash_f32 (OpenMP over (token, head)) on sampled query
    rows of the headline workload and returns TFLOP/s over the sampled rows."""
    from oracle import sg_oracle as O

    O.set_threads(len(os.sched_getaffinity(0)))  # all host cores this process may use, whatever OMP_NUM_THREADS says
    q0 = ctx_len - m
    rng = np.random.default_rng(seed)
    n_kv = KV
    # The CPU sample uses its own seeded N(0,1) data of the same shape and layout (quantised by the
    # oracle); throughput does not depend on the values.
    keys = ctx_len
    x = rng.standard_normal((2, keys, n_kv * D), dtype=np.float32).astype(np.float16).astype(np.float32)
    ks_, kq_ = O.quant_q8_0(x[0])
    vs_, vq_ = O.quant_q8_0(x[1])
    del x
    table = fisher_yates(seed + 0x100, keys // PAGE)
    # scatter rows through the table so the oracle walks the same indirection
    t = np.arange(keys)
    phys = table[t // PAGE].astype(np.int64) * PAGE + t % PAGE
    inv = np.empty(keys, np.int64)
    inv[phys] = t
    kq_p = np.ascontiguousarray(kq_.reshape(keys, -1)[inv])
    ks_p = np.ascontiguousarray(ks_.reshape(keys, -1)[inv])
    vq_p = np.ascontiguousarray(vq_.reshape(keys, -1)[inv])
    vs_p = np.ascontiguousarray(vs_.reshape(keys, -1)[inv])
    ksrc = O.KvSrc(quants=kq_p, scales=ks_p, page_table=table, page=PAGE, round_f16=True)
    vsrc = O.KvSrc(quants=vq_p, scales=vs_p, page_table=table, page=PAGE, round_f16=True)
    q16 = rng.standard_normal((m, H, D), dtype=np.float32).astype(np.float16)
    cores = O.num_threads()

    def run(tokens):
        t0 = time.perf_counter()
        O.prefill_flash_f32(q16.view(np.uint16), ksrc, vsrc, m, q0, H, n_kv, D, 0, SCALE, 64, tokens=tokens)
        dt = time.perf_counter() - t0
        pairs = sum(q0 + int(i) + 1 for i in tokens)
        return dt, 4.0 * D * pairs * H

    n0 = max(1, cores // H)
    dt, _ = run(np.arange(n0, dtype=np.uint32) * (m // max(n0, 1)))
    n = int(max(n0, min(m, n0 * target_s / max(dt, 1e-3))))
    tokens = np.linspace(0, m - 1, n).astype(np.uint32)
    dt, flop = run(tokens)
    return {"value": flop / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{n} of {m} query tokens x {H} heads of the headline workload ({dt:.1f} s of oracle/sg_oracle.c "
                      f"sgo_prefill_flash_f32, OpenMP)", "seconds": dt}, (lambda: run(tokens))


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m, ctx_len = args.m, args.ctx
    base, rerun = cpu_prefill_sample(m, ctx_len, target_s=max(2.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(max(0, args.warmup - 1)):
        rerun()
    t0 = time.perf_counter()
    flop = 0.0
    for _ in range(args.steps):
        _, f = rerun()
        flop += f
    dt = time.perf_counter() - t0
    v = flop / dt / 1e12
    base["value"] = v
    line = {"impl": "reference", "metric": "prefill_attn_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, max(1, args.gpus)), "cpu_baseline": base,  # the arm it is compared with
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def probe_mma(n_mma=4096):
    """diag_mma_cycles: every CTA issues n_mma back-to-back tcgen05.mma of one shape from one thread and reports the SM
    cycles until they have completed; one or two CTAs per SM.  One JSON line per (shape, CTAs per SM)."""
    import super_gemma_b200 as sg

    ctx = sg.GpuContext(0)
    k = ctx.load_kernel("diag_mma_cycles")
    sms = sg.lib().sgb_ctx_sm_count(ctx._h)
    names = ["SS M128xN64xK16", "SS M128xN128xK16", "TS M128xN128xK16", "8 x SS M128xN128xK16 then 8 x TS M128xN128xK16"]
    for per_sm in (1, 2):
        for shape, name in enumerate(names):
            buf = ctx.new_buffer(2 * sms * per_sm, np.uint64)
            for _ in range(3):
                ctx.dispatch_blocking(k, [sg.BufferBinding.buffer(0, buf)], (shape, n_mma), [per_sm, 1, 1])
            c = buf.read().reshape(-1, 2).astype(np.float64) / n_mma
            print(json.dumps({"shape": name, "ctas_per_sm": per_sm, "n_mma": n_mma, "cycles_per_mma_per_cta": float(np.median(c[:, 0])),
                              "cycles_per_mma_per_sm": float(np.median(c[:, 0])) / per_sm, "min": float(c[:, 0].min()), "max": float(c[:, 0].max()),
                              "issue_cycles_per_mma": float(np.median(c[:, 1]))}), flush=True)


def probe_mma_sustained(seconds=3.0, n_mma=1 << 20):
    """The same instruction streams run for `seconds` each with the clocks and the power sampled: what the tensor pipe
    alone sustains under the board's power limit, i.e. the ceiling of any kernel built from these instructions."""
    import super_gemma_b200 as sg

    ctx = sg.GpuContext(0)
    k = ctx.load_kernel("diag_mma_cycles")
    sms = sg.lib().sgb_ctx_sm_count(ctx._h)
    cases = [(0, 2, "SS M128xN64xK16", 2 * 128 * 64 * 16), (1, 2, "SS M128xN128xK16", 2 * 128 * 128 * 16),
             (2, 2, "TS M128xN128xK16", 2 * 128 * 128 * 16), (3, 2, "8 x SS N128 then 8 x TS N128", 2 * 128 * 128 * 16),
             (3, 1, "8 x SS N128 then 8 x TS N128", 2 * 128 * 128 * 16)]
    for data, (shape, per_sm, name, flop) in [(d, c) for d in (2, 1) for c in cases]:
        buf = ctx.new_buffer(2 * sms * per_sm, np.uint64)
        bind = [sg.BufferBinding.buffer(0, buf)]
        ctx.dispatch_blocking(k, bind, (shape, 4096), [per_sm, data, 1])
        with ClockSampler(0) as clocks:
            t0 = time.time()
            launches = 0
            while time.time() - t0 < seconds:
                ctx.dispatch_blocking(k, bind, (shape, n_mma), [per_sm, data, 1])
                launches += 1
            t1 = time.time()
        clk = clocks.summary((t0 + 0.5 * (t1 - t0), t1))  # the second half: the clocks have settled by then
        c = buf.read().reshape(-1, 2).astype(np.float64) / n_mma
        print(json.dumps({"shape": name, "operands": "seeded values in (-1, 1)" if data == 2 else "all 1.0", "ctas_per_sm": per_sm,
                          "seconds": t1 - t0, "launches": launches,
                          "tflops": launches * n_mma * flop * sms * per_sm / (t1 - t0) / 1e12,
                          "cycles_per_mma_per_sm": float(np.median(c[:, 0])) / per_sm, "clocks": clk}), flush=True)


def workload_config(args, world):
    return {"workload": f"BASELINE config 5a: chunked prefill, {args.m} queries at q0={args.ctx - args.m} over {args.ctx} cached "
                        f"Q8_0 tokens (256-token pages, seeded random page table), 32 q / 16 kv heads, head_dim 128, causal",
            "m": args.m, "ctx": args.ctx, "kv_heads_per_gpu": KV // world, "parallelism": f"kv-head groups x{world}",
            "l2": "K/V pools plus the f16 scratch written and re-read each step exceed the 126 MB L2; no flush"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--no-extra", action="store_true", help="headline workload only")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host buffers) leg")
    ap.add_argument("--decode-only", type=int, default=0, metavar="CTX",
                    help="run only the decode step over a CTX-token cache (decode kernel + combine, graph-replayed) and print its line; "
                         "for profiler launch lists")
    ap.add_argument("--probe-mma", action="store_true", help="print SM cycles per tcgen05.mma for the shapes the prefill kernels issue, and exit")
    ap.add_argument("--probe-mma-sustained", type=float, default=0.0, metavar="SECONDS",
                    help="run each tcgen05.mma stream for SECONDS with clocks and power sampled, print TFLOP/s, and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        reference_arm(args)
        return
    if args.probe_mma:
        probe_mma()
        return
    if args.probe_mma_sustained:
        probe_mma_sustained(args.probe_mma_sustained)
        return

    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    if world != args.gpus and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE={world}; launch N > 1 with torch.distributed.run", file=sys.stderr)
    if KV % world:
        raise SystemExit("the kv heads (16) must divide over the ranks")

    dev = Dev(local_rank)  # raises without the CUDA library or a B200: there is no fallback
    pk = peaks()
    if args.decode_only:
        d = run_decode(dev, rank, world, args.steps, args.warmup, dist, args.decode_only, 1,
                       dev.ctx.decode_splits_hint(KV, args.decode_only // world), 0x5603, copies=2)
        if rank == 0:
            d["hbm_frac_kernel"], d["hbm_frac_step"] = d["kernel_gbs"] / pk["hbm_gbs"], d["gbs"] / pk["hbm_gbs"] / world
            print(json.dumps({"decode_only": args.decode_only, **d}), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    with ClockSampler(local_rank) as clocks:
        head = run_prefill(dev, rank, world, args.steps, args.warmup, dist, args.m, args.ctx, False, SEED, e2e=not args.no_e2e)
    clk = clocks.summary(head.pop("timed_window", None))
    check = head.pop("_check", None)
    parity = check() if check else None
    del check
    torch.cuda.empty_cache()

    extra = {}
    if world > 1:
        try:
            extra["sharded_prefill_check"] = check_sharded_prefill(dev, rank, world, dist)
        except Exception as e:
            extra["sharded_prefill_check"] = {"error": repr(e)}
        torch.cuda.empty_cache()
    if not args.no_extra:
        try:
            if world == 1:
                c2 = run_prefill(dev, rank, world, max(3, args.steps), 3, dist, 8192, 8192, True, 0x5602)
                extra["config2_prefill_8192"] = {"tflops": c2["tflops"], "ms_per_step": c2["ms_per_step"], "flash_ms": c2["flash_ms"],
                                                 "frac_of_burst_peak": c2["flop_total"] / (c2["flash_ms"] * 1e-3) / 1e12 / pk["tf_burst"],
                                                 "parity_sample": c2.pop("_check")()}
                del c2
                torch.cuda.empty_cache()
                best = None
                # the library's hint (74 on 148 SMs: 16 kv heads x 74 splits x 2 warps fill every SM evenly) beside 32 / 64
                hint = dev.ctx.decode_splits_hint(KV, 32768)
                for ns in sorted({32, 64, hint}):
                    d3 = run_decode(dev, rank, world, 40, 5, dist, 32768, 1, ns, 0x5603)
                    if best is None or d3["us_per_step"] < best["us_per_step"]:
                        best = d3
                best["hbm_frac_kernel"], best["hbm_frac_step"] = best["kernel_gbs"] / pk["hbm_gbs"], best["gbs"] / pk["hbm_gbs"]
                extra["config3_decode_32k"] = best
                torch.cuda.empty_cache()
                d4 = run_decode(dev, rank, world, 40, 5, dist, 65536, 4, dev.ctx.decode_splits_hint(KV, 65536), 0x5604, copies=2)
                d4["hbm_frac_kernel"], d4["hbm_frac_step"] = d4["kernel_gbs"] / pk["hbm_gbs"], d4["gbs"] / pk["hbm_gbs"]
                extra["config4_verify_64k"] = d4
                torch.cuda.empty_cache()
                extra["decode_block_32k"] = run_decode_block(dev, 40, 5, 32768, dev.ctx.decode_splits_hint(KV, 32768), 0x5606)
                torch.cuda.empty_cache()
            d5 = run_decode(dev, rank, world, 40, 5, dist, 131072, 1, dev.ctx.decode_splits_hint(KV, 131072 // world), 0x5605, copies=2)
            d5["hbm_frac_kernel"] = d5["kernel_gbs"] / pk["hbm_gbs"]
            if "gbs" in d5:
                d5["hbm_frac_step"] = d5["gbs"] / pk["hbm_gbs"] / world
            extra["config5b_decode_128k"] = d5
        except Exception as e:  # the headline line must still be printed
            extra["error"] = repr(e)

    if rank == 0:
        cpu = None
        if not args.no_cpu and world == 1:
            try:
                cpu, _ = cpu_prefill_sample(args.m, args.ctx, target_s=15.0)
            except Exception as e:
                cpu = {"error": repr(e)}
        flash_s = head["flash_ms"] * 1e-3
        achieved = head["flop_per_rank"] / flash_s / 1e12
        long_run = head["ms_per_step"] * args.steps > 1000.0
        peak = pk["tf_sustained"] if long_run else pk["tf_burst"]
        line = {
            "metric": "prefill_attn_tflops", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 x f16 -> f32 (Q8_0 K/V dequantised to f16)", "data": "synthetic",
            "config": workload_config(args, world),
            "roofline": {"bound": "tensor", "kernel": "flash_prefill_kernel (attn_prefill_flash_f16_d128)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_kind": f"{pk['kind']} bf16 {'sustained' if long_run else 'burst'}",
                         "traffic": FLASH_DRAM_BYTES.get((args.m, args.ctx, world)),
                         "ms_per_launch": head["flash_ms"], "dequant_ms_per_step": head["dequant_ms"]},
            "parity_sample": parity, "cpu_baseline": cpu, "e2e": head.get("e2e"), "gpu_launches": int(head["launches"]), "clocks": clk, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
