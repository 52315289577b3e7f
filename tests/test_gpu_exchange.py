"""attn_reduce_exchange_d128: the split-K combine fused with the exchange between the ranks of a
sequence-parallel decode.  On one GPU the exchange is with itself and must reproduce attn_reduce_f32_d128 bit
for bit, step after step (alternating slots, epochs); with two or more GPUs a worker per rank checks the
kernel against reduce + NCCL all-gather + rank-ordered combine."""
import os
import subprocess
import sys

import numpy as np
import pytest

from cases import D, bind

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_exchange_equals_plain_reduce():
    import super_gemma_b200 as sg
    from super_gemma_b200 import sharding

    ctx = sg.GpuContext(0)
    rows, n_splits = 32, 9
    xbuf = ctx.new_buffer(sharding.exchange_words(1, rows), np.float32)  # zero-initialised
    peers = ctx.buffer_from_iter(np.array([xbuf.device_ptr], np.uint64))
    red, fused = ctx.load_kernel("attn_reduce_f32_d128"), ctx.load_kernel("attn_reduce_exchange_d128")
    rng = np.random.default_rng(9)
    for step in range(5):
        part = rng.standard_normal((rows, n_splits, D + 2)).astype(np.float32)
        part[:, :, D + 1] = np.abs(part[:, :, D + 1]) + 0.25
        part[:, 7:, D], part[:, 7:, D + 1], part[:, 7:, :D] = -3.0e38, 0.0, 0.0  # empty splits
        p = ctx.buffer_from_iter(part.reshape(-1))
        want, got = ctx.new_buffer(rows * D, np.float32), ctx.new_buffer(rows * D, np.float32)
        ctx.dispatch_blocking(red, bind(p, want), n_splits, [rows, 1, 1])
        ctx.dispatch_blocking(fused, bind(p, xbuf, peers, got), (n_splits, 1, 0, 0), [rows, 1, 1])
        assert np.array_equal(got.read().view(np.uint32), want.read().view(np.uint32)), f"step {step}"
    words = xbuf.read().view(np.uint32)
    assert np.all(words[-rows:] == 5)  # the per-row epoch counts the launches


def test_rejects_bad_arguments():
    import super_gemma_b200 as sg

    ctx = sg.GpuContext(0)
    k = ctx.load_kernel("attn_reduce_exchange_d128")
    small = ctx.new_buffer(64, np.float32)
    part = ctx.new_buffer(32 * 2 * (D + 2), np.float32)
    out = ctx.new_buffer(32 * D, np.float32)
    peers = ctx.new_buffer(1, np.uint64)
    with pytest.raises(sg.Validation):
        ctx.dispatch_blocking(k, bind(part, small, peers, out), (2, 1, 0, 0), [32, 1, 1])  # exchange buffer too small
    with pytest.raises(sg.Validation):
        ctx.dispatch_blocking(k, bind(part, small, peers, out), (2, 2, 2, 0), [32, 1, 1])  # rank outside the world


def test_two_ranks_match_the_nccl_path():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "exchange_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0 and "exchange worker: OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("world", [4, 8])
def test_many_ranks_on_one_gpu_the_last_rank_finds_every_row(world):
    """Slot addressing for 4 and 8 ranks without 4 or 8 GPUs: every rank's exchange buffer lives on this GPU and the
    ranks are launched one after the other.  A rank stores its rows into all buffers before it waits, so ranks
    0 .. world-2 give up after their (20 us) bounded wait -- the ranks after them have not run yet -- and report a
    timeout, and the last rank finds every row in place and must produce exactly what the NCCL form produces:
    attn_reduce_partial_d128 per rank, the partials laid out in rank order, attn_combine_ranks_d128.  Nothing here
    waits for a launch that is not running: every wait runs out by itself."""
    import super_gemma_b200 as sg
    from super_gemma_b200 import sharding

    ctx = sg.GpuContext(0)
    rows, n_splits = 32, 5
    bufs = [ctx.new_buffer(sharding.exchange_words(world, rows), np.float32) for _ in range(world)]
    peers = ctx.buffer_from_iter(np.array([b.device_ptr for b in bufs], np.uint64))
    rng = np.random.default_rng(40 + world)
    parts = []
    for r in range(world):
        part = rng.standard_normal((rows, n_splits, D + 2)).astype(np.float32)
        part[:, :, D] += 3.0 * r  # the ranks' maxima differ, so the order of the merge shows in the bits
        part[:, :, D + 1] = np.abs(part[:, :, D + 1]) + 0.25
        parts.append(ctx.buffer_from_iter(part.reshape(-1)))
    redp, comb, fused = (ctx.load_kernel(n) for n in ("attn_reduce_partial_d128", "attn_combine_ranks_d128", "attn_reduce_exchange_d128"))
    gathered = ctx.new_buffer(world * rows * (D + 2), np.float32)
    one = ctx.new_buffer(rows * (D + 2), np.float32)
    for r in range(world):
        ctx.dispatch_blocking(redp, bind(parts[r], one), n_splits, [rows, 1, 1])
        gathered.write(one.read(), r * rows * (D + 2))
    want = ctx.new_buffer(rows * D, np.float32)
    ctx.dispatch_blocking(comb, bind(gathered, want), world, [rows, 1, 1])
    out = ctx.new_buffer(rows * D, np.float32)
    for r in range(world - 1):
        with pytest.raises(sg.Timeout):
            ctx.dispatch_blocking(fused, bind(parts[r], bufs[r], peers, out), (n_splits, world, r, 20), [rows, 1, 1])
    ctx.dispatch_blocking(fused, bind(parts[world - 1], bufs[world - 1], peers, out), (n_splits, world, world - 1, 0), [rows, 1, 1])
    assert np.array_equal(out.read().view(np.uint32), want.read().view(np.uint32))


def test_absent_peer_ends_in_a_timeout_status_not_a_hang():
    """The wait for a peer's row is bounded (the push block's wait_us, here 50 ms; about a second by default): with a second rank that never stores its row the kernel
    gives up, reports DEV_ERR_TIMEOUT through the status word, writes NaN (never stale data), and the context stays
    usable.  The absent peer is a second local buffer that nothing writes; no GPU is faulted or hung."""
    import super_gemma_b200 as sg
    from super_gemma_b200 import sharding

    ctx = sg.GpuContext(0)
    rows, n_splits = 4, 2
    mine = ctx.new_buffer(sharding.exchange_words(2, rows), np.float32)
    absent = ctx.new_buffer(sharding.exchange_words(2, rows), np.float32)
    peers = ctx.buffer_from_iter(np.array([mine.device_ptr, absent.device_ptr], np.uint64))
    part = np.random.default_rng(3).standard_normal((rows, n_splits, D + 2)).astype(np.float32)
    part[:, :, D + 1] = 1.0
    out = ctx.new_buffer(rows * D, np.float32)
    fused = ctx.load_kernel("attn_reduce_exchange_d128")
    with pytest.raises(sg.Timeout):
        ctx.dispatch_blocking(fused, bind(ctx.buffer_from_iter(part.reshape(-1)), mine, peers, out), (n_splits, 2, 0, 50_000), [rows, 1, 1])
    assert np.all(np.isnan(out.read()))
    # the context is still good: the single-rank form runs right after
    solo = ctx.new_buffer(sharding.exchange_words(1, rows), np.float32)
    solo_peers = ctx.buffer_from_iter(np.array([solo.device_ptr], np.uint64))
    ctx.dispatch_blocking(fused, bind(ctx.buffer_from_iter(part.reshape(-1)), solo, solo_peers, out), (n_splits, 1, 0, 0), [rows, 1, 1])
    assert np.all(np.isfinite(out.read()))
