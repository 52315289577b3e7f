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
