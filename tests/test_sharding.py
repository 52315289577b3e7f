"""CPU tests of the multi-GPU host logic: shard arithmetic, and a world_size-2 gloo run of the
sequence-split decode protocol (local split-K -> (acc, m, l) -> all-gather -> rank-ordered combine)
and of the kv-head-group prefill partition, with the oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest

from oracle import sg_oracle as O
from super_gemma_b200 import sharding as S

H, KV, D, PAGE, SCALE = 8, 4, 128, 64, 0.0884


def test_head_shards_cover_all_heads_once():
    for world in (1, 2, 4):
        kv, q = [], []
        for r in range(world):
            s = S.head_shard(r, world, 16, 2)
            kv += list(s.kv_heads)
            q += list(s.q_heads)
        assert kv == list(range(16)) and q == list(range(32))
    with pytest.raises(ValueError):
        S.head_shard(0, 3, 16, 2)


def test_seq_shards_are_contiguous_whole_pages():
    for kv_len, world in ((131072, 8), (1000, 4), (100, 8), (65540, 2)):
        toks = []
        for r in range(world):
            s = S.seq_shard(r, world, kv_len, 256)
            assert s.tokens.start % 256 == 0 or len(s.tokens) == 0
            toks += list(s.tokens)
        assert toks == list(range(kv_len))


def test_local_page_table_renumbers_in_first_use_order():
    table = np.array([7, 3, 9, 3, 1], np.uint32)
    sh = S.SeqShard(range(64, 256), range(1, 4))
    assert S.local_page_table(table, sh).tolist() == [0, 1, 0]


def _case():
    rng = np.random.default_rng(42)
    kv_len = 700
    q = rng.standard_normal((1, H, D), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((kv_len, KV, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((kv_len, KV, D), dtype=np.float32).astype(np.float16)
    return kv_len, q, k, v


def _rank_main(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    kv_len, q, k, v = _case()
    # ---- decode: sequence split ----
    sh = S.seq_shard(rank, world, kv_len, PAGE)
    n_local, n_splits = len(sh.tokens), 3
    ks = O.KvSrc(f16=np.ascontiguousarray(k[sh.tokens.start:sh.tokens.stop]).view(np.uint16))
    vs = O.KvSrc(f16=np.ascontiguousarray(v[sh.tokens.start:sh.tokens.stop]).view(np.uint16))
    part = O.decode_partials_f32(q.view(np.uint16), ks, vs, H, KV, D, n_local, n_splits, SCALE)
    mine = torch.from_numpy(O.reduce_f32(part, D, n_splits, out_mode=1))
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    out = S.combine_ranks(torch.stack(gathered).numpy())
    np.save(os.path.join(out_dir, f"decode_{rank}.npy"), out)
    # ---- prefill: kv-head groups, no exchange ----
    hs = S.head_shard(rank, world, KV, H // KV)
    m, q0 = 5, kv_len - 5
    qp = np.random.default_rng(7).standard_normal((m, H, D), dtype=np.float32).astype(np.float16)
    got = O.attention_f64(np.ascontiguousarray(qp[:, hs.q_heads.start:hs.q_heads.stop]).astype(np.float32),
                          np.ascontiguousarray(k[:, hs.kv_heads.start:hs.kv_heads.stop]).astype(np.float32),
                          np.ascontiguousarray(v[:, hs.kv_heads.start:hs.kv_heads.stop]).astype(np.float32), m, q0, len(hs.q_heads),
                          len(hs.kv_heads), D, SCALE)
    np.save(os.path.join(out_dir, f"prefill_{rank}.npy"), got)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_protocols_match_the_single_rank_oracle(tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    kv_len, q, k, v = _case()
    want = O.attention_f64(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), 1, kv_len - 1, H, KV, D, SCALE)[0]
    outs = [np.load(tmp_path / f"decode_{r}.npy") for r in range(world)]
    assert np.array_equal(outs[0], outs[1])  # rank-ordered combine: identical bits on every rank
    assert np.allclose(outs[0], want, rtol=1e-4, atol=1e-5)
    m, q0 = 5, kv_len - 5
    qp = np.random.default_rng(7).standard_normal((m, H, D), dtype=np.float32).astype(np.float16)
    full = O.attention_f64(qp.astype(np.float32), k.astype(np.float32), v.astype(np.float32), m, q0, H, KV, D, SCALE)
    got = np.concatenate([np.load(tmp_path / f"prefill_{r}.npy") for r in range(world)], axis=1)
    assert np.array_equal(got, full)


def _absent_rank_main(rank, world, port, out_dir):
    import datetime
    import time

    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    dist.barrier()  # both ranks are up
    if rank == 1:
        time.sleep(12)  # this rank never brings its partial: a stalled or lost process
        os._exit(0)
    mine = torch.zeros(4)
    t0 = time.time()
    outcome = "completed"
    try:
        dist.all_gather([torch.empty_like(mine) for _ in range(world)], mine)
    except Exception as e:  # the process-group timeout ends the collective with an error on the host
        outcome = "error: " + type(e).__name__
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(f"{outcome}\n{time.time() - t0:.1f}\n")
    os._exit(0)


def test_absent_rank_is_detected_on_the_host(tmp_path):
    """Failure detection without touching a GPU: a rank that never joins the exchange makes the other rank's
    collective end with an error after the process-group timeout, on the host, instead of waiting for ever."""
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_absent_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    outcome, seconds = (tmp_path / "outcome.txt").read_text().split()[0:1], (tmp_path / "outcome.txt").read_text().strip().split("\n")[-1]
    assert outcome[0].startswith("error"), outcome
    assert float(seconds) < 11.0


def test_exchange_buffer_layout():
    """Words of one rank's exchange buffer for attn_reduce_exchange_d128: two parities of world x rows merged rows
    of 65 lines {value, epoch, value, epoch}, and one epoch per row."""
    from super_gemma_b200 import sharding

    assert sharding.exchange_words(1, 32) == 2 * 32 * 65 * 4 + 32
    assert sharding.exchange_words(8, 128) == 2 * 8 * 128 * 65 * 4 + 128
