"""How the attention path is split over the GPUs of one box (host-side arithmetic only).

The reference is single-GPU; the two partitions below are the ones its own kernel grids already
imply (crates/sg-gpu/shaders/attn_decode_global_q8k.wgsl:47-54: the outer grid axis is the kv head,
the second axis a contiguous range of the KV sequence).

* prefill: kv heads are dealt out in contiguous groups; a rank holds its heads' K/V pages and its
  slice of Q, writes its slice of the output, and exchanges nothing.
* decode: the KV sequence is cut into contiguous page ranges; a rank runs split-K over its range,
  merges its own splits to one (acc, m, l) per query row, the ranks all-gather those 130-float rows
  and every rank merges them in RANK ORDER, so all ranks hold the same bits.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

NEG_SENTINEL = np.float32(-3.0e38)


@dataclass(frozen=True)
class HeadShard:
    kv_heads: range  # global kv head indices owned by the rank
    q_heads: range   # the query heads that read them (GQA: contiguous blocks of q_per_kv)


def head_shard(rank: int, world: int, n_kv_heads: int, q_per_kv: int) -> HeadShard:
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    if n_kv_heads % world:
        raise ValueError(f"{n_kv_heads} kv heads do not divide over {world} ranks")
    per = n_kv_heads // world
    kv = range(rank * per, (rank + 1) * per)
    return HeadShard(kv, range(kv.start * q_per_kv, kv.stop * q_per_kv))


@dataclass(frozen=True)
class SeqShard:
    tokens: range  # logical tokens owned by the rank
    pages: range   # logical pages that hold them


def seq_shard(rank: int, world: int, kv_len: int, page: int) -> SeqShard:
    """Contiguous page ranges, as even as whole pages allow; trailing ranks may own nothing."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    n_pages = -(-kv_len // page)
    per = -(-n_pages // world)
    p0, p1 = min(rank * per, n_pages), min((rank + 1) * per, n_pages)
    return SeqShard(range(min(p0 * page, kv_len), min(p1 * page, kv_len)), range(p0, p1))


def local_page_table(table: np.ndarray, shard: SeqShard) -> np.ndarray:
    """The slice of the global page table a rank needs; its pool holds only those pages, renumbered
    in order of first use so that local pool page i is global physical page `order[i]`."""
    mine = np.asarray(table[shard.pages.start:shard.pages.stop], dtype=np.uint32)
    order = {p: i for i, p in enumerate(dict.fromkeys(mine.tolist()))}
    return np.array([order[p] for p in mine.tolist()], dtype=np.uint32)


def combine_ranks(gathered: np.ndarray) -> np.ndarray:
    """Host statement of attn_combine_ranks_d128: gathered [world, rows, hd + 2] = (acc, m, l) per
    rank; returns [rows, hd] = merged acc / l, ranks taken in ascending order."""
    g = np.asarray(gathered, np.float32)
    hd = g.shape[2] - 2
    m_all = g[:, :, hd].max(axis=0)
    w = np.exp(g[:, :, hd] - m_all[None, :]).astype(np.float32)
    acc = np.zeros((g.shape[1], hd), np.float32)
    l = np.zeros(g.shape[1], np.float32)
    for r in range(g.shape[0]):
        acc += w[r][:, None] * g[r, :, :hd]
        l += w[r] * g[r, :, hd + 1]
    return acc / l[:, None]


# ---- the fused combine + exchange of sequence-parallel decode (attn_reduce_exchange_d128) ------------------
def exchange_words(world: int, rows: int, hd: int = 128) -> int:
    """4-byte words of one rank's exchange buffer: lines u32[2][world][rows][(hd + 2) / 2][4] (every 16-byte line is
    {value, epoch, value, epoch}), then epoch u32[rows]."""
    return 2 * world * rows * ((hd + 2) // 2) * 4 + rows


def alloc_exchange(dist, device, world: int, rank: int, rows: int):
    """Allocate the zeroed exchange buffer of this rank so that every rank of `dist`'s world can store into it,
    and return (buffer tensor, int64 tensor of all ranks' buffer addresses as seen from this GPU, keep-alive).
    Peer mappings come from torch's symmetric memory when the platform offers it, else from CUDA IPC
    handles.  Plain peer mappings only."""
    import os

    import torch

    words = exchange_words(world, rows)
    keep = []
    try:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        buf = symm_mem.empty(words, dtype=torch.float32, device=device)
        hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        keep.append(hdl)
        how = "symmetric memory"
    except Exception:
        buf = torch.zeros(words, dtype=torch.float32, device=device)
        handle = buf.untyped_storage()._share_cuda_()
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        ptrs = []
        for r, h in enumerate(handles):
            if r == rank:
                ptrs.append(buf.data_ptr())
                continue
            storage = torch.UntypedStorage._new_shared_cuda(*h)
            peer = torch.empty(0, dtype=torch.float32, device=device).set_(storage)
            keep.append(peer)
            ptrs.append(peer.data_ptr())
        how = "CUDA IPC"
    buf.zero_()
    torch.cuda.synchronize()
    dist.barrier()  # nobody stores into a buffer that its owner has not zeroed yet
    peers = torch.tensor(ptrs, dtype=torch.int64, device=device)
    return buf, peers, (keep, how)
