"""One rank of the multi-GPU test of the sequence-parallel decode exchange (launched by tests/test_gpu_exchange.py
through torch.distributed.run): attn_reduce_exchange_d128, on synthetic partials and behind the decode kernel on a
real paged Q8_0 shard per rank, must give, step after step, the bits of reduce + NCCL all-gather + rank-ordered
combine."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import super_gemma_b200 as sg  # noqa: E402
from super_gemma_b200 import sharding  # noqa: E402

D = 128


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    stream = torch.cuda.Stream(device)
    ctx = sg.GpuContext(local, stream=stream.cuda_stream)
    rows, n_splits, steps = 64, 5, 7
    xbuf, peers, keep = sharding.alloc_exchange(dist, device, world, rank, rows)
    wrap = lambda t: ctx.adopt(t.data_ptr(), t.numel() * t.element_size(), np.uint8, keep=t)
    B = lambda *bufs: [sg.BufferBinding.buffer(i, b) for i, b in enumerate(bufs)]
    mine = torch.zeros(rows * (D + 2), dtype=torch.float32, device=device)
    gathered = torch.zeros(world * rows * (D + 2), dtype=torch.float32, device=device)
    out_nccl = torch.zeros(rows * D, dtype=torch.float32, device=device)
    out_fused = torch.zeros(rows * D, dtype=torch.float32, device=device)
    redp, comb, fused = (ctx.load_kernel(n) for n in ("attn_reduce_partial_d128", "attn_combine_ranks_d128", "attn_reduce_exchange_d128"))
    ok = True
    for step in range(steps):
        g = torch.Generator(device=device)
        g.manual_seed(1000 * step + rank)
        part = torch.randn(rows, n_splits, D + 2, generator=g, device=device, dtype=torch.float32)
        part[:, :, D] = part[:, :, D] * 3.0 + 2.0 * rank          # m: different ranges per rank
        part[:, :, D + 1] = part[:, :, D + 1].abs() + 0.5          # l > 0
        if step == 3 and rank == 1:                                 # a rank whose range was empty for some rows
            part[:8, :, D] = -3.0e38
            part[:8, :, D + 1] = 0.0
            part[:8, :, :D] = 0.0
        part = part.contiguous()
        torch.cuda.synchronize()
        b_part = wrap(part)
        ctx.dispatch(redp, B(b_part, wrap(mine)), n_splits, [rows, 1, 1])
        ctx.sync()
        with torch.cuda.stream(stream):
            dist.all_gather_into_tensor(gathered, mine)
        stream.synchronize()
        ctx.dispatch_blocking(comb, B(wrap(gathered), wrap(out_nccl)), world, [rows, 1, 1])
        ctx.dispatch_blocking(fused, B(b_part, wrap(xbuf), wrap(peers), wrap(out_fused)), (n_splits, world, rank, 0), [rows, 1, 1])
        same = torch.equal(out_nccl.view(torch.int32), out_fused.view(torch.int32))
        finite = bool(torch.isfinite(out_fused).all())
        ok = ok and same and finite
        if not (same and finite):
            print(f"rank {rank} step {step}: fused != nccl path (max abs diff {(out_nccl - out_fused).abs().max().item()})", flush=True)
    # ---- the sequence-parallel decode step (decode kernel, then attn_reduce_exchange_d128) against decode + reduce +
    #      NCCL all-gather + combine, on a real paged Q8_0 shard per rank ------------------------------------------
    import bench

    dev = bench.Dev.__new__(bench.Dev)
    dev.torch, dev.sg, dev.device, dev.stream, dev.ctx, dev.k = torch, sg, device, stream, ctx, {}
    H, KV, PAGE, local_len, n_splits2 = bench.H, bench.KV, bench.PAGE, 2048 + 256 * rank, 9  # shards of different lengths
    for m_q in (1, 4):
        n_pages = local_len // PAGE
        kq, ks, vq, vs, tab = bench.build_paged_kv(dev, 77 + rank, local_len, list(range(KV)), bench.fisher_yates(5 + rank, n_pages), n_pages)
        q = bench.build_q(dev, 99, m_q, list(range(H)))
        rows2 = m_q * H
        part2 = torch.zeros(rows2 * n_splits2 * (D + 2), dtype=torch.float32, device=device)
        mine2 = torch.zeros(rows2 * (D + 2), dtype=torch.float32, device=device)
        gath2 = torch.zeros(world * rows2 * (D + 2), dtype=torch.float32, device=device)
        o_nccl, o_x = torch.zeros(rows2 * D, dtype=torch.float32, device=device), torch.zeros(rows2 * D, dtype=torch.float32, device=device)
        step_t = torch.tensor([0, 0, local_len, 0], dtype=torch.int32, device=device)
        xb2, peers2, keep2 = sharding.alloc_exchange(dist, device, world, rank, rows2)
        torch.cuda.synchronize()
        pools = [wrap(t) for t in (q, kq, ks, vq, vs, tab)]
        dec = ctx.load_kernel("attn_verify_paged_q8kv_d128")
        for it in range(3):
            ctx.dispatch(dec, B(*pools, wrap(part2), wrap(step_t)), (n_splits2, bench.SCALE, PAGE), [KV, n_splits2, m_q])
            ctx.dispatch(redp, B(wrap(part2), wrap(mine2)), n_splits2, [rows2, 1, 1])
            ctx.sync()
            with torch.cuda.stream(stream):
                dist.all_gather_into_tensor(gath2, mine2)
            stream.synchronize()
            ctx.dispatch_blocking(comb, B(wrap(gath2), wrap(o_nccl)), world, [rows2, 1, 1])
            ctx.dispatch(dec, B(*pools, wrap(part2), wrap(step_t)), (n_splits2, bench.SCALE, PAGE), [KV, n_splits2, m_q])
            ctx.dispatch_blocking(fused, B(wrap(part2), wrap(xb2), wrap(peers2), wrap(o_x)), (n_splits2, world, rank, 0), [rows2, 1, 1])
            same = torch.equal(o_nccl.view(torch.int32), o_x.view(torch.int32)) and bool(torch.isfinite(o_x).all())
            ok = ok and same
            if not same:
                print(f"rank {rank} m_q {m_q} it {it}: fused exchange != nccl path (max abs diff {(o_nccl - o_x).abs().max().item()})", flush=True)
            dist.barrier()

    flag = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"exchange worker: {'OK' if flag.item() == 1 else 'MISMATCH'} over {steps} steps, world {world}, peers by {keep[1]}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
