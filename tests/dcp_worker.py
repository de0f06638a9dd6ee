"""Multi-GPU worker (one process per GPU): context-parallel attention over a token-sharded KV cache vs the fp32
reference over the whole cache."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from layerstorm_b200.parallel.dcp import DcpAttention, local_index, local_length, owner_of


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    H, dl, dr, page, chunk = 16 * world, 128, 16, 16, 16
    D, Hh = dl + dr, 16
    n_seq, ctx, max_pages = 2, 150, 12
    g = torch.Generator().manual_seed(3)                                  # same data on every rank
    full = (torch.randn(n_seq, ctx, D, generator=g) * 0.5).to(torch.bfloat16)
    bt = torch.arange(n_seq * max_pages, dtype=torch.int32).view(n_seq, max_pages)
    cache = torch.zeros(n_seq * max_pages * page, D, dtype=torch.bfloat16)
    for s in range(n_seq):
        for t in range(ctx):
            if owner_of(t, chunk, world) == rank:
                li = local_index(t, chunk, world)
                cache[int(bt[s, li // page]) * page + li % page] = full[s, t]
    dcp = DcpAttention(H, dl, dr, max_rows=24, device=dev, chunk=chunk, n_splits=2)
    scale = D ** -0.5
    ok = True
    for R, sparse in ((3, False), (5, True), (20, False), (24, True), (3, False)):
        q = (torch.randn(R, H, D, generator=g) * 0.5).to(torch.bfloat16)
        row_seq = torch.tensor([i % n_seq for i in range(R)], dtype=torch.int32)
        row_len = torch.tensor([1 + (11 * i + 7) % ctx for i in range(R)], dtype=torch.int32)
        row_len_local = torch.tensor([local_length(int(n), chunk, world, rank) for n in row_len], dtype=torch.int32)
        sel_ld = 64
        sel_idx = torch.full((R, sel_ld), -1, dtype=torch.int32)
        sel_cnt = torch.zeros(R, dtype=torch.int32)
        if sparse:
            for i in range(R):
                n = int(row_len[i])
                pick = torch.randperm(n, generator=g)[: min(n, 4 + (5 * i) % 50)]
                sel_idx[i, : len(pick)] = pick.int()
                sel_cnt[i] = len(pick)
        out = torch.zeros(R, Hh, dl, dtype=torch.bfloat16, device=dev)
        dcp.forward(q[:, rank * Hh: (rank + 1) * Hh].contiguous().to(dev), cache.to(dev).view(torch.uint8), bt.to(dev), max_pages, row_seq.to(dev),
                    row_len_local.to(dev), out, page, 0, scale, sel_idx.to(dev) if sparse else None, sel_cnt.to(dev) if sparse else None)
        torch.cuda.synchronize()
        err = 0.0
        for i in range(R):
            pos = sel_idx[i, : int(sel_cnt[i])].long() if sparse else torch.arange(int(row_len[i]))
            k = full[int(row_seq[i])][pos].float()
            pr = torch.softmax(q[i].float() @ k.T * scale, -1)
            ref = (pr @ k[:, :dl])[rank * Hh: (rank + 1) * Hh]
            err = max(err, float((out[i].float().cpu() - ref).abs().max()))
        good = err < 2e-2 and dcp.error() == 0
        print(f"rank {rank} R={R} sparse={sparse} max_err={err:.4g} err_word={dcp.error()}", flush=True)
        ok = ok and good
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("DCP_OK" if int(flag[0]) == 1 else "DCP_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag[0]) == 1 else 1)


if __name__ == "__main__":
    main()
