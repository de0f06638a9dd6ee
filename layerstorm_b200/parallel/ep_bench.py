"""Expert-parallel microbenchmark: fused dispatch -> grouped GEMM -> combine vs the NCCL all-to-all +
grouped-GEMM baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m layerstorm_b200.parallel.ep_bench --tokens 1,8,64,512,4096,8192

Shape: hidden 7168, 256 routed experts, top-8, expert FFN 2048 SwiGLU, FP8 e4m3 weights with 128x128 block
scales; router logits N(0,1) + Zipf(1.1) per-expert bias; tokens per rank swept.  Each case: 3 warm-up
calls, then `--iters` timed calls bracketed by CUDA events on the launching stream; the reported time is the
maximum over ranks.  Rank 0 prints one JSON line per case with the roofline terms:
    compute  = pairs_on_the_busiest_rank * 3 * 2 * H * F / measured GEMM peak
    nvlink   = bytes that must cross the links of the busiest rank (fp16 rows in, fp32 rows out) / 770 GB/s
    hbm      = expert bytes the busiest rank must stream once / measured copy bandwidth
and ``roofline_fraction = max(compute, nvlink, hbm) / measured time``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..models.device_model import ExpertArena, QLinear, expert_layout
from .ep import EpMoE, zipf_router

NVLINK_GBS = 770.0           # measured peer copy, per direction per GPU


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,8,64,512,2048,8192")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--fmt", default="fp8_e4m3", choices=["fp8_e4m3", "nvfp4", "bf16"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip-nccl", action="store_true")
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    H, F, E, S = a.hidden, a.inter, a.experts, a.top_k
    hbm_gbs, tflops, tag = _peaks()
    ef = expert_layout(a.fmt, H, F)
    mine = [e for e in range(E) if e % world == rank]
    arena = ExpertArena(ef, len(mine), E, dev)
    g = torch.Generator(device=dev).manual_seed(rank)
    for s, e in enumerate(mine):                               # random expert bytes in storage format
        mats = [torch.randn(n, k, generator=g, device=dev) * 0.02 for n, k in ((F, H), (F, H), (H, F))]
        arena.write_expert(s, *(QLinear.from_float(m, a.fmt, dev) for m in mats))
        arena.slot_of[e] = s
    toks = [int(t) for t in a.tokens.split(",")]
    ep = EpMoE(H, F, E, S, max_tokens=max(toks), device=dev, arena=arena, capacity_factor=4.0)

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            fn()
        t1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([t0.elapsed_time(t1) / n], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    for T in toks:
        ids, wts = zipf_router(T, E, S, dev, seed=17 * rank + T)
        x = (torch.randn(T, H, device=dev) * 1.0).to(torch.bfloat16)
        out = torch.zeros(T, H, device=dev)
        fused_ms = timed(lambda: ep.forward(x, ids, wts, out), a.iters)
        rows_in = torch.tensor([ep.rows_received()], device=dev)
        # pairs that leave this rank / arrive from other ranks (NVLink bytes), and experts touched here (HBM bytes)
        owner = ids.reshape(-1).long() % world
        remote_out = int((owner != rank).sum())
        all_ids = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(all_ids, ids)
        cat = torch.cat([t.reshape(-1) for t in all_ids]).long()
        local_pairs = cat[cat % world == rank]
        touched = int(torch.unique(local_pairs).numel())
        remote_in = int(rows_in) - int((owner == rank).sum())
        stats = torch.tensor([int(rows_in), max(remote_out, remote_in), touched], device=dev, dtype=torch.float64)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        rows_max, link_pairs, touched_max = (float(v) for v in stats)
        t_compute = rows_max * 3 * 2 * H * F / (tflops * 1e12) * 1e3
        t_link = link_pairs * (H * 2 + H * 4) / (NVLINK_GBS * 1e9) * 1e3 if world > 1 else 0.0
        t_hbm = touched_max * ef.stride / (hbm_gbs * 1e9) * 1e3
        roof = max(t_compute, t_link, t_hbm)
        # two library baselines: fixed-capacity slabs (no host round trip; the fair comparison) and exact splits (one .tolist() per call)
        nccl_ms = None if (a.skip_nccl or world == 1) else timed(lambda: ep.forward_nccl(x, ids, wts, out), max(2, a.iters // 2))
        nccl_var_ms = None if (a.skip_nccl or world == 1) else timed(lambda: ep.forward_nccl_variable(x, ids, wts, out), max(2, a.iters // 2))
        err = torch.tensor([ep.error()], device=dev)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(json.dumps({"bench": "ep_fused_dispatch_gemm_combine", "n_gpus": world, "tokens_per_rank": T, "fmt": a.fmt, "hidden": H, "experts": E,
                              "top_k": S, "inter": F, "fused_ms": round(fused_ms, 4), "nccl_ms": None if nccl_ms is None else round(nccl_ms, 4),
                              "speedup_vs_nccl": None if nccl_ms is None else round(min(nccl_ms, nccl_var_ms) / fused_ms, 3),      # against the FASTER of the two baselines
                              "nccl_baseline": "fixed-capacity all_to_all_single, no host synchronisation",
                              "nccl_variable_splits_ms": None if nccl_var_ms is None else round(nccl_var_ms, 4),
                              "roofline_ms": {"compute": round(t_compute, 4), "nvlink": round(t_link, 4), "hbm": round(t_hbm, 4)},
                              "roofline_fraction": round(roof / fused_ms, 3), "roofline_basis": tag, "rows_on_busiest_rank": int(rows_max),
                              "experts_touched_on_busiest_rank": int(touched_max), "error_word": int(err)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
