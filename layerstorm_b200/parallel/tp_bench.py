"""Tensor-parallel microbenchmark: row-parallel projection with the all-reduce fused into its epilogue vs the same
projection followed by an NCCL all-reduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m layerstorm_b200.parallel.tp_bench --rows 1,4,32,256,2048

One "layer step" = out-projection of this rank's heads (bf16 weights [hidden, K / N]) on R rows + cross-rank sum +
residual add + RMSNorm (the consumer of the sum), i.e. the o_proj -> next-norm edge of a decoder layer.
  fused    projection kernel stores its fp32 partial tile by tile into every peer's receive buffer over NVLink (GEMV
           epilogue for 1/2/4 rows, tcgen05 GEMM epilogue for >= 8 rows, push kernel otherwise); the add+RMSNorm
           kernel waits for the peers' flags and sums the slots in rank order.  No collective library call.
  nccl     same projection kernel writing locally, ``dist.all_reduce``, same add+RMSNorm kernel.
Each case: 5 warm-up iterations, then ``--iters`` timed iterations between CUDA events on the launching stream; the
weights of 8 layers (larger than L2 together) are cycled so every iteration streams its matrix from HBM; the reported
time is the maximum over ranks.  Roofline per step = max(FLOPs / measured GEMM peak, weight bytes / measured copy
bandwidth, bytes this rank must send = R * hidden * 4 * (N - 1) / 770 GB/s per direction).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..models.device_model import QLinear
from ..ops import _native as nat
from .symm import PeerComm

NVLINK_GBS = 770.0


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="1,4,32,256,2048")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--v-head", type=int, default=128)
    ap.add_argument("--iters", type=int, default=40)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    H, K = a.hidden, a.heads * a.v_head // world
    hbm_gbs, tflops, tag = _peaks()
    rows = [int(r) for r in a.rows.split(",")]
    g = torch.Generator(device=dev).manual_seed(rank)
    layers = [QLinear.random(H, K, "bf16", dev, gen=g) for _ in range(8)]
    comm = PeerComm(max(rows) * H, dev)
    norm_w = torch.ones(H, device=dev)

    for R in rows:
        x = (torch.randn(R, K, device=dev, generator=g) * 0.1).to(torch.bfloat16)
        sub = torch.zeros(R, H, device=dev)
        resid = torch.zeros(R, H, device=dev)
        out = torch.zeros(R, H, dtype=torch.bfloat16, device=dev)

        def fused(i):
            layers[i % 8](sub, x, R, comm=comm.ptr)
            nat.call("lsb_add_rmsnorm", out, resid, sub, norm_w, R, H, 1e-6, comm.ptr)

        def nccl(i):
            layers[i % 8](sub, x, R)
            dist.all_reduce(sub)
            nat.call("lsb_add_rmsnorm", out, resid, sub, norm_w, R, H, 1e-6, None)

        res = {}
        for name, fn in (("fused", fused), ("nccl", nccl)):
            if world == 1 and name == "fused":
                continue
            for i in range(5):
                fn(i)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(a.iters):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            res[name] = float(ms)
        # the two paths must agree (same partials, same summation order is not guaranteed for NCCL: compare loosely)
        resid.zero_(); fused(0) if world > 1 else nccl(0); torch.cuda.synchronize(); ref_a = out.float().clone()
        resid.zero_(); nccl(0); torch.cuda.synchronize()
        diff = float((out.float() - ref_a).abs().max())
        t_flop = 2.0 * R * H * K / (tflops * 1e12) * 1e3
        t_hbm = H * K * 2 / (hbm_gbs * 1e9) * 1e3
        t_link = R * H * 4 * (world - 1) / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_flop, t_hbm, t_link)
        err = torch.tensor([comm.error()], device=dev)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        if rank == 0:
            f = res.get("fused")
            print(json.dumps({"bench": "tp_row_parallel_gemm_allreduce_rmsnorm", "n_gpus": world, "rows": R, "hidden": H, "k_per_rank": K,
                              "fused_us": None if f is None else round(f * 1e3, 2), "nccl_us": round(res["nccl"] * 1e3, 2),
                              "speedup_vs_nccl": None if f is None else round(res["nccl"] / f, 3),
                              "roofline_us": {"compute": round(t_flop * 1e3, 2), "hbm": round(t_hbm * 1e3, 2), "nvlink": round(t_link * 1e3, 2)},
                              "roofline_fraction": None if f is None else round(roof / f, 3), "roofline_basis": tag,
                              "max_abs_diff_fused_vs_nccl": diff, "error_word": int(err)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
