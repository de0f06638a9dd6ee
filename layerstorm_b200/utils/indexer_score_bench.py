"""Decode-side indexer scoring over long index rows: the three scoring kernels side by side.

    python -m layerstorm_b200.utils.indexer_score_bench [--entries 32768,131072,262144] [--rows 1] [--heads 32] [--iters 20]

One query row (``--rows``: a decode batch, every row its own sequence) scores every cached entry of its sequence in a paged FP8 index
cache (16 entries per page, scattered pages, random keys and scales):
  * ``cuda_core``    one thread per (row, entry), bf16 query, fp32 FMAs (``lsb_indexer_score``)
  * ``tensor_core``  the prefill path: keys gathered to a dense bf16 operand, one bf16 GEMM (``lsb_indexer_score_tc``; single sequence only)
  * ``fp8``          keys by TMA straight from the cache, query heads quantised to E4M3 in the CTA, ``tcgen05.mma kind::f8f6f4``
                     (``lsb_indexer_score_f8``)
CUDA events around ``--iters`` calls after 3 warm-up calls; one JSON line with microseconds per call and the largest difference of the
tensor-core results against the CUDA-core scores, relative to the largest score.  262144 entries is a 1M-token context pooled by 4.
"""
from __future__ import annotations

import argparse
import json


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--entries", default="32768,131072,262144")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args(argv)

    import torch

    from ..models.device_model import TcScratch
    from ..ops import _native as nat

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1)
    R, IH, page_e = a.rows, a.heads, 16
    out = {"rows": R, "heads": IH, "entries_per_page": page_e, "by_entries": {}}
    for ne_ in [int(x) for x in a.entries.split(",") if x.strip()]:
        per_seq = ne_ // page_e + 2
        n_pages = R * per_seq
        cache = torch.zeros(n_pages, page_e, 144, dtype=torch.uint8, device=dev)
        cache[:, :, :128] = torch.randint(0, 256, (n_pages, page_e, 128), device=dev, generator=g, dtype=torch.uint8) & 0x77
        cache[:, :, 128:132] = (torch.rand(n_pages, page_e, 1, device=dev, generator=g) * 0.05 + 0.01).view(torch.uint8)
        bt = torch.randperm(n_pages, device=dev, generator=g).int().view(R, per_seq).contiguous()
        q = torch.randn(R, IH, 128, device=dev, generator=g).to(torch.bfloat16)
        w = torch.randn(R, IH, device=dev, generator=g)
        row_seq = torch.arange(R, dtype=torch.int32, device=dev)
        ne = torch.full((R,), ne_, dtype=torch.int32, device=dev)
        ld = ne_ + 64
        res = {k: torch.zeros(R, ld, device=dev) for k in ("cuda_core", "tensor_core", "fp8")}
        kr = (ld + 127) // 128 * 128
        kbf, ksc = torch.zeros(kr, 128, dtype=torch.bfloat16, device=dev), torch.zeros(kr, device=dev)
        err = TcScratch.get(dev).err
        err.zero_()
        fns = {"cuda_core": lambda: nat.call("lsb_indexer_score", q, w, IH, cache, bt, per_seq, page_e, row_seq, ne, res["cuda_core"], ld, R, ld),
               "fp8": lambda: nat.call("lsb_indexer_score_f8", q, w, IH, cache, n_pages, bt, per_seq, page_e, row_seq, ne, res["fp8"], ld, R, ld, err)}
        if R == 1 and 256 % IH == 0:
            fns["tensor_core"] = lambda: nat.call("lsb_indexer_score_tc", q, w, IH, cache, bt, per_seq, page_e, row_seq, ne, res["tensor_core"], ld, R, kr,
                                                  kbf, kr, ksc, err)
        row = {}
        for k, fn in fns.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            row[k + "_us"] = round(e0.elapsed_time(e1) * 1e3 / a.iters, 1)
        ref = res["cuda_core"]
        for k in fns:
            if k != "cuda_core":
                row[k + "_max_diff_rel"] = round(float((res[k] - ref).abs().max() / ref.abs().max()), 6)
        row["cache_mb"] = round(R * ne_ * 144 / 1e6, 1)
        row["error_word"] = int(err.item())
        out["by_entries"][str(ne_)] = row
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
