"""Top-k selection over long index rows: one block per row against the selection spread over many blocks.

    python -m layerstorm_b200.utils.indexer_topk_bench [--entries 8192,32768,262144] [--rows 1] [--budget 512] [--pool 4]

Random scores (``--relu``: most of them exactly zero, as after the indexer's ReLU), CUDA events around 20 calls after 3 warm-up calls,
one JSON line: microseconds per call of ``lsb_indexer_topk`` and of ``lsb_indexer_topk_split`` for every row length, and whether the
two selections are identical.  262144 entries is a 1M-token context pooled by 4.
"""
from __future__ import annotations

import argparse
import json


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--entries", default="8192,32768,131072,262144")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--budget", type=int, default=512)
    ap.add_argument("--pool", type=int, default=4)
    ap.add_argument("--relu", action="store_true")
    a = ap.parse_args(argv)

    import torch

    from ..ops import _native as nat

    dev = torch.device("cuda", 0)
    R, P, B = a.rows, a.pool, a.budget
    rows = []
    for ne_ in [int(x) for x in a.entries.split(",") if x.strip()]:
        ld = ne_ + 8
        sc = torch.randn(R, ld, device=dev, generator=torch.Generator(device=dev).manual_seed(ne_))
        if a.relu:
            sc = (sc - 2.2).clamp_min(0)
        ne = torch.full((R,), ne_, dtype=torch.int32, device=dev)
        row_len = (ne * P).int()
        row_seq = torch.arange(R, dtype=torch.int32, device=dev)
        sel_ld = B * P + P
        out = [torch.zeros(R, sel_ld, dtype=torch.int32, device=dev) for _ in range(2)]
        cnt = [torch.zeros(R, dtype=torch.int32, device=dev) for _ in range(2)]
        scratch = torch.zeros((int(nat.call("lsb_indexer_topk_split_scratch", R, ld)) + 3) // 4, dtype=torch.int32, device=dev)
        calls = [lambda: nat.call("lsb_indexer_topk", sc, ld, ne, row_len, row_seq, B, P, out[0], cnt[0], sel_ld, R),
                 lambda: nat.call("lsb_indexer_topk_split", sc, ld, ne, row_len, row_seq, B, P, out[1], cnt[1], sel_ld, R, ld, scratch)]
        us = []
        for fn in calls:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                fn()
            e1.record()
            torch.cuda.synchronize()
            us.append(e0.elapsed_time(e1) * 1e3 / 20)
        rows.append({"entries": ne_, "one_block_us": round(us[0], 1), "split_us": round(us[1], 1), "speedup": round(us[0] / us[1], 2),
                     "same_selection": bool(torch.equal(out[0], out[1]) and torch.equal(cnt[0], cnt[1]))})
    print(json.dumps({"rows": R, "budget_entries": B, "pool": P, "scores": "relu" if a.relu else "normal", "by_entries": rows}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
