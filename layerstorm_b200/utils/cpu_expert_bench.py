"""Stand-alone benchmark of the CPU expert kernels (the host-side expert device): one expert FFN from a slot image in a device storage format.

    python -m layerstorm_b200.utils.cpu_expert_bench --hidden 4096 --inter 2048 --formats bf16,fp8_e4m3,nvfp4,gguf_q4_k --tokens 1,8,64 --threads 0

No GPU needed.  For every (format, token count): median wall time of ``CpuExperts.ffn`` over a random slot image (3 warm-up calls), the
slot bytes streamed per second and the useful GFLOP/s (2 x tokens x 3 x hidden x inter), with the thread count of the fork-join pool.
Reference: tools/scout (stand-alone CPU expert benches).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import statistics
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--formats", default="bf16,fp8_e4m3,nvfp4,gguf_q4_k")
    ap.add_argument("--tokens", default="1,8,64")
    ap.add_argument("--threads", type=int, default=0, help="0 = min(32, cores)")
    ap.add_argument("--reps", type=int, default=7)
    a = ap.parse_args(argv)

    import torch

    from ..models.device_model import expert_layout
    from ..runtime import native as rt

    pool = rt.CpuExperts(a.threads)
    H, F = a.hidden, a.inter
    g = torch.Generator().manual_seed(3)
    rows = []
    for fmt in [f.strip() for f in a.formats.split(",") if f.strip()]:
        ef = expert_layout(fmt, H, F)
        slot = torch.empty(ef.stride, dtype=torch.uint8)
        slot.random_(0, 256, generator=g)
        if fmt == "bf16":
            slot.view(torch.bfloat16).normal_(0.0, 0.02, generator=g)
        elif fmt == "fp8_e4m3":
            slot[: ef.off_sg] &= 0xBF
            slot[ef.off_sg: ef.off_tail].view(torch.float32).fill_(0.03)
        elif fmt == "nvfp4":
            slot[ef.off_sg: ef.off_tail].random_(0x30, 0x40, generator=g)
            slot[ef.off_tail: ef.off_tail + 12].view(torch.float32).fill_(0.01)
        elif fmt == "gguf_q4_k":
            blocks = slot[: 3 * (H * F // 256 * 144)].view(-1, 144)
            blocks[:, :4] = torch.tensor([0.02 / 7.5 / 32.0, 0.02 / 32.0], dtype=torch.float16).view(torch.uint8)
            blocks[:, 4:16] = (blocks[:, 4:16] & 0x1F) | 0x10
        efp = ctypes.addressof(ef)
        for n in [int(t) for t in a.tokens.split(",") if t.strip()]:
            x = torch.randn(n, H, generator=g)
            out = torch.zeros(n, H)
            for _ in range(3):
                pool.ffn(efp, slot, x, limit=7.0, out=out)
            ts = []
            for _ in range(a.reps):
                t0 = time.perf_counter()
                pool.ffn(efp, slot, x, limit=7.0, out=out)
                ts.append(time.perf_counter() - t0)
            t = statistics.median(ts)
            wbytes = int(ef.off_tail if ef.off_tail > 0 else ef.stride)
            rows.append({"format": fmt, "tokens": n, "ms": round(t * 1e3, 3), "slot_gb_s": round(wbytes / t / 1e9, 2),
                         "gflop_s": round(2.0 * n * 3 * H * F / t / 1e9, 1), "finite": bool(torch.isfinite(out).all())})
    print(json.dumps({"hidden": H, "inter": F, "threads": pool.threads, "rows": rows}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
