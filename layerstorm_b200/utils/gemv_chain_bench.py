"""Decode GEMV chain microbenchmark: the weight-streaming kernels of one MoE layer's tail at M = 1.

The chain is the one the reference times in bench/gemv_chain (README.md:27-50 there): the attention output projection,
the routed experts' gate / up / down projections for the token's top-k experts and the shared expert, i.e. every byte
one decode token streams between attention and the next layer's norm.  The reference reports 318.8 us (its own kernels)
and 94.7 us (ggml) on an RTX 5090 for a GGUF-quantised chain; here the chain runs in this engine's storage formats
(bf16 / FP8 projection, NVFP4 or Q4_K experts).

    python -m layerstorm_b200.utils.gemv_chain_bench --hidden 4096 --o-in 16384 --inter 2048 --experts 288 --top-k 8

Timing: CUDA events around the chain on the launching stream, 5 warm-up iterations, an L2 flush (a 256 MB write) before
every timed iteration, median of ``--iters``.  Prints one JSON line with the time, the bytes streamed and the fraction of
the measured copy bandwidth (``--hbm-gbs``, default: ``hbm_gbs`` of MEASURED_PEAKS.json in the working directory, else 6650).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--o-in", type=int, default=16384, help="input width of the attention output projection (heads x v_head)")
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=288)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--dense-quant", default="bf16", choices=["bf16", "fp8_e4m3", "nvfp4", "gguf_q4_k"])
    ap.add_argument("--expert-quant", default="nvfp4", choices=["nvfp4", "gguf_q4_k", "fp8_e4m3", "bf16"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--hbm-gbs", type=float, default=0.0)
    a = ap.parse_args(argv)

    import torch

    from ..models.device_model import ExpertArena, QLinear, expert_layout
    from ..ops import _native as nat

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    H, F, E, K = a.hidden, a.inter, a.experts, a.top_k
    S = K + 1
    gen = torch.Generator(device=dev).manual_seed(1)
    o_proj = QLinear.random(H, a.o_in, a.dense_quant, dev, gen=gen)
    ef = expert_layout(a.expert_quant, H, F)
    arena = ExpertArena(ef, E + 1, E + 1, dev)
    arena.data.random_(0, 256, generator=gen)
    if a.expert_quant == "nvfp4":
        arena.data[:, ef.off_sg: ef.off_tail].random_(0x30, 0x40, generator=gen)
        arena.data[:, ef.off_tail: ef.off_tail + 12].view(torch.float32).fill_(0.01)
    elif a.expert_quant == "fp8_e4m3":
        arena.data[:, : ef.off_sg] &= 0xBF
        arena.data[:, ef.off_sg: ef.off_tail].view(torch.float32).fill_(0.03)
    elif a.expert_quant == "bf16":
        arena.data.view(torch.bfloat16).normal_(0.0, 0.02, generator=gen)
    arena.slot_of.copy_(torch.arange(E + 1, dtype=torch.int32))
    efp = ctypes.addressof(arena.ef)
    x_attn = torch.randn(1, a.o_in, device=dev, generator=gen).to(torch.bfloat16)
    x = torch.randn(1, H, device=dev, generator=gen).to(torch.bfloat16)
    sub = torch.zeros(1, H, device=dev)
    ids = torch.cat([torch.randperm(E, device=dev, generator=gen)[:K], torch.tensor([E], device=dev)]).int().view(1, S).contiguous()
    wts = torch.rand(1, S, device=dev, generator=gen)
    act = torch.zeros(S, F, dtype=torch.bfloat16, device=dev)
    y = torch.zeros(S, H, device=dev)
    out = torch.zeros(1, H, device=dev)
    pair_mode = a.expert_quant == "nvfp4" and H % 128 == 0 and F % 128 == 0
    if not pair_mode:
        i32 = dict(dtype=torch.int32, device=dev)
        g_e, g_n, g_p, n_g, cnt = (torch.zeros(S, **i32), torch.zeros(S, **i32), torch.zeros(4 * S, **i32), torch.zeros(1, **i32),
                                   torch.zeros(2 * (E + 1) + 2, **i32))

    def chain():
        o_proj(sub, x_attn, 1)
        if pair_mode:
            nat.call("lsb_moe_gateup", x, arena.data, arena.slot_of, efp, ids, None, None, None, act, S, S, 0.0, None, 0)
            nat.call("lsb_moe_down", act, arena.data, arena.slot_of, efp, ids, None, None, None, y, S, 0)
        else:
            nat.call("lsb_moe_build_groups", ids, S, E + 1, g_e, g_n, g_p, n_g, cnt)
            nat.call("lsb_moe_gateup", x, arena.data, arena.slot_of, efp, g_e, g_n, g_p, n_g, act, S, S, 0.0, None, 0)
            nat.call("lsb_moe_down", act, arena.data, arena.slot_of, efp, g_e, g_n, g_p, n_g, y, S, 0)
        nat.call("lsb_moe_combine", out, y, wts, ids, arena.slot_of, 1, S, H, 0, None)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(5):
        chain()
    torch.cuda.synchronize()
    times = []
    for _ in range(a.iters):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        chain()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    us = statistics.median(times)
    stream_bytes = o_proj.nbytes() + S * (ef.off_tail if ef.off_tail > 0 else ef.stride)
    peak = a.hbm_gbs
    src = "argument"
    if peak <= 0:
        try:
            peak, src = float(json.load(open("MEASURED_PEAKS.json"))["hbm_gbs"]), "of measured"
        except Exception:
            peak, src = 6650.0, "of fallback"
    gbs = stream_bytes / (us * 1e-6) / 1e9
    print(json.dumps({"chain": f"o_proj[{H}x{a.o_in}] {a.dense_quant} + {K} routed + 1 shared experts {a.expert_quant} (hidden {H}, inter {F}) + combine",
                      "us_median": round(us, 2), "us_min": round(min(times), 2), "iters": a.iters, "bytes_streamed": stream_bytes,
                      "gb_per_s": round(gbs, 1), "fraction_of_copy_peak": round(gbs / peak, 3), "peak": src,
                      "l2": "256 MB flush write before every timed iteration", "reference_published_us": {"own_kernels_rtx5090": 318.8, "ggml_rtx5090": 94.7}}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
