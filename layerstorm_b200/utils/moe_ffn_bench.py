"""Routed-expert FFN microbenchmark for many-row steps (prefill chunks, large decode batches): the two tensor-core paths over
NVFP4 experts (``--format nvfp4``, default) or FP8 experts with power-of-two block scales (``--format fp8``), side by side.

  * ``fp16``          weights expanded to fp16 inside the operand pipeline, fp16 x fp16 tcgen05.mma (``lsb_moe_tc_ffn``)
  * ``block_scaled``  activations quantised to the weights' format, 4-bit x 4-bit (kind::mxf4nvf4) or 8-bit x 8-bit (kind::mxf8f6f4)
                      tcgen05.mma with block scales (``lsb_moe_bs_ffn`` / ``lsb_moe_bs_ffn_fp8``)

Both run sort -> (gather | quantise) -> gate/up + SwiGLU -> (quantise) -> down over the same routing.  Timing: CUDA events on
the launching stream, 3 warm-up iterations, median of ``--iters``; the expert weights of the default shape (289 experts,
4.1 GB) are larger than L2, so every iteration streams them from HBM.  One JSON line: per-phase and total microseconds, the
useful FLOPs (2 x pairs x 3 x hidden x inter) and the fraction of the measured bf16 GEMM peak (``bf16_tflops`` of
MEASURED_PEAKS.json in the working directory, else 1590), and the relative difference of the two results.

    python -m layerstorm_b200.utils.moe_ffn_bench --tokens 2048 --experts 288 --top-k 8 --hidden 4096 --inter 2048
"""
from __future__ import annotations

import argparse
import ctypes
import json
import statistics


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=288)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--shared", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--bn", type=int, default=0, help="token tile (32, 64, 128); 0 = by rows per expert")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--format", default="nvfp4", choices=["nvfp4", "fp8"])
    a = ap.parse_args(argv)

    import torch

    from ..models.device_model import ExpertArena, TcScratch, expert_layout
    from ..ops import _native as nat

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    H, F, E, S, R = a.hidden, a.inter, a.experts + a.shared, a.top_k + a.shared, a.tokens
    P = R * S
    gen = torch.Generator(device=dev).manual_seed(1)
    fp8 = a.format == "fp8"
    ef = expert_layout("fp8_e4m3" if fp8 else "nvfp4", H, F)
    arena = ExpertArena(ef, E, E, dev)
    arena.data.random_(0, 256, generator=gen)
    if fp8:
        arena.data[:, : ef.off_sg] &= 0xBF                                  # no NaN codes
        arena.data[:, ef.off_sg: ef.off_tail].view(torch.float32).fill_(2.0 ** -6)
    else:
        arena.data[:, ef.off_sg: ef.off_tail].random_(0x30, 0x40, generator=gen)
        arena.data[:, ef.off_tail: ef.off_tail + 12].view(torch.float32).fill_(0.01)
    arena.slot_of.copy_(torch.arange(E, dtype=torch.int32))
    efp = ctypes.addressof(arena.ef)
    x = torch.randn(R, H, device=dev, generator=gen).to(torch.bfloat16)
    routed = torch.stack([torch.randperm(a.experts, device=dev, generator=gen)[: a.top_k] for _ in range(R)])
    shared = torch.arange(a.experts, E, device=dev).expand(R, a.shared)
    ids = torch.cat([routed, shared], dim=1).int().contiguous()
    avg = P / max(1, min(E, P))
    bn = a.bn or (32 if avg <= 32 else (64 if avg <= 96 else 128))
    tiles = P // bn + E + 1
    i32 = dict(dtype=torch.int32, device=dev)
    sp, te, tr, tn, cnt = (torch.zeros(P, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32),
                           torch.zeros(2, **i32))
    err = TcScratch.get(dev).err
    u8 = torch.uint8
    xs = torch.zeros(P, H, dtype=torch.float16, device=dev)
    act16 = torch.zeros(P, F, dtype=torch.float16, device=dev)
    rows = tiles * bn
    vb, ak = (1, 128) if fp8 else (2, 64)                                   # values per byte, reduction elements per scale atom
    xq, xsf, xa = torch.zeros(rows, H // vb, dtype=u8, device=dev), torch.zeros(tiles * (H // ak) * 512, dtype=u8, device=dev), torch.zeros(rows, device=dev)
    actb = torch.zeros(rows, F, dtype=torch.float16, device=dev)
    aq, asf, aa = torch.zeros(rows, F // vb, dtype=u8, device=dev), torch.zeros(tiles * (F // ak) * 512, dtype=u8, device=dev), torch.zeros(rows, device=dev)
    y16, ybs = torch.zeros(P, H, device=dev), torch.zeros(P, H, device=dev)
    tl = (arena.data, arena.slot_of, efp, te, tr, tn, cnt, sp)
    if fp8:
        wsf, og, ou, od = arena.bs_scale_atoms()
        tb = (arena.data, arena.slot_of, efp, wsf, wsf.shape[1], og, ou, od, te, tr, tn, cnt, sp)
        quant_fn, ffn_fn = "lsb_quant_fp8_tiles", "lsb_moe_bs_ffn_fp8"
    else:
        tb, quant_fn, ffn_fn = tl, "lsb_quant_nvfp4_tiles", "lsb_moe_bs_ffn"

    phases = {
        "fp16": [("sort", lambda: nat.call("lsb_moe_tc_sort", ids, P, E, bn, sp, te, tr, tn, cnt)),
                 ("gather", lambda: nat.call("lsb_moe_tc_gather", x, sp, cnt, xs, P, S, H)),
                 ("gate_up", lambda: nat.call("lsb_moe_tc_ffn", 1, xs, P, *tl, act16, bn, tiles, 0.0, None, err, None)),
                 ("down", lambda: nat.call("lsb_moe_tc_ffn", 0, act16, P, *tl, y16, bn, tiles, 0.0, None, err, None))],
        "block_scaled": [("sort", lambda: nat.call("lsb_moe_tc_sort", ids, P, E, bn, sp, te, tr, tn, cnt)),
                         ("quant_x", lambda: nat.call(quant_fn, x, 0, sp, tr, tn, cnt, S, H, bn, tiles, xq, xsf, xa)),
                         ("gate_up", lambda: nat.call(ffn_fn, 1, xq, xsf, xa, *tb, actb, bn, tiles, 0.0, None, err)),
                         ("quant_act", lambda: nat.call(quant_fn, actb, 1, None, tr, tn, cnt, S, F, bn, tiles, aq, asf, aa)),
                         ("down", lambda: nat.call(ffn_fn, 0, aq, asf, aa, *tb, ybs, bn, tiles, 0.0, None, err))],
    }
    flops = 2.0 * P * 3 * H * F
    try:
        peak, src = float(json.load(open("MEASURED_PEAKS.json"))["bf16_tflops"]), "of measured"
    except Exception:
        peak, src = 1590.0, "of fallback"
    out = {"shape": {"tokens": R, "experts": a.experts, "top_k": a.top_k, "shared": a.shared, "hidden": H, "inter": F, "pairs": P, "token_tile": bn, "format": a.format},
           "weight_bytes": int(E * ef.stride), "useful_gflop": round(flops / 1e9, 1), "peak": src}
    for name, ph in phases.items():
        times = {k: [] for k, _ in ph}
        total = []
        for it in range(3 + a.iters):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(ph) + 1)]
            evs[0].record()
            for i, (_, fn) in enumerate(ph):
                fn()
                evs[i + 1].record()
            torch.cuda.synchronize()
            if it >= 3:
                for i, (k, _) in enumerate(ph):
                    times[k].append(evs[i].elapsed_time(evs[i + 1]) * 1e3)
                total.append(evs[0].elapsed_time(evs[-1]) * 1e3)
        us = statistics.median(total)
        out[name] = {"us_total": round(us, 1), "us_by_phase": {k: round(statistics.median(v), 1) for k, v in times.items()},
                     "tflops": round(flops / us / 1e6, 1), "fraction_of_bf16_gemm_peak": round(flops / us / 1e6 / peak, 3)}
    if int(err.item()) != 0:
        out["error_word"] = int(err.item())
    out["relative_difference_block_scaled_vs_fp16"] = round(float((ybs - y16).norm() / y16.norm()), 4)
    out["speedup_block_scaled"] = round(out["fp16"]["us_total"] / out["block_scaled"]["us_total"], 2)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
