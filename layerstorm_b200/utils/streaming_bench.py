"""Decode with a capped expert cache: routed experts live in pinned host memory and stream into a fixed number of HBM slots per layer.

    python -m layerstorm_b200.utils.streaming_bench --model glm-5.2 --layers 15 --slots 38 --ctx 2048 --steps 24

One GPU, random-init weights of the named shape cut to ``--layers`` layers at full width (the slice must fit in HBM once: the
streamer takes a resident model and moves its expert slots to the host).  Measured in this order on the same sequence:
  1. chunked prefill of ``--ctx`` synthetic tokens and ``--steps`` greedy decode steps with every expert resident (eager steps);
  2. ``ExpertStreamer`` with ``--slots`` slots per layer (+ next-layer prefetch unless ``--no-prefetch``), the same number of decode
     steps: device time per step, cache hit rate, host->device bytes and rate, waves, degraded steps.
With random weights the router is close to uniform, so the hit rate is about slots / experts - the worst case for a cache; trained
routers are far more skewed.  ``projected_full_depth`` scales the per-MoE-layer cost to the shape's real depth.  One JSON line.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="glm-5.2")
    ap.add_argument("--layers", type=int, default=15)
    ap.add_argument("--slots", type=int, default=38, help="expert slots per MoE layer kept in HBM")
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--expert-quant", default=None)
    ap.add_argument("--no-prefetch", action="store_true")
    ap.add_argument("--random-tokens", action="store_true",
                    help="feed a fresh random token every step instead of the greedy one: consecutive steps then route to different experts "
                         "(greedy decoding of a random-init model keeps choosing the same experts, which flatters the cache)")
    ap.add_argument("--zero-router-bias", action="store_true",
                    help="clear the routers' selection bias: a random-init bias dominates the random-init logits and sends every token to the "
                         "same experts; without it the routing follows the token")
    ap.add_argument("--deadline-ms", type=float, default=0.0, help="fetch deadline per wave (0 = wait for every expert)")
    a = ap.parse_args(argv)

    import torch

    from ..models.config import get_preset
    from ..models.device_model import DeviceModel
    from ..runtime.engine import Engine
    from ..runtime.streaming import ExpertStreamer

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    full = get_preset(a.model)
    cfg = full
    if a.layers and a.layers < full.n_layers:
        cfg = dataclasses.replace(full, n_layers=a.layers, **({"layer_types": list(full.layer_types[:a.layers])} if full.layer_types else {}))
    if a.expert_quant:
        cfg = dataclasses.replace(cfg, expert_quant=a.expert_quant)
    t0 = time.time()
    model = DeviceModel.random_init(cfg, dev, kv_fmt="fp8", page=64, seed=1234, expert_slots=None, embed_on_host=True)
    init_s = time.time() - t0
    if a.zero_router_bias:
        for L in model.layers:
            if L.get("router_bias") is not None:
                L["router_bias"].zero_()
    n_moe = sum(1 for i in range(cfg.n_layers) if cfg.is_moe_layer(i))
    n_moe_full = sum(1 for i in range(full.n_layers) if full.is_moe_layer(i))
    arena0 = next(L["arena"] for L in model.layers if L.get("arena") is not None)
    eng = Engine(model, max_seqs=1, max_ctx=a.ctx + 3 * a.steps + 64, prefill_chunk=2048, max_batch=1, use_graph=False)
    prompt = torch.randint(0, cfg.vocab, (a.ctx,), generator=torch.Generator().manual_seed(7)).tolist()
    sid = eng.create_sequence()
    tok = eng.prefill(sid, prompt)
    rg = torch.Generator().manual_seed(11)

    def decode(n):
        nonlocal tok
        ms = []
        for _ in range(n):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(eng.stream)
            tok = eng.decode([sid], [int(torch.randint(0, cfg.vocab, (1,), generator=rg)) if a.random_tokens else tok])[0]
            e1.record(eng.stream)
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        return ms

    decode(3)
    res_ms = sorted(decode(a.steps))[a.steps // 2]
    t1 = time.time()
    st = ExpertStreamer(model, slots_per_layer=a.slots, prefetch=not a.no_prefetch, fetch_deadline_ms=a.deadline_ms or None)
    move_s = time.time() - t1
    decode(3)
    s0 = dict(st.summary())
    w0 = time.time()
    ms = decode(a.steps)
    wall = time.time() - w0
    s1 = st.summary()
    d = {k: s1[k] - s0.get(k, 0) for k in ("hits", "misses", "bytes_h2d", "waves", "degraded_steps", "late_experts") if k in s1}
    med = sorted(ms)[a.steps // 2]
    per_moe_layer = (med - res_ms) / max(1, n_moe)
    out = {"model": full.name, "layers": cfg.n_layers, "moe_layers": n_moe, "experts_per_layer": cfg.n_routed + cfg.n_shared,
           "slots_per_layer": a.slots, "expert_format": cfg.expert_quant, "slot_bytes": int(arena0.ef.stride), "ctx": a.ctx, "steps": a.steps,
           "init_s": round(init_s, 1), "move_to_host_s": round(move_s, 1),
           "resident": {"decode_ms_per_step": round(res_ms, 3), "tok_s": round(1e3 / res_ms, 1)},
           "streamed": {"decode_ms_per_step": round(med, 3), "tok_s": round(1e3 / med, 2), "hit_rate": round(d["hits"] / max(1, d["hits"] + d["misses"]), 3),
                        "h2d_gb_per_step": round(d["bytes_h2d"] / a.steps / 1e9, 3), "h2d_gb_s": round(d["bytes_h2d"] / wall / 1e9, 1),
                        "waves_per_step": round(d["waves"] / a.steps, 1), "degraded_steps": d.get("degraded_steps", 0), "prefetch": not a.no_prefetch,
                        "tokens": "random per step" if a.random_tokens else "greedy",
                        "router_bias": "zeroed" if a.zero_router_bias else "random-init"},
           "projected_full_depth": {"moe_layers": n_moe_full,
                                    "decode_ms_per_step": round(res_ms / max(1, cfg.n_layers) * full.n_layers + per_moe_layer * n_moe_full, 1),
                                    "note": "resident time scaled by depth + streamed extra per MoE layer x the shape's MoE layers"},
           "valid_as_full_model_number": False}
    out["projected_full_depth"]["tok_s"] = round(1e3 / out["projected_full_depth"]["decode_ms_per_step"], 2)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
