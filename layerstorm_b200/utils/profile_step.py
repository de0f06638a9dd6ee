"""Depth-reduced decode / prefill driver for kernel profiling.

A full-size model holds 100+ GB on the device, which is the wrong thing to put under a multi-pass profiler
(the profiler saves and restores device memory around every pass).  This driver builds the first ``--layers``
layers of a preset with the real widths (hidden size, heads, experts, vocabulary), so every kernel of a step
runs at its production shape while only a few GB are resident, and runs eager (no CUDA graph) steps so that a
profiler sees the individual launches:

    python -m layerstorm_b200.utils.profile_step --model glm-5.3-flash --layers 4 --ctx 8192 --steps 3
    python -m layerstorm_b200.utils.profile_step --model glm-5.3-flash --layers 4 --ctx 4096 --prefill --steps 0

``--no-prefill`` (default for decode profiling) marks the context as filled without computing it, so the first
launches a profiler meets are already decode launches.  The printed times are wall-clock per eager step and are
not benchmark numbers.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="glm-5.3-flash")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--prefill", action="store_true", help="compute the context with chunked prefill instead of marking it filled")
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--kv-format", default="fp8", choices=["fp8", "bf16", "tq4"])
    ap.add_argument("--expert-quant", default=None)
    ap.add_argument("--time-calls", action="store_true",
                    help="with --prefill: after the context is filled, run ONE more prefill chunk with CUDA events around every kernel-launcher "
                         "call and print the table (device time per launcher; the chunk's kernels are long, the event overhead is not)")
    a = ap.parse_args(argv)

    import torch

    from ..models.config import get_preset
    from ..models.device_model import DeviceModel
    from ..runtime.engine import Engine

    cfg = get_preset(a.model)
    L = min(a.layers, cfg.n_layers)
    repl = {"n_layers": L}
    if getattr(cfg, "layer_types", None):
        repl["layer_types"] = list(cfg.layer_types[:L])
    if a.expert_quant:
        repl["expert_quant"] = a.expert_quant
    cfg = dataclasses.replace(cfg, **repl)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    model = DeviceModel.random_init(cfg, dev, kv_fmt=a.kv_format, page=64, seed=1234, embed_on_host=True)
    eng = Engine(model, max_seqs=a.batch, max_ctx=a.ctx + a.steps + 64 + (a.prefill_chunk if a.time_calls else 0), prefill_chunk=a.prefill_chunk, max_batch=a.batch, use_graph=False)
    g = torch.Generator().manual_seed(7)
    sids = [eng.create_sequence() for _ in range(a.batch)]
    toks = []
    t0 = time.time()
    if a.prefill:
        for sid in sids:
            toks.append(eng.prefill(sid, torch.randint(0, cfg.vocab, (a.ctx,), generator=g).tolist()))
    else:
        for sid in sids:
            s = eng.seqs[sid]
            eng._ensure_pages(s, a.ctx)
            s.length = a.ctx
            toks.append(1)
    torch.cuda.synchronize()
    t_fill = time.time() - t0
    if a.time_calls:
        from ..ops import _native as nat
        chunk = torch.randint(0, cfg.vocab, (a.prefill_chunk,), generator=g).tolist()
        with nat.call_timer() as tm:
            eng.prefill(sids[0], chunk)
        rows = sorted(tm.summary().items(), key=lambda kv: -kv[1][1])
        total = sum(ms for _, (_, ms) in rows)
        print(f"# one {a.prefill_chunk}-token prefill chunk at context {a.ctx}, {L} layers ({', '.join(getattr(cfg, 'layer_types', []) or [])}): "
              f"{total:.2f} ms in launcher calls")
        print("| launcher | calls | ms | share |\n|---|---|---|---|")
        for name, (c, ms) in rows:
            print(f"| `{name}` | {c} | {ms:.3f} | {100 * ms / total:.1f}% |")
    times = []
    for _ in range(a.steps):
        t0 = time.time()
        toks = eng.decode(sids, toks)
        torch.cuda.synchronize()
        times.append((time.time() - t0) * 1e3)
    print(json.dumps({"model": cfg.name, "layers": L, "layer_types": list(getattr(cfg, "layer_types", []) or []), "ctx": a.ctx, "batch": a.batch,
                      "fill_s": round(t_fill, 3), "prefill": a.prefill, "eager_step_ms": [round(t, 3) for t in times],
                      "device_gib": round(torch.cuda.memory_allocated() / 2 ** 30, 2)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
