"""Long-context decode with and without row-granular KV tiering, after a real chunked prefill of the whole context.

    python -m layerstorm_b200.utils.long_context_bench --ctx 131072 --hot-window 8192 --steps 16

One process, one GPU, random-init weights of the named shape (``--layers N`` keeps the first N layers at full width):
  1. untiered engine: chunked prefill of ``--ctx`` synthetic tokens (timed), then ``--steps`` greedy decode steps under the
     CUDA graph (device time per step, CUDA events);
  2. tiered engine (``row_tiering``: only the last ``--hot-window`` tokens keep their HBM pages): the same prefill, at whose end the
     window slides (everything older moves to pinned host memory; included in the prefill time), then the same decode steps - every attention layer copies
     its selected rows' indices to the host, gathers the cold rows from pinned memory, copies them back and scatters them
     into the dense buffer the attention kernel reads.  These steps cannot be one CUDA graph (one host wait per layer).
The two runs must produce the same tokens (the tiering moves bytes verbatim).  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="glm-5.3-flash")
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--hot-window", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--headroom-gib", type=float, default=0.0, help="HBM kept free of weights (0 = sized from the context)")
    ap.add_argument("--no-tiered", action="store_true", help="measure the untiered engine only (a second prefill of a very long context is expensive)")
    ap.add_argument("--check-determinism", action="store_true", help="run the untiered case twice and compare the tokens")
    a = ap.parse_args(argv)

    import torch

    from ..models.config import get_preset
    from ..models.device_model import DeviceModel
    from ..runtime.engine import Engine

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = get_preset(a.model)
    if a.layers and a.layers < cfg.n_layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers, **({"layer_types": list(cfg.layer_types[:a.layers])} if cfg.layer_types else {}))
    n_attn = sum(1 for i in range(cfg.n_layers) if not cfg.is_kda_layer(i))
    page = 64
    max_ctx = a.ctx + a.steps + 2 * page
    kv_bytes = 700 * n_attn * (max_ctx + page)
    # prefill workspaces: indexer scores of a chunk against the whole context (fp32) dominate at long context
    ws_bytes = a.prefill_chunk * (max_ctx // max(1, cfg.index_kpool)) * 4 + int(2.6 * 2 ** 30)
    headroom = int(a.headroom_gib * 2 ** 30) if a.headroom_gib > 0 else kv_bytes + ws_bytes + int(1.0 * 2 ** 30)
    t0 = time.time()
    model = DeviceModel.random_init(cfg, dev, kv_fmt="fp8", page=page, seed=1234, expert_slots="auto", embed_on_host=True, reserve_bytes=headroom)
    slots = getattr(model, "expert_slots", cfg.n_routed)
    init_s = time.time() - t0
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, cfg.vocab, (a.ctx,), generator=g).tolist()
    num_pages = (max_ctx + page - 1) // page + 4
    out = {"model": cfg.name, "layers": cfg.n_layers, "attention_layers": n_attn, "ctx": a.ctx, "hot_window": a.hot_window, "steps": a.steps,
           "prefill_chunk": a.prefill_chunk, "kv_format": "fp8 latent, 64-token pages", "init_s": round(init_s, 1),
           "resident_expert_slots_per_layer": int(slots), "experts_per_layer": cfg.n_routed + cfg.n_shared,
           "valid_as_full_model_number": bool(not a.layers or a.layers >= get_preset(a.model).n_layers) and int(slots) >= cfg.n_routed + cfg.n_shared}

    def run(tiered: bool):
        cold_pages = (a.ctx + page - 1) // page + 2
        eng = Engine(model, max_seqs=1, max_ctx=max_ctx, prefill_chunk=a.prefill_chunk, max_batch=1, num_pages=num_pages, use_graph=not tiered,
                     row_tiering={"hot_window_tokens": a.hot_window, "cold_pages": cold_pages} if tiered else None)
        if not tiered:
            model.row_tier, model.idx_identity = None, False
        sid = eng.create_sequence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(eng.stream)
        tok = eng.prefill(sid, prompt)
        e1.record(eng.stream)
        torch.cuda.synchronize()
        r = {"prefill_s": round(e0.elapsed_time(e1) / 1e3, 2), "prefill_tok_s": round(a.ctx / (e0.elapsed_time(e1) / 1e3), 1)}
        if tiered:
            # the prefill call ends by sliding the window: its time includes the move of every older page to pinned host memory
            r["pages_moved_to_host"] = int(eng.row_tier.stats["demoted_pages"])
            r["d2h_bytes_of_the_move"] = int(eng.row_tier.stats["bytes_d2h"])
        toks = [tok]
        for _ in range(3):                                  # warm-up: graph capture (untiered), first use of the staging buffers (tiered)
            toks.append(eng.decode([sid], [toks[-1]])[0])
        torch.cuda.synchronize()
        st0 = dict(eng.row_tier.stats) if tiered else None
        ms = []
        for _ in range(a.steps):
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(eng.stream)
            toks.append(eng.decode([sid], [toks[-1]])[0])
            s1.record(eng.stream)
            torch.cuda.synchronize()
            ms.append(s0.elapsed_time(s1))
        ms.sort()
        r["decode_ms_per_step_median"] = round(ms[len(ms) // 2], 3)
        r["decode_tok_s"] = round(1e3 / ms[len(ms) // 2], 1)
        if tiered:
            st = eng.row_tier.stats
            r["cold_rows_fetched_per_step"] = round((st["cold_rows_fetched"] - st0["cold_rows_fetched"]) / a.steps, 1)
            r["h2d_bytes_per_step"] = int((st["bytes_h2d"] - st0["bytes_h2d"]) / a.steps)
            r["hbm_pages_in_use"] = int(num_pages - eng.free_page_count())
        else:
            r["hbm_pages_in_use"] = int(num_pages - eng.free_page_count())
        eng.free_sequence(sid)
        del eng
        torch.cuda.empty_cache()
        return toks, r

    t_plain, out["untiered"] = run(False)
    if a.check_determinism:
        t_again, _ = run(False)
        out["untiered_run_twice_same_tokens"] = t_plain == t_again
    if not a.no_tiered:
        t_tier, out["tiered"] = run(True)
        out["same_tokens"] = t_plain == t_tier
        if not out["same_tokens"]:
            out["first_different_token"] = next(i for i, (x, y) in enumerate(zip(t_plain, t_tier)) if x != y)    # 0 = the prefill's token
        out["tiering_cost"] = round(out["tiered"]["decode_ms_per_step_median"] / out["untiered"]["decode_ms_per_step_median"], 2)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
