#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s at 8k context on a GLM-5.3-Flash-shape model (glm5_next: 45 layers, hidden
4096, 34 KDA + 11 sparse-MLA layers, mHC x4, 288 routed NVFP4 experts top-8 + 1 shared, bf16 attention, FP8 KV cache),
random-init weights and synthetic token ids.  The reference publishes, for this workload on its own hardware
(README.md:57,124): decode 24.5 tok/s @8k, prefill 159 tok/s on a 27k prompt with 2048-token chunks, TTFT not published.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference ...                     # the reference arm

One process measures, in this order, everything the metric names:
  1. chunked prefill of a 27k-token prompt (2048-token chunks): prefill tok/s and time to first token;
  2. batch-1 decode at 8k context after a real prefill (the headline ``value`` and ``e2e``);
  3. batch-32 decode at 8k context after a real prefill of all 32 sequences (skipped with a reason where the weights
     leave no room for 32 sequences of recurrent state on one GPU).
One JSON line is printed by rank 0.  ``value`` times only the device work of the K decode steps (CUDA events around each
step's graph replay, summed, max over ranks); ``e2e`` times the same K steps through the public ``Engine.decode`` call,
including each step's host->device copy of the inputs from pinned memory and the device->host read of the sampled token.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

BASELINE_DECODE_8K = 24.5      # tok/s, reference README.md:57 (GLM-5.3-Flash, decode @8k)
BASELINE_PREFILL_27K = 159.0   # tok/s, reference README.md:57 (27k prompt, 2048-token chunks)


def reference_arm(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference cannot be installed offline: no setup.py/pyproject.toml (pip: 'not installable'), its CUDA "
                       "kernel submodules are empty and every CUDA target is compute_120-only",
    }))
    return 0


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = f"/tmp/lsb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def streamed_bytes_per_step(model, batch: int) -> int:
    """Weight bytes one decode step of ``batch`` rows reads on THIS rank: every dense matrix once, per MoE layer the routed
    experts the rows select (at most the resident ones) plus the shared expert."""
    from layerstorm_b200.models.device_model import ExpertArena, QLinear
    cfg = model.cfg
    tot = model.head.nbytes()
    for L in model.layers:
        for v in L.values():
            if isinstance(v, QLinear):
                tot += v.nbytes()
            elif isinstance(v, ExpertArena):
                hit = min(cfg.n_routed, batch * cfg.top_k)
                per_rank = hit + cfg.n_shared if model.expert_shard == "tp" else (hit + model.tp_size - 1) // model.tp_size + cfg.n_shared
                tot += min(v.n_slots, per_rank) * v.ef.stride
            elif hasattr(v, "numel") and not isinstance(v, tuple):
                tot += v.numel() * v.element_size()
            elif isinstance(v, tuple):
                tot += sum(t.numel() * t.element_size() for t in v)
    return tot


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="glm-5.3-flash")
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--long-prompt", type=int, default=27000, help="prompt length of the prefill / TTFT case (0 = skip)")
    ap.add_argument("--headroom-gib", type=float, default=None,
                    help="HBM left free after weights (KV / recurrent state, workspaces); default: sized from the largest batch")
    ap.add_argument("--no-graph", action="store_true", help="eager launches (for per-kernel profiling)")
    ap.add_argument("--synthetic-fill", action="store_true", help="skip the real prefill; decode over an uninitialised cache (the line is marked invalid)")
    ap.add_argument("--extra-batches", default="32", help="comma-separated batch sizes measured after the main case in the same process ('' = none)")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel degree (0 = the number of GPUs; other values are refused: attention, "
                                                      "KDA and dense FFN are sharded over all ranks of the job)")
    ap.add_argument("--ep", type=int, default=0, help="expert-parallel degree (0 = the number of GPUs; other values are refused)")
    ap.add_argument("--expert-shard", default=None, choices=["ep", "tp"],
                    help="N > 1 GPUs: 'ep' = whole experts, expert e on GPU e %% N; 'tp' = every GPU holds a 1/N slice of every expert (default: tp)")
    ap.add_argument("--moe-block-scaled", action="store_true",
                    help="many-row steps (prefill chunks, batch >= 16) quantise the expert activations to NVFP4 and run the 4-bit x 4-bit "
                         "block-scaled tensor-core kernel (the reference's NVFP4 expert path does the same); default: bf16 -> fp16 activations")
    ap.add_argument("--dcp-chunk", type=int, default=0,
                    help="N > 1 GPUs: shard the latent KV cache over the ranks in chunks of this many tokens (context parallel); 0 = replicated")
    ap.add_argument("--layers", type=int, default=0, help="smoke runs only: keep the first N layers (the JSON line is then marked invalid)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.moe_block_scaled:
        os.environ["LSB_MOE_BLOCK_SCALED"] = "1"
    if args.warmup < 3:
        args.warmup = 3
    extra = [int(x) for x in args.extra_batches.split(",") if x.strip() and int(x) != args.batch]

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if (args.tp and args.tp != world) or (args.ep and args.ep != world):
        if rank == 0:
            print(json.dumps({"unavailable": f"tp{args.tp or world} x ep{args.ep or world} on {world} GPUs: this engine shards attention, KDA and the "
                                             f"dense FFN over all ranks of the job and owns expert e on rank e % N (tp{world}ep{world}); "
                                             "expert-only ranks (EP beyond TP) are not built"}))
        return 0
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.runtime.engine import Engine

    cfg = get_preset(args.model)
    if args.layers and args.layers < cfg.n_layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, n_layers=args.layers, **({"layer_types": list(cfg.layer_types[:args.layers])} if cfg.layer_types else {}))
    dev = torch.device("cuda", local)
    t0 = time.time()

    # ---- how many sequences fit next to the weights: recurrent state + KV of a sequence, workspaces of a step ----
    n_kda = sum(1 for i in range(cfg.n_layers) if cfg.is_kda_layer(i))
    kda_seq = n_kda * (cfg.kda_heads // world) * (cfg.kda_head_dim ** 2 * 4 + 9 * cfg.kda_head_dim * 4)
    kv_tok = 700 * sum(1 for i in range(cfg.n_layers) if not cfg.is_kda_layer(i))           # FP8 latent + rope + indexer entry, rounded up
    per_seq = kda_seq + kv_tok * (args.ctx + 256)
    fixed = int(2.6 * 2 ** 30) + kv_tok * (args.long_prompt + 4096)                          # prefill workspaces + the long prompt's cache
    free_b, total_b = torch.cuda.mem_get_info(dev)
    bmax = max([args.batch] + extra)
    if args.headroom_gib is None:
        headroom = fixed + per_seq * bmax + int(0.04 * 2 ** 30) * bmax
    else:
        headroom = int(args.headroom_gib * 2 ** 30)
    # as many routed-expert slots per layer as fit in HBM next to the other weights; any remainder
    # would be streamed from pinned host RAM by the expert cache
    model = DeviceModel.random_init(cfg, dev, kv_fmt="fp8", page=64, seed=1234, expert_slots="auto", embed_on_host=True,
                                    reserve_bytes=headroom, tp_rank=rank, tp_size=world, expert_shard=args.expert_shard)
    slots = getattr(model, "expert_slots", cfg.n_routed)
    owned = max(sum(1 for e in range(cfg.n_routed + cfg.n_shared) if model.owns_expert(i, e)) for i in range(cfg.n_layers) if cfg.is_moe_layer(i)) \
        if cfg.n_routed else 0
    skipped = {}
    if cfg.n_routed and slots < owned and bmax > args.batch and args.headroom_gib is None:
        # the large batch does not fit next to fully resident experts on this many GPUs: rebuild for the main case only
        del model
        torch.cuda.empty_cache()
        for b_ in extra:
            skipped[b_] = (f"weights ({owned} experts per MoE layer resident) leave no room for {b_} sequences of recurrent state and "
                           f"workspaces on {world} GPU(s) of {total_b / 2 ** 30:.0f} GiB; measured from the GPU count where they fit")
        extra, bmax = [], args.batch
        headroom = fixed + per_seq * bmax + int(0.04 * 2 ** 30) * bmax
        model = DeviceModel.random_init(cfg, dev, kv_fmt="fp8", page=64, seed=1234, expert_slots="auto", embed_on_host=True,
                                        reserve_bytes=headroom, tp_rank=rank, tp_size=world, expert_shard=args.expert_shard)
        slots = getattr(model, "expert_slots", cfg.n_routed)
    if world > 1:
        # in-kernel NVLink all-reduce buffers (peer-mapped) sized for the largest step (a prefill chunk); NCCL only bootstraps
        from layerstorm_b200.parallel.symm import PeerComm
        comm = PeerComm(max(4, bmax, args.prefill_chunk) * cfg.hidden, dev)
        comm_amax = PeerComm(2 * max(bmax, 4), dev)
        model.attach_comm(comm, comm_amax)
        if args.dcp_chunk > 0:
            from layerstorm_b200.parallel.dcp import DcpAttention
            model.enable_dcp(DcpAttention(cfg.n_heads, cfg.kv_lora, cfg.qk_rope, max_rows=max(bmax, args.prefill_chunk), device=dev,
                                          chunk=args.dcp_chunk, n_splits=4))
    max_ctx = max(args.ctx + args.steps + args.warmup + 64, args.long_prompt + 64)
    page = 64
    num_pages = bmax * ((args.ctx + args.steps + args.warmup + 64 + page - 1) // page + 1) + (args.long_prompt + page - 1) // page + 2
    eng = Engine(model, max_seqs=bmax, max_ctx=max_ctx, prefill_chunk=args.prefill_chunk, max_batch=bmax, num_pages=num_pages,
                 use_graph=not args.no_graph)
    torch.cuda.synchronize()
    t_init = time.time() - t0
    g = torch.Generator().manual_seed(7)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(*vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def timed_prefill(sid, prompt):
        """Device time of a chunked prefill through the public call (CUDA events on the engine stream), max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(eng.stream)
        tok = eng.prefill(sid, prompt)
        e1.record(eng.stream)
        barrier()
        return tok, max_over_ranks(e0.elapsed_time(e1))[0]

    # ---- case 1: the long prompt (prefill tok/s, time to first token) ----
    long_case = None
    if args.long_prompt > 0 and not args.synthetic_fill:
        warm = eng.create_sequence()                       # first use of the prefill workspace, kernels' one-time set-up
        eng.prefill(warm, torch.randint(0, cfg.vocab, (args.prefill_chunk,), generator=g).tolist())
        eng.free_sequence(warm)
        sid = eng.create_sequence()
        prompt = torch.randint(0, cfg.vocab, (args.long_prompt,), generator=g).tolist()
        _, ms = timed_prefill(sid, prompt)
        eng.free_sequence(sid)
        long_case = {"prompt_tokens": args.long_prompt, "chunk": args.prefill_chunk, "prefill_tok_s": round(args.long_prompt / (ms / 1e3), 1),
                     "ttft_ms": round(ms, 2), "vs_baseline_prefill": round(args.long_prompt / (ms / 1e3) / BASELINE_PREFILL_27K, 2)
                     if (args.model == "glm-5.3-flash" and args.long_prompt == 27000 and args.prefill_chunk == 2048) else None,
                     "expert_activations": "nvfp4 (block-scaled)" if getattr(eng.ws_prefill, "bs_ok", False) else "fp16"}
        # the same prompt once more with the other many-row expert path (NVFP4 activations on the block-scaled 4-bit x 4-bit kernel, as the
        # reference's NVFP4 expert path computes): a second, separately labelled number; the headline keys above stay on the default path
        ws_p = eng.ws_prefill
        if ws_p is not None and getattr(ws_p, "bs_can", False) and not ws_p.bs_ok:
            try:
                ws_p.set_block_scaled(True)
                sid = eng.create_sequence()
                eng.prefill(sid, prompt[: args.prefill_chunk])         # first use of the path's buffers and tensor maps
                eng.free_sequence(sid)
                sid = eng.create_sequence()
                _, ms2 = timed_prefill(sid, prompt)
                eng.free_sequence(sid)
                long_case["block_scaled_experts"] = {"prefill_tok_s": round(args.long_prompt / (ms2 / 1e3), 1), "ttft_ms": round(ms2, 2),
                                                     "expert_activations": "nvfp4, tcgen05.mma kind::mxf4nvf4.block_scale"}
            except RuntimeError as e:                                   # no room for the second path's buffers beside the weights
                long_case["block_scaled_experts"] = {"unavailable": str(e).splitlines()[0][:160]}
                torch.cuda.empty_cache()
            finally:
                ws_p.set_block_scaled(False)

    # ---- cases 2..: decode at the context length, main batch first, then the extra batches on top of the same sequences ----
    sids, toks, results = [], [], []
    ttft_ctx_ms = None
    for case_i, B_case in enumerate([args.batch] + extra):
        while len(sids) < B_case:
            sid = eng.create_sequence()
            if args.synthetic_fill:
                s = eng.seqs[sid]
                eng._ensure_pages(s, args.ctx)
                s.length = args.ctx
                tok = 1
            else:
                prompt = torch.randint(0, cfg.vocab, (args.ctx,), generator=g).tolist()
                if ttft_ctx_ms is None:
                    tok, ttft_ctx_ms = timed_prefill(sid, prompt)
                else:
                    tok = eng.prefill(sid, prompt)
            sids.append(sid)
            toks.append(tok)
        for _ in range(args.warmup):
            toks = eng.decode(sids, toks)

        # ---- timed region 1: public API end to end (H2D inputs + graph + D2H token per step) ----
        sampler = ClockSampler(local)
        sampler.start()
        h2d0, d2h0, l0 = eng.h2d_bytes, eng.d2h_bytes, eng.kernel_launches
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(eng.stream)
        for _ in range(args.steps):
            toks = eng.decode(sids, toks)
        e1.record(eng.stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1)
        h2d = (eng.h2d_bytes - h2d0) / args.steps
        d2h = (eng.d2h_bytes - d2h0) / args.steps
        launches = eng.kernel_launches - l0

        # ---- timed region 2: device time of the step itself (graph replay only) ----
        B = B_case
        graph = eng.graphs.get(B)
        if graph is None:      # eager mode: device timing = the same loop
            class _G:
                def replay(self_inner):
                    eng.model.forward(eng.ws_decode[B], B, B, 0, B)
                    eng.model.argmax(eng.ws_decode[B], B)
            graph = _G()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        torch.cuda.synchronize()
        with torch.cuda.stream(eng.stream):
            for a, b in evs:
                # advance the sequences like decode() does, without the host round trip
                for sid in sids:
                    s = eng.seqs[sid]
                    eng._ensure_pages(s, s.length + 1)
                rows = [(int(t), eng.seqs[sid].slot, eng.seqs[sid].length) for sid, t in zip(sids, toks)]
                eng._stage(eng.ws_decode[B], rows, [(j, 1, eng.seqs[sid].slot) for j, sid in enumerate(sids)])
                a.record(eng.stream)
                graph.replay()
                b.record(eng.stream)
                for sid in sids:
                    eng.seqs[sid].length += 1
        torch.cuda.synchronize()
        dev_ms = sum(a.elapsed_time(b) for a, b in evs)
        clocks = sampler.stop()
        miss = int(eng.ws_decode[B].miss[0]) if hasattr(eng.ws_decode[B], "miss") else 0
        dev_ms, e2e_ms = max_over_ranks(dev_ms, e2e_ms)
        results.append({"batch": B, "tok_s": round(B * args.steps / (dev_ms / 1e3), 3), "ms_per_step": round(dev_ms / args.steps, 4),
                        "e2e_tok_s": round(B * args.steps / (e2e_ms / 1e3), 3), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "gpu_launches": launches, "clocks": clocks, "expert_miss_flag": miss,
                        "weights_streamed_gb_per_step_per_gpu": round(streamed_bytes_per_step(model, B) / 1e9, 2)})
    comm_err = (model.comm.error() or model.comm_amax.error()) if model.comm is not None else 0

    if rank == 0:
        main_r = results[0]
        headline = args.model == "glm-5.3-flash" and args.ctx == 8192 and args.batch == 1 and not args.layers
        fill = "synthetic (uninitialised cache)" if args.synthetic_fill else "real chunked prefill of every sequence"
        out = {
            "metric": "decode tok/s @8k ctx" if args.ctx == 8192 else f"decode tok/s @{args.ctx} ctx",
            "value": main_r["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main_r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(main_r["tok_s"] / BASELINE_DECODE_8K, 3) if headline else None,
            "dtype": "bf16", "data": "synthetic token ids, random-init weights",
            "config": {"model": cfg.name + "-shape", "global_batch": args.batch, "seq_len": args.ctx,
                       "parallelism": (f"tp{world}" + (f"ep{world}" if model.expert_shard == "ep" else f" (experts sliced over the {world} GPUs)")) if world > 1 else "single-gpu",
                       "weights": f"experts {cfg.expert_quant}, attention {cfg.dense_quant}",
                       "expert_activations_many_rows": "nvfp4 (block-scaled 4-bit x 4-bit MMA)" if os.environ.get("LSB_MOE_BLOCK_SCALED", "0") not in ("", "0") else "fp16",
                       "kv_cache": "fp8+bf16-rope, 64-token pages" + (f", sharded over the ranks in {args.dcp_chunk}-token chunks" if (world > 1 and args.dcp_chunk > 0) else ""),
                       "l2": f"inputs larger than L2 (each step streams {main_r['weights_streamed_gb_per_step_per_gpu']} GB of weights per GPU; L2 is 0.126 GB)",
                       "resident_expert_slots_per_layer_per_gpu": slots, "routed_experts": cfg.n_routed, "expert_miss_flag": main_r["expert_miss_flag"],
                       "comm_error_word": comm_err,
                       "collectives": ("fused in-kernel NVLink all-reduce (P2P stores + flags) in the GEMV / tcgen05-GEMM / MoE-combine epilogues, argmax exchange; no NCCL on the step path"
                                       if world > 1 else "none"),
                       "context_fill": fill},
            "clocks": main_r["clocks"],
            "e2e": {"value": main_r["e2e_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": main_r["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": main_r["d2h_bytes_per_step"]},
            "gpu_launches": main_r["gpu_launches"],
            # the rest of the metric BASELINE.json names, measured in the same process with the same rules
            "prefill": long_case if long_case is not None else {"unavailable": "skipped (--long-prompt 0 or --synthetic-fill)"},
            "ttft_ms": {"prompt_%d" % args.ctx: round(ttft_ctx_ms, 2) if ttft_ctx_ms is not None else None,
                        **({"prompt_%d" % args.long_prompt: long_case["ttft_ms"]} if long_case else {})},
            "decode_batches": {str(r["batch"]): {k: r[k] for k in ("tok_s", "ms_per_step", "e2e_tok_s", "h2d_bytes_per_step", "d2h_bytes_per_step",
                                                                     "gpu_launches", "expert_miss_flag", "weights_streamed_gb_per_step_per_gpu")}
                               | {"steps": args.steps, "warmup": args.warmup, "context_fill": fill, "clock_reasons": r["clocks"]["reasons"]}
                               for r in results} | {str(b_): {"unavailable": why} for b_, why in skipped.items()},
            **({"invalid": "context marked filled, not prefilled (--synthetic-fill)"} if args.synthetic_fill else {}),
            **({"invalid": f"depth reduced to {args.layers} layers (smoke run)"} if args.layers else {}),
            "extra": {"init_s": round(t_init, 1), "weight_gib": round(model.weight_bytes() / 2 ** 30, 2),
                      "reference_published": {"decode_tok_s_8k": BASELINE_DECODE_8K, "prefill_tok_s_27k": BASELINE_PREFILL_27K,
                                              "hardware": "2x RTX 5090 + 2x RTX 5080 (reference README.md:47-57)"}},
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
