#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode tokens/s at 8k context on a GLM-5.3-Flash-shape
model (glm5_next: 45 layers, hidden 4096, 34 KDA + 11 sparse-MLA layers, mHC x4, 288 routed
NVFP4 experts top-8 + 1 shared, bf16 attention, FP8 KV cache), random-init weights and
synthetic token ids.  The reference publishes 24.5 tok/s for this workload on its own
hardware (README.md:57,124).

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference ...                     # the reference arm

One JSON line is printed by rank 0.  ``value`` times only the device work of the K decode
steps (CUDA events around each step's graph replay, summed, max over ranks); ``e2e`` times the
same K steps through the public ``Engine.decode`` call, including each step's host->device
copy of the inputs from pinned memory and the device->host read of the sampled token.
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
    ap.add_argument("--headroom-gib", type=float, default=None,
                    help="HBM left free after weights (KV / recurrent state, workspaces); default 2.5 GiB + 0.35 GiB per sequence of the batch")
    ap.add_argument("--no-graph", action="store_true", help="eager launches (for per-kernel profiling)")
    ap.add_argument("--synthetic-fill", action="store_true", help="skip the real prefill; decode over an uninitialised cache")
    ap.add_argument("--extra-batches", default="", help="comma-separated batch sizes measured after the main case in the same process (one more JSON line each)")
    ap.add_argument("--dcp-chunk", type=int, default=0,
                    help="N > 1 GPUs: shard the latent KV cache over the ranks in chunks of this many tokens (context parallel); 0 = replicated")
    ap.add_argument("--layers", type=int, default=0, help="smoke runs only: keep the first N layers (the JSON line is then marked invalid)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.headroom_gib is None:
        args.headroom_gib = 2.5 + 0.35 * max([args.batch] + [int(x) for x in args.extra_batches.split(",") if x.strip()])

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel, expert_layout
    from layerstorm_b200.runtime.engine import Engine

    cfg = get_preset(args.model)
    if args.layers and args.layers < cfg.n_layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, n_layers=args.layers, **({"layer_types": list(cfg.layer_types[:args.layers])} if cfg.layer_types else {}))
    dev = torch.device("cuda", local)
    t0 = time.time()
    # as many routed-expert slots per layer as fit in HBM next to the other weights; any remainder
    # would be streamed from pinned host RAM by the expert cache
    model = DeviceModel.random_init(cfg, dev, kv_fmt="fp8", page=64, seed=1234, expert_slots="auto", embed_on_host=True,
                                    reserve_bytes=int(args.headroom_gib * 2 ** 30), tp_rank=rank, tp_size=world)
    slots = getattr(model, "expert_slots", cfg.n_routed)
    if world > 1:
        # in-kernel NVLink all-reduce buffers (peer-mapped) sized for the largest step (a prefill chunk); NCCL only bootstraps
        from layerstorm_b200.parallel.symm import PeerComm
        bmax = max([args.batch] + [int(x) for x in args.extra_batches.split(",") if x.strip()])
        comm = PeerComm(max(4, bmax, args.prefill_chunk) * cfg.hidden, dev)
        comm_amax = PeerComm(2 * max(bmax, 4), dev)
        model.attach_comm(comm, comm_amax)
        if args.dcp_chunk > 0:
            from layerstorm_b200.parallel.dcp import DcpAttention
            model.enable_dcp(DcpAttention(cfg.n_heads, cfg.kv_lora, cfg.qk_rope, max_rows=max(bmax, args.prefill_chunk), device=dev,
                                          chunk=args.dcp_chunk, n_splits=4))
    extra = [int(x) for x in args.extra_batches.split(",") if x.strip()]
    cases = [(args.batch, args.synthetic_fill)] + [(b_, True) for b_ in extra]
    eng = None
    for case_i, (B_case, synth_case) in enumerate(cases):
        if eng is not None:
            del eng, graph
            torch.cuda.empty_cache()
        max_ctx = args.ctx + args.steps + args.warmup + 64
        eng = Engine(model, max_seqs=B_case, max_ctx=max_ctx, prefill_chunk=args.prefill_chunk, max_batch=B_case, use_graph=not args.no_graph)
        torch.cuda.synchronize()
        if case_i == 0:
            t_init = time.time() - t0

        g = torch.Generator().manual_seed(7)
        prompts = [torch.randint(0, cfg.vocab, (args.ctx,), generator=g).tolist() for _ in range(B_case)]
        sids = [eng.create_sequence() for _ in range(B_case)]
        t0 = time.time()
        toks = []
        if synth_case:
            for sid in sids:
                s = eng.seqs[sid]
                eng._ensure_pages(s, args.ctx)
                s.length = args.ctx
                toks.append(1)
        else:
            for sid, p in zip(sids, prompts):
                toks.append(eng.prefill(sid, p))
        torch.cuda.synchronize()
        t_prefill = time.time() - t0
        prefill_tps = B_case * args.ctx / t_prefill if not synth_case else None

        # when resident slots < routed experts, restrict routing to resident experts is NOT done: a miss is counted
        for _ in range(args.warmup):
            toks = eng.decode(sids, toks)

        # ---- timed region 1: public API end to end (H2D inputs + graph + D2H token per step) ----
        sampler = ClockSampler(local)
        sampler.start()
        h2d0, d2h0, l0 = eng.h2d_bytes, eng.d2h_bytes, eng.kernel_launches
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(eng.stream)
        for _ in range(args.steps):
            toks = eng.decode(sids, toks)
        e1.record(eng.stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
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
                # advance the sequence like decode() does, without the host round trip
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
        comm_err = (model.comm.error() or model.comm_amax.error()) if model.comm is not None else 0

        if world > 1:
            t = torch.tensor([dev_ms, e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dev_ms, e2e_ms = float(t[0]), float(t[1])
        if rank == 0:
            value = B_case * args.steps / (dev_ms / 1e3)
            e2e = B_case * args.steps / (e2e_ms / 1e3)
            out = {
                "metric": "decode tok/s @8k ctx" if args.ctx == 8192 else f"decode tok/s @{args.ctx} ctx",
                "value": round(value, 3), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
                "vs_baseline": round(value / BASELINE_DECODE_8K, 3) if (args.model == "glm-5.3-flash" and args.ctx == 8192 and B == 1) else None,
                "dtype": "bf16", "data": "synthetic token ids, random-init weights",
                "config": {"model": cfg.name + "-shape", "global_batch": B, "seq_len": args.ctx,
                           "parallelism": f"tp{world}ep{world}" if world > 1 else "single-gpu",
                           "weights": f"experts {cfg.expert_quant}, attention {cfg.dense_quant}",
                       "kv_cache": "fp8+bf16-rope, 64-token pages" + (f", sharded over the ranks in {args.dcp_chunk}-token chunks" if (world > 1 and args.dcp_chunk > 0) else ""),
                           "l2": "inputs larger than L2 (each step streams ~20 GB of weights)",
                           "resident_expert_slots_per_layer_per_gpu": slots, "routed_experts": cfg.n_routed, "expert_miss_flag": miss, "comm_error_word": comm_err,
                           "collectives": ("fused in-kernel NVLink all-reduce (P2P stores + flags) in the GEMV / tcgen05-GEMM / MoE-combine epilogues, argmax exchange; no NCCL on the step path"
                                           if world > 1 else "none"),
                           "context_fill": "synthetic (uninitialised cache)" if synth_case else "real chunked prefill"},
                "clocks": clocks,
                "e2e": {"value": round(e2e, 3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "gpu_launches": launches,
                **({"extra_case": "second batch size measured in the same process (context marked filled, not prefilled)"} if case_i else {}),
                **({"invalid": f"depth reduced to {args.layers} layers (smoke run)"} if args.layers else {}),
                "extra": {"prefill_tok_s": round(prefill_tps, 1) if prefill_tps else None, "init_s": round(t_init, 1),
                          "weight_gib": round(model.weight_bytes() / 2 ** 30, 2)},
            }
            print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
