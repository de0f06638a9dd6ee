"""Per-kernel timeline of a decode step as it really runs: inside the CUDA graph, with programmatic dependent launch
overlapping neighbouring kernels, on 1..N GPUs.

A profiler serialises launches and flushes caches between them, so its per-kernel times do not add up to the step.  Here
every kernel stamps ``%globaltimer`` itself (``pdl_wait`` in ``csrc/kernels/common.cuh``): when block (0,0,0) reaches its
dependency wait and when the wait returns, i.e. when the previous kernel of the stream has completed.  The difference of
consecutive "wait returned" stamps is what each kernel contributes to the critical path of the step.

    python -m layerstorm_b200.utils.step_trace --model glm-5.3-flash --ctx 8192 --steps 8
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m layerstorm_b200.utils.step_trace --model glm-5.3-flash

Kernel names come from one eager step in which the launcher calls are recorded together with the number of trace records
each of them produced.  Output: a table (launches per step, mean microseconds per launch, microseconds and share per
step, mean time the kernel's first block spent resident before its dependency resolved) and one JSON line.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
from collections import OrderedDict


def install_trace(buf) -> None:
    """Point every translation unit of the kernel library at ``buf`` (int64 tensor: [0] count, [1] capacity, 4 words per record);
    ``None`` switches tracing off."""
    from ..ops import _native as nat
    for name in nat.SIGS:
        if name.startswith("lsb_trace_set_"):
            rc = nat.call(name, buf)
            if rc != 0:
                raise RuntimeError(f"{name} failed with status {rc}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="glm-5.3-flash")
    ap.add_argument("--layers", type=int, default=0, help="keep only the first N layers (0 = the whole model)")
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--prefill", action="store_true", help="compute the context with chunked prefill instead of marking it filled")
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--headroom-gib", type=float, default=4.0)
    ap.add_argument("--expert-shard", default=None, choices=["ep", "tp"])
    ap.add_argument("--by-call", action="store_true", help="aggregate by launcher call only (not by grid shape)")
    ap.add_argument("--sequence", action="store_true", help="also print the kernels of one step in launch order")
    a = ap.parse_args(argv)

    import torch
    import torch.distributed as dist

    from ..models.config import get_preset
    from ..models.device_model import DeviceModel
    from ..ops import _native as nat
    from ..runtime.engine import Engine

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = get_preset(a.model)
    if a.layers and a.layers < cfg.n_layers:
        repl = {"n_layers": a.layers}
        if getattr(cfg, "layer_types", None):
            repl["layer_types"] = list(cfg.layer_types[:a.layers])
        cfg = dataclasses.replace(cfg, **repl)
    model = DeviceModel.random_init(cfg, dev, kv_fmt="fp8", page=64, seed=1234, expert_slots="auto", embed_on_host=True,
                                    reserve_bytes=int(a.headroom_gib * 2 ** 30), tp_rank=rank, tp_size=world, expert_shard=a.expert_shard)
    if world > 1:
        from ..parallel.symm import PeerComm
        model.attach_comm(PeerComm(max(4, a.batch, a.prefill_chunk if a.prefill else 4) * cfg.hidden, dev), PeerComm(2 * max(a.batch, 4), dev))
    eng = Engine(model, max_seqs=a.batch, max_ctx=a.ctx + 2 * a.steps + 80, prefill_chunk=a.prefill_chunk, max_batch=a.batch)
    g = torch.Generator().manual_seed(7)
    sids = [eng.create_sequence() for _ in range(a.batch)]
    toks = []
    for sid in sids:
        if a.prefill:
            toks.append(eng.prefill(sid, torch.randint(0, cfg.vocab, (a.ctx,), generator=g).tolist()))
        else:
            s = eng.seqs[sid]
            eng._ensure_pages(s, a.ctx)
            s.length = a.ctx
            toks.append(1)
    for _ in range(4):                                   # captures the graph, warms the caches
        toks = eng.decode(sids, toks)
    torch.cuda.synchronize()

    cap = 8192
    buf = torch.zeros(2 + 4 * cap, dtype=torch.int64, device=dev)
    buf[1] = cap
    install_trace(buf)

    # ---- pass 1: eager step, launcher names and records per call ----
    names = []
    real_call = nat.call

    def recording_call(name, *args, **kw):
        before = int(buf[0])
        rc = real_call(name, *args, **kw)
        if nat.SIGS[name][1]:
            torch.cuda.synchronize()
            n = int(buf[0]) - before
            names.extend(f"{name}#{j}" if n > 1 else name for j in range(n))
        return rc

    eng.use_graph = False
    nat.call = recording_call
    try:
        toks = eng.decode(sids, toks)
    finally:
        nat.call = real_call
    eng.use_graph = True
    n_kernels = len(names)

    # ---- pass 2: graph replays ----
    torch.cuda.synchronize()
    buf[0] = 0
    step_ms = []
    for _ in range(a.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(eng.stream)
        toks = eng.decode(sids, toks)
        e1.record(eng.stream)
        torch.cuda.synchronize()
        step_ms.append(e0.elapsed_time(e1))
    rec = buf.cpu()
    install_trace(None)
    n_rec = int(rec[0])
    if n_rec != n_kernels * a.steps:
        raise RuntimeError(f"trace has {n_rec} records for {a.steps} steps of {n_kernels} kernels (eager and graph steps differ)")
    r = rec[2: 2 + 4 * n_rec].view(a.steps, n_kernels, 4)
    t0, t1 = r[:, :, 0], r[:, :, 1]
    # critical-path share of kernel k: from its dependency release to the release of kernel k + 1 (the last kernel of a step has no
    # successor inside the step and is left out)
    dt = (t1[:, 1:] - t1[:, :-1]).float() / 1e3          # us, [steps, n_kernels - 1]
    resident = (t1 - t0).float() / 1e3                   # us the first block waited at its dependency (prologue overlap)
    span_ms = float((t1[:, -1] - t1[:, 0]).float().mean()) / 1e6
    agg = OrderedDict()
    for k in range(n_kernels - 1):
        gx, gy = int(r[0, k, 2]) & 0xffffffff, int(r[0, k, 2]) >> 32
        bx, gz = int(r[0, k, 3]) & 0xffffffff, int(r[0, k, 3]) >> 32
        key = names[k] if a.by_call else f"{names[k]} ({gx},{gy},{gz})x{bx}"
        e = agg.setdefault(key, [0, 0.0, 0.0])
        e[0] += 1
        e[1] += float(dt[:, k].mean())
        e[2] += float(resident[:, k].mean())
    if rank == 0:
        tot = sum(e[1] for e in agg.values())
        print(f"# {cfg.name}: {n_kernels} kernels per step, {a.steps} graph replays, batch {a.batch}, context {a.ctx}, {world} GPU(s)")
        print(f"# step {sum(step_ms) / len(step_ms):.3f} ms by CUDA events, first-to-last dependency release {span_ms:.3f} ms")
        print("| kernel (launcher call, grid x block) | launches/step | us/launch | us/step | share | resident before release, us |")
        print("|---|---|---|---|---|---|")
        for key, (n, us, res) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
            print(f"| `{key}` | {n} | {us / n:.2f} | {us:.1f} | {100 * us / tot:.1f}% | {res / n:.1f} |")
        if a.sequence:
            print("# one step in launch order: index, kernel, us to the next release, us resident before release")
            for k in range(n_kernels - 1):
                print(f"{k:4d} {names[k]:<40s} {float(dt[:, k].mean()):8.2f} {float(resident[:, k].mean()):8.2f}")
        print(json.dumps({"model": cfg.name, "n_gpus": world, "batch": a.batch, "ctx": a.ctx, "kernels_per_step": n_kernels,
                          "step_ms_events": round(sum(step_ms) / len(step_ms), 4), "span_ms_trace": round(span_ms, 4),
                          "by_kernel_us_per_step": {k: round(v[1], 2) for k, v in agg.items()}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
