"""Offline replay of the expert-cache decision stack on a recorded routing trace (no GPU).

Replays which experts every MoE layer routed, step by step, through the REAL native cache bookkeeping
(``csrc/runtime/expert_cache.cpp``: reserve / lock / touch / pick_victim with the configured eviction policy and weights) and,
optionally, the advisory reuse predictor (``speculation/expert_ridge.py``) as a prefetcher with a per-step byte budget.  Reports hit
rate, host->device bytes, demand misses per step and - with ``--decisions`` - the eviction stream, so that a cache size, an eviction
policy or prefetch budget can be chosen from a trace instead of GPU experiments.

Trace: text, one line per (step, layer):  ``<step> <layer> <expert> <expert> ...``  (``#`` starts a comment).  ``write_trace`` writes
one; ``synthetic_trace`` makes a Zipf-distributed one with temporal locality for tests and dry runs.

    python -m layerstorm_b200.utils.cache_sim --trace routing.txt --slots 64 --policy impact_weighted_lru \
        --weights 0.4,0.35,0.25,0,0,0,0 --prefetch-budget 4 --slot-mib 18 [--decisions out.txt]

Reference counterpart: tools/reef_sim/reef_sim.cpp (offline replay of the real loader decision stack on a recorded engine trace,
CUDA-free), in spirit: this replays THIS framework's cache / eviction / prefetch decisions.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, Iterable, List, Optional, Sequence, TextIO, Tuple

import numpy as np

Trace = List[Tuple[int, int, List[int]]]          # (step, layer, experts)


def read_trace(path: str) -> Trace:
    out: Trace = []
    with open(path) as fh:
        for line in fh:
            line = line.split("#", 1)[0].split()
            if len(line) >= 2:
                out.append((int(line[0]), int(line[1]), [int(x) for x in line[2:]]))
    return out


def write_trace(path: str, trace: Iterable[Tuple[int, int, Sequence[int]]]):
    with open(path, "w") as fh:
        fh.write("# step layer experts...\n")
        for step, layer, ids in trace:
            fh.write(f"{step} {layer} {' '.join(str(int(e)) for e in ids)}\n")


def synthetic_trace(steps: int, layers: int, n_experts: int, top_k: int, zipf: float = 1.1, stickiness: float = 0.5, seed: int = 0) -> Trace:
    """Zipf popularity per layer (own permutation each) + temporal locality: each routed expert is kept for the next step with
    probability ``stickiness``."""
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, n_experts + 1) ** zipf
    p /= p.sum()
    perms = [rng.permutation(n_experts) for _ in range(layers)]
    prev: Dict[int, List[int]] = {}
    out: Trace = []
    for s in range(steps):
        for l in range(layers):
            keep = [e for e in prev.get(l, []) if rng.random() < stickiness]
            ids = list(dict.fromkeys(keep))
            while len(ids) < top_k:
                e = int(perms[l][rng.choice(n_experts, p=p)])
                if e not in ids:
                    ids.append(e)
            prev[l] = ids[:top_k]
            out.append((s, l, prev[l]))
    return out


def simulate(trace: Trace, slots: int, policy: str = "impact_weighted_lru", weights: Optional[Sequence[float]] = None, prefetch_budget: int = 0,
             slot_bytes: int = 18 << 20, n_experts: Optional[int] = None, top_k: Optional[int] = None, decisions: Optional[TextIO] = None,
             predictor_weights: Optional[str] = None, h2d_gbs: float = 0.0, cpu_expert_ms: float = 0.0) -> dict:
    from ..runtime import native as rt
    layers = sorted({l for _, l, _ in trace})
    lid = {l: i for i, l in enumerate(layers)}
    n_experts = n_experts or 1 + max((max(ids) for _, _, ids in trace if ids), default=0)
    top_k = top_k or max(len(ids) for _, _, ids in trace)
    caches = {l: rt.ExpertCache(0, slots, policy) for l in layers}
    if weights is not None:
        for c in caches.values():
            c.set_weights(policy, weights)
    ridge = None
    if prefetch_budget > 0:
        from ..speculation.expert_ridge import ExpertRidge
        ridge = ExpertRidge(len(layers), n_experts, top_k)
        if predictor_weights:
            ridge.load_weights(predictor_weights)          # a trained bundle (utils/expert_predictor_train.py), frozen
    hits = misses = prefetched = useful_prefetch = evictions = 0
    per_step_miss: Dict[int, int] = {}
    per_layer_step_miss: Dict[Tuple[int, int], int] = {}      # (step, layer) -> demand misses: the exposed copies of that layer
    pending_prefetch: Dict[int, set] = {l: set() for l in layers}
    routed_now = np.full((len(layers), top_k), -1, np.int64)
    last_step = None

    def admit(l, cache, e) -> bool:
        nonlocal evictions
        try:
            cache.reserve(l, e, rt.ZONE_STREAMING, True)
        except rt.NativeError:
            v = cache.pick_victim(-1)
            if v is None:
                return False
            cache.evict(v[1], v[2])
            evictions += 1
            if decisions:
                decisions.write(f"E {l} {v[2]} for {e}\n")
            cache.reserve(l, e, rt.ZONE_STREAMING, True)
        cache.mark_ready(l, e)
        return True

    def close_step():
        nonlocal prefetched
        if ridge is None:
            return
        ridge.step(routed_now)
        routed_now[:] = -1
        pool = ridge.pool(min(n_experts, top_k + prefetch_budget))
        for l in layers:
            cache, n = caches[l], 0
            for e in pool[lid[l]]:
                if n >= prefetch_budget:
                    break
                if cache.lookup(l, int(e)) < 0 and admit(l, cache, int(e)):
                    pending_prefetch[l].add(int(e))
                    prefetched += 1
                    n += 1

    for step, l, ids in trace:
        if last_step is not None and step != last_step:
            close_step()
        last_step = step
        cache = caches[l]
        # a step that needs more experts than the layer has slots (a prefill chunk) runs in waves, as the streamer does: at most
        # ``slots`` experts are locked at a time, the next wave may evict the previous one's
        for w0 in range(0, max(len(ids), 1), slots):
            locked = []
            for e in ids[w0: w0 + slots]:
                if cache.is_ready(l, e):
                    hits += 1
                    if e in pending_prefetch[l]:
                        useful_prefetch += 1
                else:
                    misses += 1
                    per_step_miss[step] = per_step_miss.get(step, 0) + 1
                    per_layer_step_miss[(step, l)] = per_layer_step_miss.get((step, l), 0) + 1
                    if not admit(l, cache, e):
                        raise RuntimeError(f"layer {l}: no slot of {slots} can be freed")
                    if decisions:
                        decisions.write(f"M {step} {l} {e}\n")
                pending_prefetch[l].discard(e)
                cache.lock(l, e)
                locked.append(e)
            for e in locked:
                cache.touch(l, e, 1.0 / max(len(ids), 1))
                cache.unlock(l, e)
        cache.end_step()
        if ridge is not None:
            routed_now[lid[l], : len(ids)] = ids[:top_k]
    tot = max(1, hits + misses)
    steps = len({s for s, _, _ in trace})
    projected = None
    if h2d_gbs > 0:
        # exposed copy time per step: a layer's demand misses are copied while the layer waits for them (prefetched experts are not
        # counted: their copies overlap other work).  With host expert kernels (cpu_expert_ms per expert and row) the m misses of a
        # layer are split so that the copy engine and the host finish together: min over n of max(n c, (m - n) f).
        f_ms = slot_bytes / (h2d_gbs * 1e6)
        copy_ms = sum(m * f_ms for m in per_layer_step_miss.values()) / max(steps, 1)
        projected = {"h2d_gb_s": h2d_gbs, "copy_ms_per_expert": round(f_ms, 4), "exposed_copy_ms_per_step": round(copy_ms, 3)}
        if cpu_expert_ms > 0:
            c = cpu_expert_ms
            split = sum(min(max(n * c, (m - n) * f_ms) for n in range(m + 1)) for m in per_layer_step_miss.values()) / max(steps, 1)
            projected.update({"cpu_expert_ms": c, "with_cpu_offload_ms_per_step": round(split, 3)})
    return {**({"projected": projected} if projected else {}), "steps": steps, "layers": len(layers), "slots_per_layer": slots, "policy": policy, "hits": hits, "misses": misses,
            "hit_rate": round(hits / tot, 4), "evictions": evictions, "prefetched": prefetched, "useful_prefetch": useful_prefetch,
            "h2d_bytes": (misses + prefetched) * slot_bytes, "demand_miss_bytes": misses * slot_bytes,
            "max_misses_in_a_step": max(per_step_miss.values(), default=0), "mean_misses_per_step": round(misses / max(steps, 1), 3)}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--trace", help="routing trace; omit for a synthetic one")
    ap.add_argument("--slots", type=int, required=True, help="expert slots per layer")
    ap.add_argument("--policy", default="impact_weighted_lru", choices=["impact_weighted_lru", "lru", "lfu"])
    ap.add_argument("--weights", help="seven comma-separated score weights (alpha .. eta)")
    ap.add_argument("--prefetch-budget", type=int, default=0, help="experts prefetched per layer and step from the reuse predictor")
    ap.add_argument("--slot-mib", type=float, default=18.0)
    ap.add_argument("--h2d-gbs", type=float, default=0.0, help="host->device rate: adds the projected exposed copy time per step")
    ap.add_argument("--cpu-expert-ms", type=float, default=0.0, help="host time of one expert for one row: adds the projection with CPU offload of misses")
    ap.add_argument("--predictor-weights", help="trained reuse-predictor bundle (.npz) for the prefetcher instead of online learning")
    ap.add_argument("--decisions", help="write the miss / eviction stream here")
    ap.add_argument("--synthetic", default="256,8,64,8", help="steps,layers,experts,top_k of the synthetic trace")
    a = ap.parse_args(argv)
    if a.trace:
        trace, ne, k = read_trace(a.trace), None, None
    else:
        s, l, ne, k = (int(x) for x in a.synthetic.split(","))
        trace = synthetic_trace(s, l, ne, k)
    w = [float(x) for x in a.weights.split(",")] if a.weights else None
    if w is not None and len(w) != 7:
        ap.error("--weights needs seven values")
    dec = open(a.decisions, "w") if a.decisions else None
    try:
        rep = simulate(trace, a.slots, a.policy, w, a.prefetch_budget, int(a.slot_mib * (1 << 20)), ne, k, dec, a.predictor_weights, a.h2d_gbs, a.cpu_expert_ms)
    finally:
        if dec:
            dec.close()
    print(json.dumps(rep))
    return 0


if __name__ == "__main__":
    sys.exit(main())
