"""Trace analysers of the expert loader: fetch-frequency table, copy cost-model fit, eviction-policy fit (no GPU).

    python -m layerstorm_b200.utils.loader_xray freq-table OUT.csv ROUTING.txt [ROUTING2.txt ...] --slots 64 [--skip-steps 3]
    python -m layerstorm_b200.utils.loader_xray fit-constants FETCH.txt [FETCH2.txt ...] [--out loader_constants_trained.json]
    python -m layerstorm_b200.utils.loader_xray fit-policy ROUTING.txt --slots 64 [--out policy_params.json] [--grid coarse|fine]

Inputs are what a serving or benchmark run with a capped expert cache leaves behind: ``LS_ROUTING_TRACE`` (which experts every MoE
layer routed, step by step) and ``LS_FETCH_TRACE`` (one line per batch of host->device expert copies: copies, bytes, device time).

``freq-table``  replays the routing through the real cache bookkeeping (``utils/cache_sim.simulate``) and counts DEMAND FETCHES per
    (layer, expert) - not routing frequency: an expert that is hot in HBM routes often but is fetched rarely, and placement wants the
    bytes on the wire.  The first ``--skip-steps`` steps (cold cache) are left out; several traces accumulate.  Output CSV
    ``layer,expert,count`` with a provenance header, read by ``ExpertStreamer(place_freq=...)`` / ``LS_ARENA_PLACE_FREQ`` to choose the
    experts that start resident; the concentration profile (share of fetches covered by the top-K keys) is printed.
``fit-constants``  least squares of  device_us = overhead_us + bytes / bandwidth  over the copy batches, per-batch residuals (p50 /
    p90 / max), R^2, and the same against a calibration's prediction when ``--calib-gbs`` is given (scale + offset correction).
    Writes ``{"h2d_gb_s", "batch_overhead_us", ...}``.
``fit-policy``  the weights of the cache's eviction score are not regressed (the objective is a closed loop): a grid over the seven
    weights is replayed through the cache simulation and ranked by hit rate; plain LRU and LFU are the baselines.  Writes the best
    ``memory.expert_cache`` section.  The replay is open-loop (it cannot see a changed trajectory); a run on the GPU stays the gate.
Reference: tools/loader_xray/{freq_table,analyze,trainer}.py and tools/loader_fit/deploy_fit.py (one driver, each parameter class
by its own method: regression for constants, black-box search through the offline simulation for policy weights).
"""
from __future__ import annotations

import argparse
import io
import itertools
import json
import sys
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .cache_sim import read_trace, simulate

WEIGHT_FIELDS = ("alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta")


# ------------------------------------------------------------------------------------------------------------- freq-table
def fetch_counts(traces: Sequence[list], slots: int, policy: str = "impact_weighted_lru", weights: Optional[Sequence[float]] = None,
                 skip_steps: int = 3) -> Dict[Tuple[int, int], int]:
    """Demand fetches per (layer, expert) when the routing traces are replayed through a cache of ``slots`` per layer."""
    counts: Dict[Tuple[int, int], int] = {}
    for tr in traces:
        if not tr:
            continue
        first = min(s for s, _, _ in tr)
        buf = io.StringIO()
        simulate(tr, slots, policy, weights, decisions=buf)
        for line in buf.getvalue().splitlines():
            p = line.split()
            if p and p[0] == "M" and int(p[1]) - first >= skip_steps:
                k = (int(p[2]), int(p[3]))
                counts[k] = counts.get(k, 0) + 1
    return counts


def concentration(counts: Dict[Tuple[int, int], int], ks=(16, 64, 256, 1024, 4096)) -> Dict[str, float]:
    v = np.sort(np.array(list(counts.values()), dtype=np.float64))[::-1]
    tot = max(1.0, float(v.sum()))
    return {f"top_{k}": round(float(v[:k].sum()) / tot, 4) for k in ks if k <= max(len(v), 1) * 4}


def write_freq_table(path: str, counts: Dict[Tuple[int, int], int], provenance: str):
    with open(path, "w") as fh:
        fh.write(f"# demand fetches per (layer, expert); {provenance}\n# layer,expert,count\n")
        for (l, e), c in sorted(counts.items(), key=lambda kv: (-kv[1], kv[0])):
            fh.write(f"{l},{e},{c}\n")


def read_freq_table(path: str) -> Dict[Tuple[int, int], int]:
    out: Dict[Tuple[int, int], int] = {}
    with open(path) as fh:
        for line in fh:
            line = line.split("#", 1)[0].strip()
            if line:
                l, e, c = line.split(",")[:3]
                out[(int(l), int(e))] = int(float(c))
    return out


# ------------------------------------------------------------------------------------------------------------- fit-constants
def read_fetch_trace(path: str) -> np.ndarray:
    """[n, 3] (copies, bytes, device_us) of the copy batches."""
    rows = []
    with open(path) as fh:
        for line in fh:
            p = line.split("#", 1)[0].split()
            if len(p) >= 5 and p[0] == "W":
                rows.append((float(p[2]), float(p[3]), float(p[4])))
    return np.array(rows, dtype=np.float64).reshape(-1, 3)


def _lsq(x: np.ndarray, y: np.ndarray) -> Tuple[float, float, float]:
    """y ~ a + b x: (a, b, R^2)."""
    A = np.stack([np.ones_like(x), x], 1)
    (a, b), *_ = np.linalg.lstsq(A, y, rcond=None)
    res = y - (a + b * x)
    ss = float(((y - y.mean()) ** 2).sum())
    return float(a), float(b), (1.0 - float((res ** 2).sum()) / ss) if ss > 0 else 1.0


def fit_constants(batches: np.ndarray, calib_gbs: Optional[float] = None) -> dict:
    if len(batches) < 2:
        raise ValueError("need at least two copy batches")
    nbytes, us = batches[:, 1], batches[:, 2]
    a, b, r2 = _lsq(nbytes, us)
    res = np.abs(us - (a + b * nbytes))
    out = {"batches": int(len(batches)), "bytes_total": int(nbytes.sum()), "h2d_gb_s": round(1e-3 / b, 2) if b > 0 else None,
           "batch_overhead_us": round(a, 1), "r2": round(r2, 4),
           "abs_residual_us": {"p50": round(float(np.percentile(res, 50)), 1), "p90": round(float(np.percentile(res, 90)), 1), "max": round(float(res.max()), 1)},
           "mean_gb_s_observed": round(float(nbytes.sum() / us.sum()) * 1e-3, 2)}
    if calib_gbs:
        pred = nbytes / (calib_gbs * 1e3)                               # us predicted by the calibration's bandwidth alone
        off, scale, r2c = _lsq(pred, us)
        out["against_calibration"] = {"calib_gb_s": calib_gbs, "bias_us": round(float((us - pred).mean()), 1), "scale": round(scale, 3),
                                      "offset_us": round(off, 1), "r2": round(r2c, 4)}
    return out


# ------------------------------------------------------------------------------------------------------------- fit-policy
def policy_grid(kind: str = "coarse") -> List[List[float]]:
    """Weight vectors (alpha .. eta) to replay: recency / frequency / impact mixes, with and without the slower terms."""
    lv = (0.0, 0.5, 1.0) if kind == "coarse" else (0.0, 0.25, 0.5, 0.75, 1.0)
    out = []
    for a, b, c in itertools.product(lv, repeat=3):
        if a + b + c == 0:
            continue
        s = a + b + c
        out.append([a / s, b / s, c / s, 0.0, 0.0, 0.0, 0.0])
    for d in ((0.1, 0.0, 0.0, 0.0), (0.0, 0.1, 0.0, 0.0), (0.0, 0.0, 0.1, 0.0), (0.0, 0.0, 0.0, 0.1)):
        out.append([0.4, 0.35, 0.25 - 0.1, *d])
    uniq = []
    for w in out:
        w = [round(x, 4) for x in w]
        if w not in uniq:
            uniq.append(w)
    return uniq


def fit_policy(trace: list, slots: int, grid: str = "coarse", slot_bytes: int = 18 << 20) -> dict:
    base = {p: simulate(trace, slots, p, slot_bytes=slot_bytes)["hit_rate"] for p in ("lru", "lfu")}
    ranked = []
    for w in policy_grid(grid):
        r = simulate(trace, slots, "impact_weighted_lru", w, slot_bytes=slot_bytes)
        ranked.append((r["hit_rate"], w, r["demand_miss_bytes"]))
    ranked.sort(key=lambda t: (-t[0], t[1]))
    hit, w, miss_bytes = ranked[0]
    best_base = max(base, key=base.get)
    section = {"eviction_policy": "impact_weighted_lru", **{k: v for k, v in zip(WEIGHT_FIELDS, w)}}
    if base[best_base] >= hit:
        section = {"eviction_policy": best_base}
    return {"slots_per_layer": slots, "grid": grid, "candidates": len(ranked), "baselines": base, "best_weighted": {"hit_rate": hit, "weights": w, "demand_miss_bytes": miss_bytes},
            "top5": [{"hit_rate": h, "weights": ww} for h, ww, _ in ranked[:5]], "memory.expert_cache": section,
            "note": "open-loop replay of a recorded routing; confirm on the GPU (streaming_bench / serve with LS_ROUTING_TRACE) before deploying"}


# ------------------------------------------------------------------------------------------------------------- CLI
def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    f = sub.add_parser("freq-table")
    f.add_argument("out")
    f.add_argument("traces", nargs="+")
    f.add_argument("--slots", type=int, required=True)
    f.add_argument("--policy", default="impact_weighted_lru")
    f.add_argument("--skip-steps", type=int, default=3)
    c = sub.add_parser("fit-constants")
    c.add_argument("traces", nargs="+")
    c.add_argument("--calib-gbs", type=float, default=None, help="bandwidth the calibration predicted, for the scale / offset correction")
    c.add_argument("--out", default=None)
    p = sub.add_parser("fit-policy")
    p.add_argument("trace")
    p.add_argument("--slots", type=int, required=True)
    p.add_argument("--grid", default="coarse", choices=["coarse", "fine"])
    p.add_argument("--slot-mib", type=float, default=18.0)
    p.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    if a.cmd == "freq-table":
        counts = fetch_counts([read_trace(t) for t in a.traces], a.slots, a.policy, skip_steps=a.skip_steps)
        write_freq_table(a.out, counts, f"slots={a.slots} policy={a.policy} skip_steps={a.skip_steps} traces={','.join(a.traces)}")
        rep = {"keys": len(counts), "fetches": int(sum(counts.values())), "concentration": concentration(counts), "out": a.out}
    elif a.cmd == "fit-constants":
        rep = fit_constants(np.concatenate([read_fetch_trace(t) for t in a.traces], 0), a.calib_gbs)
        if a.out:
            json.dump(rep, open(a.out, "w"), indent=1)
    else:
        rep = fit_policy(read_trace(a.trace), a.slots, a.grid, int(a.slot_mib * (1 << 20)))
        if a.out:
            json.dump(rep, open(a.out, "w"), indent=1)
    print(json.dumps(rep))
    return 0


if __name__ == "__main__":
    sys.exit(main())
