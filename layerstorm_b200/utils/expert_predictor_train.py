"""Offline training and evaluation of the expert-reuse predictor on recorded routing traces (no GPU).

    python -m layerstorm_b200.utils.expert_predictor_train --traces run1.txt run2.txt ... --out predictor.npz [--held-out 0.2]
        [--lam 1.0] [--lag 1] [--pool 2.0] [--report report.json]
    python -m layerstorm_b200.utils.expert_predictor_train --traces held.txt --evaluate predictor.npz

The predictor (``speculation/expert_ridge.py``) scores, per MoE layer and expert, how likely the expert is to be routed at the next
position from causal features of the routing history; its scores rank prefetch candidates and eviction victims.  Online it learns by
decayed ridge regression while serving; this tool fits the same weights in closed form over whole recorded runs
(``LS_ROUTING_TRACE``), checks them on sequences it has not seen and writes a bundle that ``ExpertRidge.load_weights`` freezes in
(``utils/cache_sim.py --predictor-weights`` replays a cache with it).
  * Split: by SEQUENCE - every trace file is one sequence; the last ``--held-out`` fraction of the files is never trained on (with
    one file, the last fraction of its steps, history reset at the cut).
  * Fit: per layer, w = (sum x x^T + lam I)^-1 sum x y over every (position, expert) of the training sequences; y = routed at that
    position.  No decay: the trained bundle is the stationary solution, the online learner adapts from it when left unfrozen.
  * Metric: recall@m = share of the routed experts that lie inside the m best-scored experts of their layer, m = top_k x {1, 2, 4}
    (the advised pool a prefetcher would load); reported for the trained weights and for three fixed rankings - routed at the previous
    position, fast EMA, slow EMA (a frequency table) - on the held-out sequences only.
Reference: tools/elb_train/ (config-driven trainer of the expert-prediction models on cached features, sequence-level splits, KL /
BCE / MSE arms, baselines, export for the C++ runtime); this is the counterpart for THIS framework's predictor, a closed-form ridge.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..speculation.expert_ridge import N_FEAT, ExpertRidge
from .cache_sim import Trace, read_trace


def to_sequences(traces: Sequence[Trace]) -> Tuple[List[np.ndarray], List[int], int, int]:
    """Every trace -> int array [steps, layers, top_k] (-1 = none); returns (sequences, layer ids, experts, top_k)."""
    layers = sorted({l for tr in traces for _, l, _ in tr})
    lid = {l: i for i, l in enumerate(layers)}
    n_experts = 1 + max((max(ids) for tr in traces for _, _, ids in tr if ids), default=0)
    top_k = max((len(ids) for tr in traces for _, _, ids in tr), default=1)
    seqs = []
    for tr in traces:
        steps = sorted({s for s, _, _ in tr})
        sid = {s: i for i, s in enumerate(steps)}
        a = np.full((len(steps), len(layers), top_k), -1, np.int64)
        for s, l, ids in tr:
            a[sid[s], lid[l], : len(ids)] = ids[:top_k]
        seqs.append(a)
    return seqs, layers, n_experts, top_k


def split_sequences(seqs: List[np.ndarray], held_out: float) -> Tuple[List[np.ndarray], List[np.ndarray]]:
    if len(seqs) >= 2:
        n_held = max(1, int(round(len(seqs) * held_out)))
        return seqs[: len(seqs) - n_held], seqs[len(seqs) - n_held:]
    a = seqs[0]
    cut = max(1, int(len(a) * (1.0 - held_out)))
    return [a[:cut]], [a[cut:]]


def fit(train: List[np.ndarray], n_experts: int, top_k: int, lam: float = 1.0, lag: int = 1) -> ExpertRidge:
    J = train[0].shape[1]
    r = ExpertRidge(J, n_experts, top_k, lag=lag, decay=1.0, lam=lam, refresh=0)
    for a in train:
        r.reset_history()
        for t in range(len(a)):
            r.step(a[t])
    r.solve()
    return r


def _fixed(J: int, n_experts: int, top_k: int, lag: int, feature: int) -> ExpertRidge:
    r = ExpertRidge(J, n_experts, top_k, lag=lag, refresh=0)
    r.w[:] = 0.0
    r.w[:, feature] = 1.0
    if feature == 1:
        r.w[:, 2] = 1e-3                      # ties among the not-routed broken by the fast EMA
    return r


def recall(r: ExpertRidge, seqs: List[np.ndarray], pools: Sequence[int]) -> Dict[int, float]:
    hit = {m: 0 for m in pools}
    seen = 0
    for a in seqs:
        r.reset_history()
        for t in range(len(a)):
            if t > 0:
                s = r.score()
                order = np.argsort(-s, axis=1, kind="stable")
                for j in range(a.shape[1]):
                    ids = a[t, j][a[t, j] >= 0]
                    seen += len(ids)
                    for m in pools:
                        hit[m] += int(np.isin(ids, order[j, :m]).sum())
            r.step(a[t])
    return {m: round(hit[m] / max(seen, 1), 4) for m in pools}


def evaluate(r: ExpertRidge, held: List[np.ndarray], n_experts: int, top_k: int) -> dict:
    pools = [top_k, min(n_experts, 2 * top_k), min(n_experts, 4 * top_k)]
    J = held[0].shape[1]
    frozen = ExpertRidge(J, n_experts, top_k, lag=r.lag, refresh=0, fast=r.fast, slow=r.slow)
    frozen.w[:] = r.w
    out = {"pools": pools, "positions": int(sum(max(0, len(a) - 1) for a in held)), "trained": recall(frozen, held, pools)}
    for name, feat in (("previous_position", 1), ("fast_ema", 2), ("slow_ema_frequency", 3)):
        out[name] = recall(_fixed(J, n_experts, top_k, r.lag, feat), held, pools)
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--traces", nargs="+", required=True)
    ap.add_argument("--out", default=None, help="write the trained bundle here (.npz)")
    ap.add_argument("--evaluate", default=None, help="evaluate this bundle on the traces instead of training")
    ap.add_argument("--held-out", type=float, default=0.2)
    ap.add_argument("--lam", type=float, default=1.0)
    ap.add_argument("--lag", type=int, default=1)
    ap.add_argument("--report", default=None)
    a = ap.parse_args(argv)
    seqs, layers, n_experts, top_k = to_sequences([read_trace(t) for t in a.traces])
    if a.evaluate:
        r = ExpertRidge(len(layers), n_experts, top_k, lag=a.lag)
        r.load_weights(a.evaluate)
        rep = {"mode": "evaluate", "bundle": a.evaluate, "sequences": len(seqs), **evaluate(r, seqs, n_experts, top_k)}
    else:
        train, held = split_sequences(seqs, a.held_out)
        r = fit(train, n_experts, top_k, a.lam, a.lag)
        rep = {"mode": "train", "layers": len(layers), "experts": n_experts, "top_k": top_k, "train_sequences": len(train), "held_out_sequences": len(held),
               "train_positions": int(sum(len(x) for x in train)), "features": ["bias", "prev", "ema_fast", "ema_slow", f"prev_layer-{a.lag}", "recency"],
               "mean_weights": [round(float(x), 4) for x in r.w.mean(0)], "held_out": evaluate(r, held, n_experts, top_k)}
        if a.out:
            r.save_weights(a.out, {"traces": list(a.traces), "lam": a.lam, "held_out": rep["held_out"]})
            rep["out"] = a.out
    if a.report:
        json.dump(rep, open(a.report, "w"), indent=1)
    print(json.dumps(rep))
    return 0


if __name__ == "__main__":
    sys.exit(main())
