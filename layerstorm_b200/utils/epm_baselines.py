"""Baselines over an expert-routing prediction corpus: how well can the target's routing of a drafted position be guessed?

    python -m layerstorm_b200.utils.epm_baselines CORPUS_DIR [--weights CHECKPOINT] [--label] [--holdout 0.25] [--ridge 1.0]
                                                  [--widths 8,16,32] [--out report.json]

``CORPUS_DIR`` holds what ``speculation/epm_corpus.py`` recorded (block records with the draft's per-layer hidden rows, verdicts,
routing records with router logits).  Three guessers, none of them a trained network - the bars a predictor has to clear:

  locality      the experts of an earlier position of the same sequence, per layer.  ``prev``: the position just before (known only
                while the block is being verified - an upper bound on what locality gives); ``block_start``: the last position known
                when the block was drafted (anchor_pos - 1 ... the anchor itself once the target ran it), the same guess for every row
                of the block - the causal variant.
  router probe  the target's own router matrix of layer j applied to the DRAFT's hidden row (after draft layer t, un-normalised):
                if draft and target share a representation, the target's router reads the draft directly.  Every (draft layer t,
                target layer j) pair is scored on the training sequences, the best t per j is reported on the held-out ones.
                Needs ``--weights`` (a checkpoint of the target).
  ridge probe   per target layer a closed-form ridge regression from the draft's hidden row (best draft layer of the router probe,
                else the last) to the target's TRUE router logits, fitted on the training sequences - the best any linear map can do.
Scoring: recall@m = share of the position's routed experts that are among the guess's best m, per (block row, target layer) cell
with its sample count (rows deeper in a block are accepted less often, so cells thin out with depth; empty cells are reported as
such, never averaged in), n-weighted overall; union coverage per block and layer = share of the experts the block's accepted rows
routed that the guesses' top-k together covered (what a prefetch of the union would have hit).  Splits are by SEQUENCE: positions of
one sequence never sit on both sides.
Reference: tools/elb_train/baselines.py (B0 / B1 / B2) and metrics.py (coverage-aware recall, union coverage).
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..speculation import epm_corpus as ec


# ------------------------------------------------------------------------------------------------------------- scoring
class Scores:
    """recall@m per (row, layer) cell and union coverage per (block, layer), with counts."""

    def __init__(self, widths: Sequence[int]):
        self.widths = list(widths)
        self.cell: Dict[Tuple[int, int, int], List[float]] = {}      # (width, row, layer) -> [sum of recalls, n]
        self.missing = 0
        self._union: Dict[Tuple[int, int, int], List[set]] = {}       # (seq, block start, layer) -> [guessed, routed]

    def add(self, ex: dict, layer: int, ranked: Optional[Sequence[int]], k: int):
        true = set(ex["labels"][layer])
        if ranked is None:
            self.missing += 1
            return
        for m in self.widths:
            if m > len(ranked) and m > k:
                continue                                     # the guesser does not rank that deep
            c = self.cell.setdefault((m, ex["row"], layer), [0.0, 0])
            c[0] += len(true & set(ranked[:m])) / max(1, len(true))
            c[1] += 1
        u = self._union.setdefault((ex["seq"], ex["pos"] - ex["row"], layer), [set(), set()])
        u[0] |= set(ranked[:k])
        u[1] |= true

    def report(self) -> dict:
        out: Dict[str, object] = {"missing_predictions": self.missing}
        for m in self.widths:
            cells = {(r, l): c for (w, r, l), c in self.cell.items() if w == m}
            n = sum(c[1] for c in cells.values())
            out[f"recall@{m}"] = {"overall": (sum(c[0] for c in cells.values()) / n) if n else None, "n": n,
                                  "by_row": {str(r): _mean([c for (rr, _), c in cells.items() if rr == r]) for r in sorted({r for r, _ in cells})},
                                  "by_layer": {str(l): _mean([c for (_, ll), c in cells.items() if ll == l]) for l in sorted({l for _, l in cells})}}
        per_layer: Dict[int, List[float]] = {}
        for (_, _, layer), (guess, true) in self._union.items():
            if true:
                per_layer.setdefault(layer, []).append(len(guess & true) / len(true))
        out["union_coverage"] = {"overall": float(np.mean([v for vs in per_layer.values() for v in vs])) if per_layer else None,
                                 "blocks": sum(len(v) for v in per_layer.values()), "by_layer": {str(l): float(np.mean(v)) for l, v in sorted(per_layer.items())}}
        return out


def _mean(cells: List[List[float]]) -> Optional[dict]:
    n = sum(c[1] for c in cells)
    return {"recall": sum(c[0] for c in cells) / n, "n": n} if n else None


def split_by_sequence(examples: Sequence[dict], holdout: float, seed: int = 0) -> Tuple[List[dict], List[dict]]:
    seqs = sorted({e["seq"] for e in examples})
    rng = np.random.default_rng(seed)
    rng.shuffle(seqs)
    n_hold = min(len(seqs) - 1, max(1, int(round(len(seqs) * holdout)))) if len(seqs) > 1 else 0
    held = set(seqs[:n_hold])
    return [e for e in examples if e["seq"] not in held], [e for e in examples if e["seq"] in held]


# ------------------------------------------------------------------------------------------------------------- the guessers
def locality(examples: Sequence[dict], routing: Dict[Tuple[int, int], Dict[int, dict]], variant: str, widths: Sequence[int], k: int) -> dict:
    sc = Scores(widths)
    for ex in examples:
        src_pos = ex["pos"] - 1 if variant == "prev" else ex["pos"] - ex["row"] - 1
        src = routing.get((ex["seq"], src_pos))
        for layer in ex["labels"]:
            row = None if src is None else src.get(layer)
            # the earlier position's experts, best weight first; beyond them the rest of its router logits, best first
            ranked = None
            if row is not None:
                first = [e for _, e in sorted(zip(row["weights"], row["ids"]), reverse=True)]
                rest = [int(e) for e in np.argsort(-row["logits"]) if int(e) not in set(first)]
                ranked = first + rest
            sc.add(ex, layer, ranked, k)
    return sc.report()


def _features(ex: dict, tap: int) -> np.ndarray:
    return ex["features"][tap].float().numpy()


def router_probe(train: Sequence[dict], held: Sequence[dict], routers: Dict[int, Tuple[np.ndarray, Optional[np.ndarray]]], widths: Sequence[int], k: int,
                 score_fn: Callable[[np.ndarray], np.ndarray]) -> Tuple[dict, Dict[int, int]]:
    taps = train[0]["features"].shape[0] if train else (held[0]["features"].shape[0] if held else 0)
    best: Dict[int, int] = {}
    sweep: Dict[str, Dict[str, float]] = {}
    for layer, (W, bias) in routers.items():
        per_tap = []
        for t in range(taps):
            hit = n = 0
            for ex in train:
                if layer not in ex["labels"]:
                    continue
                s = score_fn(_features(ex, t) @ W.T) + (bias if bias is not None else 0.0)
                hit += len(set(np.argsort(-s)[:k].tolist()) & set(ex["labels"][layer]))
                n += len(ex["labels"][layer])
            per_tap.append(hit / n if n else 0.0)
        best[layer] = int(np.argmax(per_tap)) if per_tap else 0          # ties: the earlier draft layer
        sweep[str(layer)] = {str(t): round(v, 4) for t, v in enumerate(per_tap)}
    sc = Scores(widths)
    for ex in held:
        for layer in ex["labels"]:
            if layer not in routers:
                sc.add(ex, layer, None, k)
                continue
            W, bias = routers[layer]
            s = score_fn(_features(ex, best[layer]) @ W.T) + (bias if bias is not None else 0.0)
            sc.add(ex, layer, np.argsort(-s).tolist(), k)
    rep = sc.report()
    rep["train_recall_by_layer_and_draft_layer"] = sweep
    rep["best_draft_layer"] = {str(l): t for l, t in best.items()}
    return rep, best


def ridge_probe(train: Sequence[dict], held: Sequence[dict], taps: Dict[int, int], lam: float, widths: Sequence[int], k: int,
                biases: Optional[Dict[int, np.ndarray]] = None) -> dict:
    layers = sorted({l for e in train for l in e["labels"]})
    last = (train[0]["features"].shape[0] - 1) if train else 0
    maps: Dict[int, np.ndarray] = {}
    for layer in layers:
        t = taps.get(layer, last)
        rows = [e for e in train if layer in e["logits"]]
        if not rows:
            continue
        X = np.stack([np.append(_features(e, t), 1.0) for e in rows]).astype(np.float64)      # a bias column, not penalised
        Y = np.stack([e["logits"][layer] for e in rows]).astype(np.float64)
        reg = lam * np.eye(X.shape[1])
        reg[-1, -1] = 0.0
        maps[layer] = np.linalg.solve(X.T @ X + reg, X.T @ Y)
    sc = Scores(widths)
    for ex in held:
        for layer in ex["labels"]:
            if layer not in maps:
                sc.add(ex, layer, None, k)
                continue
            s = np.append(_features(ex, taps.get(layer, last)), 1.0) @ maps[layer]
            if biases and layer in biases:
                s = _sigmoid(s) + biases[layer]                  # selection as the target does it: biased scores
            sc.add(ex, layer, np.argsort(-s).tolist(), k)
    rep = sc.report()
    rep["ridge"] = lam
    return rep


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def target_routers(weights: dict, layers: Sequence[int]) -> Dict[int, Tuple[np.ndarray, Optional[np.ndarray]]]:
    out = {}
    for l in layers:
        w = weights.get(f"layers.{l}.moe.router")
        if w is not None:
            b = weights.get(f"layers.{l}.moe.router_bias")
            out[l] = (w.float().numpy(), None if b is None else b.float().numpy())
    return out


def evaluate(directory: str, weights: Optional[dict] = None, holdout: float = 0.25, lam: float = 1.0, widths: Sequence[int] = (8, 16, 32),
             sigmoid_scores: bool = True, seed: int = 0) -> dict:
    examples = ec.join_examples(directory)
    if not examples:
        raise ValueError(f"{directory}: no block row has both a verdict and a routing record")
    routing = {(r["seq"], r["pos"]): {x["layer"]: x for x in r["rows"]} for r in ec.read_routing(directory)}
    k = len(next(iter(examples[0]["labels"].values())))
    widths = sorted({min(w, len(next(iter(examples[0]["logits"].values())))) for w in widths} | {k})
    train, held = split_by_sequence(examples, holdout, seed)
    if not held:
        held = train                                              # one sequence only: in-sample numbers, flagged below
    rep = {"corpus": directory, "examples": len(examples), "sequences": len({e["seq"] for e in examples}), "top_k": k,
           "train_examples": len(train), "heldout_examples": len(held), "in_sample": held is train,
           "locality_prev": locality(held, routing, "prev", widths, k), "locality_block_start": locality(held, routing, "block_start", widths, k)}
    taps: Dict[int, int] = {}
    biases = None
    if weights is not None:
        routers = target_routers(weights, sorted({l for e in examples for l in e["labels"]}))
        if routers:
            rep["router_probe"], taps = router_probe(train, held, routers, widths, k, _sigmoid if sigmoid_scores else (lambda x: x))
            biases = {l: b for l, (_, b) in routers.items() if b is not None} if sigmoid_scores else None
    rep["ridge_probe"] = ridge_probe(train, held, taps, lam, widths, k, biases)
    return rep


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("corpus")
    ap.add_argument("--weights", help="checkpoint of the target (for the router probe)")
    ap.add_argument("--holdout", type=float, default=0.25)
    ap.add_argument("--ridge", type=float, default=1.0)
    ap.add_argument("--widths", default="8,16,32")
    ap.add_argument("--out")
    ap.add_argument("--label", action="store_true", help="first write the corpus's routing records by re-running its recorded sequences through the fp32 "
                                                         "reference model of --weights (exact and slow: small targets)")
    a = ap.parse_args(argv)
    weights = None
    if a.weights:
        from ..models.checkpoint import open_checkpoint
        shape, ck = open_checkpoint(a.weights)
        if a.label:
            from ..models.reference import Oracle
            from ..models.weights import init_weights
            names = init_weights(shape, 0).keys()              # the tensor names of the architecture (the labeller is for small targets)
            n = ec.label_with_oracle(a.corpus, Oracle(shape, {k: ck[k].float() if ck[k].is_floating_point() else ck[k] for k in names if k in ck}))
            print(f"labelled {n} positions", file=sys.stderr)
        weights = {}
        for l in range(shape.n_layers):
            for k in (f"layers.{l}.moe.router", f"layers.{l}.moe.router_bias"):
                if k in ck:
                    weights[k] = ck[k]
    elif a.label:
        print("--label needs --weights", file=sys.stderr)
        return 2
    try:
        rep = evaluate(a.corpus, weights, a.holdout, a.ridge, [int(x) for x in a.widths.split(",")])
    except ValueError as e:
        print(str(e), file=sys.stderr)
        return 2
    if a.out:
        json.dump(rep, open(a.out, "w"), indent=1)
    brief = {name: {m: (rep[name][m]["overall"], rep[name][m]["n"]) for m in rep[name] if m.startswith("recall@")} | {"union": rep[name]["union_coverage"]["overall"]}
             for name in ("locality_prev", "locality_block_start", "router_probe", "ridge_probe") if name in rep}
    print(json.dumps({"examples": rep["examples"], "heldout": rep["heldout_examples"], "in_sample": rep["in_sample"], **brief}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
