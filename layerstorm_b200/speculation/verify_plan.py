"""Verification transfer planning from a draft's gating, and Sequential Temperature Scaling of draft confidences.

``plan_verification``: a speculative draft that runs the target's routers (self-speculative or layer-sharing drafts)
knows, per drafted position and MoE layer, the gating weights the verification pass is likely to see.  From them:
  1. adaptive top-k per (position, layer): keep experts by descending weight until the cumulative weight reaches a threshold;
  2. union over positions; drop experts already resident in the HBM cache;
  3. order the missing ones by (first position that needs them, layer) - the verification pass walks layers for all rows
     at once, so an expert needed by the first drafted positions matters for every accepted prefix;
  4. the deepest position whose experts are all resident by the time verification starts + its per-layer progress,
     under a single-stream bandwidth model, is the verifiable depth.
``fit_sts_temperatures``: one temperature per draft position, fitted left to right on recorded (confidences, accepted
length) rounds so that the cumulative-product survival estimate is calibrated (1-D grid search on the expected calibration
error, earlier temperatures held fixed).  The temperature acts on the logit, so rankings within a position never change.
Reference counterparts: python/orchestrator/speculative_prefetch.py (SP-MoE plan: adaptive top-K, union, schedule,
max depth) and python/orchestrator/dspark_calibration.py (STS fit over recorded rounds).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Set, Tuple

import numpy as np


def adaptive_topk(weights: np.ndarray, threshold: float, k_max: int) -> List[int]:
    order = np.argsort(-weights)[:k_max]
    tot = float(weights[order].sum())
    if tot <= 0:
        return []
    out, acc = [], 0.0
    for e in order:
        out.append(int(e))
        acc += float(weights[e]) / tot
        if acc >= threshold:
            break
    return out


@dataclass
class VerificationPlan:
    required: Dict[int, Set[Tuple[int, int]]]                 # position -> {(layer, expert)}
    transfers: List[Tuple[int, int]]                          # missing (layer, expert) in issue order
    max_depth: int                                            # drafted positions worth verifying now
    eta_ms: Dict[Tuple[int, int], float] = field(default_factory=dict)


def plan_verification(gating: Dict[Tuple[int, int], np.ndarray], resident: Set[Tuple[int, int]], slot_bytes: int, bandwidth_gbs: float,
                      layer_ms: float, threshold: float = 0.92, k_max: int = 8, start_ms: float = 0.0) -> VerificationPlan:
    """``gating[(position, layer)]`` = weight vector over the experts.  ``layer_ms``: time the verification pass spends per layer, so
    layer j starts at ``start_ms + j_rank * layer_ms`` (j_rank = its order among the planned layers)."""
    required: Dict[int, Set[Tuple[int, int]]] = {}
    first_need: Dict[Tuple[int, int], int] = {}
    for (pos, layer), w in sorted(gating.items()):
        for e in adaptive_topk(np.asarray(w, np.float64), threshold, k_max):
            required.setdefault(pos, set()).add((layer, e))
            first_need.setdefault((layer, e), pos)
    missing = [k for k in first_need if k not in resident]
    missing.sort(key=lambda k: (first_need[k], k[0], k[1]))
    per_ms = slot_bytes / (bandwidth_gbs * 1e6) if bandwidth_gbs > 0 else float("inf")
    eta = {k: (i + 1) * per_ms for i, k in enumerate(missing)}
    layers = sorted({l for (_, l) in gating})
    start_of = {l: start_ms + i * layer_ms for i, l in enumerate(layers)}
    depth = 0
    for pos in sorted(required):
        if pos != depth:
            break                                              # positions must be contiguous from 0
        if all(k in resident or eta[k] <= start_of[k[0]] for k in required[pos]):
            depth += 1
        else:
            break
    return VerificationPlan(required, missing, depth, eta)


# ---------------------------------------------------------------------------------------------------------------- STS
def _logit(c):
    c = np.clip(c, 1e-6, 1 - 1e-6)
    return np.log(c / (1 - c))


def apply_temperature(c, T: float):
    return 1.0 / (1.0 + np.exp(-_logit(np.asarray(c, np.float64)) / T))


def expected_calibration_error(pred: np.ndarray, label: np.ndarray, bins: int = 10) -> float:
    pred, label = np.asarray(pred, np.float64), np.asarray(label, np.float64)
    if pred.size == 0:
        return 0.0
    idx = np.minimum((pred * bins).astype(int), bins - 1)
    ece = 0.0
    for b in range(bins):
        m = idx == b
        if m.any():
            ece += m.mean() * abs(pred[m].mean() - label[m].mean())
    return float(ece)


def fit_sts_temperatures(rounds: Sequence[Tuple[Sequence[float], int]], gamma: int, grid: Sequence[float] = tuple(np.geomspace(0.25, 4.0, 33))) -> List[float]:
    """``rounds``: (per-position confidences c_0..c_{g-1}, accepted prefix length).  Returns ``gamma`` temperatures."""
    rows = [(np.asarray(c, np.float64), int(a)) for c, a in rounds if len(c) > 0]
    temps: List[float] = []
    for k in range(gamma):
        use = [(c, a) for c, a in rows if len(c) > k]
        if not use:
            temps.append(1.0)
            continue
        label = np.array([1.0 if a > k else 0.0 for _, a in use])
        prefix = np.array([np.prod([apply_temperature(c[i], temps[i]) for i in range(k)]) if k else 1.0 for c, _ in use])
        ck = np.array([c[k] for c, _ in use])
        best, best_T = None, 1.0
        for T in grid:
            e = expected_calibration_error(prefix * apply_temperature(ck, T), label)
            if best is None or e < best - 1e-12 or (abs(e - best) <= 1e-12 and abs(np.log(T)) < abs(np.log(best_T))):
                best, best_T = e, float(T)
        temps.append(best_T)
    return temps


def cumulative_survival_ece(rounds, temps: Sequence[float]) -> List[float]:
    out = []
    for k in range(len(temps)):
        use = [(np.asarray(c, np.float64), a) for c, a in rounds if len(c) > k]
        pred = np.array([np.prod([apply_temperature(c[i], temps[i]) for i in range(k + 1)]) for c, _ in use])
        label = np.array([1.0 if a > k else 0.0 for _, a in use])
        out.append(expected_calibration_error(pred, label))
    return out


# ---------------------------------------------------------------------------------------------------------------- coverage
@dataclass
class CoverageReport:
    per_position_min: List[float]            # lowest per-layer coverage of each drafted position
    per_position_mode: List[int]             # 0 = every selected expert resident, 1 = some missing (fetch before verifying)
    depth: int                               # longest prefix whose every layer meets the floor
    truncation_reason: str = ""


def coverage_depth(draft_gating: np.ndarray, resident: Set[Tuple[int, int]], moe_layers: Sequence[int], floor: float = 0.85,
                   threshold: float = 0.92, k_max: int = 8) -> CoverageReport:
    """Residency coverage of a drafted block: ``draft_gating`` is [positions, moe layers, experts].  Coverage of (position, layer) =
    gating weight of the selected experts that are resident / weight of all selected experts.  The verification pass of this engine
    always runs every selected expert (missing ones are fetched first), so the depth is advice on how much of the draft can be verified
    WITHOUT waiting for transfers, not a licence to mask experts.
    Reference: python/orchestrator/verifier.py (analyze_moe_coverage / compute_verifiable_depth with the verification quality floor)."""
    g = np.asarray(draft_gating, np.float64)
    mins, modes, depth, reason, open_ = [], [], 0, "", True
    for d in range(g.shape[0]):
        lo, mode = 1.0, 0
        for m, layer in enumerate(moe_layers):
            sel = adaptive_topk(g[d, m], threshold, k_max)
            tot = sum(g[d, m, e] for e in sel)
            res = sum(g[d, m, e] for e in sel if (layer, e) in resident)
            cov = res / tot if tot > 0 else 0.0
            if cov < 1.0:
                mode = 1
            if cov < lo:
                lo = cov
                if cov < floor and open_ and not reason:
                    reason = f"coverage {cov:.2f} below floor at position {d}, layer {layer}"
        mins.append(lo)
        modes.append(mode)
        if open_ and lo >= floor:
            depth += 1
        else:
            open_ = False
    return CoverageReport(mins, modes, depth, reason if depth < g.shape[0] else "")
