"""Small speculation policies, all pure functions of configuration + observations (no engine calls).

``ThinkTracker`` / ``ReasoningMode``   follow the <think> ... </think> state of a token stream and, while inside a thinking block, return
                                       deeper speculation and a relaxed verification threshold; the first token after the closing tag
                                       gets the base values again.
``PerformanceObjective``               normalised latency / throughput weights and the blended score schedulers rank choices by.
``LayerSkipPolicy``                    which layers a self-speculative draft may skip: layer l+1 is skipped when the residual stream barely
                                       moved across the last ``min_contiguous`` layers (cosine similarity above a threshold) and, with a
                                       product window, when the product of the similarities stays above a second threshold.  The first and
                                       last layers are never skipped; the policy only enables itself while the draft's acceptance holds up.
``SelfSpeculativePlan``                per-layer plan of a reduced-expert draft pass (top-k experts instead of the model's k, skipped layers)
                                       with running acceptance statistics and the early-exit rule on draft confidence.
Reference counterparts: python/orchestrator/reasoning_mode.py + context_annotation.py (think state), performance_objective.py,
layer_skip.py, self_speculative.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Set


# --------------------------------------------------------------------------------------------------------- reasoning
class ThinkTracker:
    """Think-block state over token ids (open / close may each be one id or a sequence of ids)."""

    def __init__(self, open_ids: Sequence[int], close_ids: Sequence[int], starts_thinking: bool = False):
        self.open, self.close = list(open_ids), list(close_ids)
        self.thinking = starts_thinking
        self._tail: List[int] = []
        self.think_tokens = 0

    def feed(self, token: int) -> bool:
        n = max(len(self.open), len(self.close))
        self._tail = (self._tail + [token])[-n:]
        if self.thinking:
            self.think_tokens += 1
            if self.close and self._tail[-len(self.close):] == self.close:
                self.thinking = False
        elif self.open and self._tail[-len(self.open):] == self.open:
            self.thinking = True
        return self.thinking


@dataclass(frozen=True)
class ReasoningOverrides:
    active: bool = False
    depth_multiplier: float = 1.0
    adaptive_topk_threshold: Optional[float] = None
    sparse_verification: Optional[bool] = None


class ReasoningMode:
    def __init__(self, cfg: dict):
        """``cfg`` = the ``speculation.reasoning_mode`` section."""
        self.enabled = bool(cfg.get("enabled", False))
        self.mult = float(cfg.get("aggressive_speculation_depth_multiplier", 2.0))
        self.relaxed = float(cfg.get("relaxed_verification_threshold", 0.85))

    def overrides(self, thinking: bool) -> ReasoningOverrides:
        if not (self.enabled and thinking):
            return ReasoningOverrides()
        return ReasoningOverrides(True, self.mult, self.relaxed, True)

    @staticmethod
    def depth(base_depth: int, ov: ReasoningOverrides) -> int:
        return int(math.floor(base_depth * ov.depth_multiplier))


# --------------------------------------------------------------------------------------------------------- objective
class PerformanceObjective:
    def __init__(self, latency_weight: float = 0.6, throughput_weight: float = 0.4):
        tot = latency_weight + throughput_weight
        self.latency_weight, self.throughput_weight = (0.5, 0.5) if tot == 0 else (latency_weight / tot, throughput_weight / tot)

    @classmethod
    def from_config(cls, cfg: dict) -> "PerformanceObjective":
        po = cfg["orchestrator"]["performance_objective"]
        return cls(po["latency_weight"], po["throughput_weight"])

    def score(self, latency_score: float, throughput_score: float) -> float:
        return self.latency_weight * latency_score + self.throughput_weight * throughput_score

    @property
    def latency_dominant(self) -> bool:
        return self.latency_weight > self.throughput_weight


# --------------------------------------------------------------------------------------------------------- layer skip
def cosine(a, b) -> float:
    import numpy as np
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    return 0.0 if na == 0 or nb == 0 else float(a @ b / (na * nb))


class LayerSkipPolicy:
    def __init__(self, cfg: dict, n_layers: int):
        """``cfg`` = the ``speculation.layer_skip_draft`` section."""
        self.enabled = bool(cfg.get("enabled", False))
        self.thr = float(cfg.get("threshold", 0.995))
        self.first, self.last = int(cfg.get("no_skip_first", 3)), int(cfg.get("no_skip_last", 3))
        self.contig = max(1, int(cfg.get("min_contiguous", 1)))
        self.window, self.prod_thr = int(cfg.get("product_window", 1)), float(cfg.get("product_threshold", 0.985))
        self.min_accept = float(cfg.get("min_acceptance_rate_to_enable", 0.5))
        self.max_fraction = float(cfg.get("target_skip_fraction", 0.5))
        self.L = n_layers

    def skippable(self, layer: int) -> bool:
        return self.first <= layer < self.L - self.last

    def active(self, acceptance_rate: float) -> bool:
        return self.enabled and acceptance_rate >= self.min_accept

    def skip_set(self, similarity: Dict[int, float]) -> Set[int]:
        """``similarity[l]`` = cosine of the residual stream before and after layer l (from the previous draft pass)."""
        out: Set[int] = set()
        budget = int(self.max_fraction * self.L)
        for l in range(self.L - 1):
            cand = l + 1
            if not self.skippable(cand) or len(out) >= budget:
                continue
            run = [similarity.get(l - o) if l - o >= 0 and self.skippable(l - o) else None for o in range(self.contig)]
            if any(s is None or s < self.thr for s in run):
                continue
            if self.window > 1:
                win = [similarity.get(l - o) if l - o >= 0 else None for o in range(self.window)]
                if any(s is None for s in win) or math.prod(win) < self.prod_thr:
                    continue
            out.add(cand)
        return out


# --------------------------------------------------------------------------------------------------------- self-speculative
@dataclass
class LayerPlan:
    layer: int
    skip: bool
    experts: int          # routed experts to run in this layer (0 for dense layers)


class SelfSpeculativePlan:
    def __init__(self, cfg: dict, moe_layers: Iterable[int], n_layers: int, model_top_k: int, max_depth: int = 4):
        """``cfg`` = the ``speculation.self_speculative`` section."""
        self.enabled = bool(cfg.get("enabled", True))
        self.k = max(1, min(int(cfg.get("draft_expert_count", 1)), model_top_k))
        self.adaptive_exit = bool(cfg.get("adaptive_exit_enabled", True))
        self.conf_thr = float(cfg.get("draft_confidence_threshold", 0.4))
        self.moe, self.L, self.max_depth = set(moe_layers), n_layers, max_depth
        self.drafts = self.steps = self.accepted = 0

    def plan(self, skip: Optional[Set[int]] = None) -> List[LayerPlan]:
        skip = skip or set()
        return [LayerPlan(l, l in skip, self.k if l in self.moe and l not in skip else 0) for l in range(self.L)]

    def expert_fraction(self, model_top_k: int, skip: Optional[Set[int]] = None) -> float:
        """Routed-expert work of a draft pass relative to a full pass."""
        p = self.plan(skip)
        return sum(x.experts for x in p) / max(1, model_top_k * len(self.moe))

    def should_continue(self, depth: int, confidence: float) -> bool:
        if depth >= self.max_depth:
            return False
        return not self.adaptive_exit or confidence >= self.conf_thr

    def record(self, drafted: int, accepted: int):
        self.drafts += 1
        self.steps += drafted
        self.accepted += accepted

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.steps if self.steps else 0.0


# --------------------------------------------------------------------------------------------------------- MTP planner
@dataclass
class MtpStep:
    step: int
    layer: int            # index of the MTP block to run: n_layers + step % n_mtp_layers (blocks are reused cyclically)
    input_token: int      # -1: the token sampled by the previous step


class MtpDraftPlanner:
    """Planner of a multi-token-prediction draft: which MTP block each draft step runs, when to stop, acceptance statistics.
    Step k combines the previous hidden state with the embedding of token k, runs MTP block ``k % n_mtp`` and the shared output head.
    Reference: python/orchestrator/mtp_draft.py (cyclic block reuse, dynamic depth gating on draft confidence, acceptance tracking)."""

    def __init__(self, cfg: dict, n_layers: int, n_mtp_layers: int):
        """``cfg`` = the ``speculation.mtp`` section."""
        self.enabled = bool(cfg.get("enabled", True)) and n_mtp_layers > 0
        self.max_depth = int(cfg.get("max_depth", 3))
        self.dynamic = bool(cfg.get("dynamic_depth", True))
        self.conf_thr = float(cfg.get("confidence_threshold", 0.4))
        self.batched_verify = bool(cfg.get("batched_verify", True))
        self.L, self.M = n_layers, n_mtp_layers
        self.drafts = self.steps = self.accepted = 0

    def layer_of(self, step: int) -> int:
        return self.L + step % self.M

    def plan(self, first_token: int, depth: Optional[int] = None) -> List[MtpStep]:
        if not self.enabled:
            return []
        d = self.max_depth if depth is None else min(depth, self.max_depth)
        return [MtpStep(k, self.layer_of(k), first_token if k == 0 else -1) for k in range(d)]

    def should_continue(self, step: int, confidence: float) -> bool:
        if step + 1 >= self.max_depth:
            return False
        return not self.dynamic or confidence >= self.conf_thr

    def record(self, drafted: int, accepted: int):
        self.drafts += 1
        self.steps += drafted
        self.accepted += accepted

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.steps if self.steps else 0.0
