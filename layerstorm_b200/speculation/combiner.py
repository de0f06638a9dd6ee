"""Choosing between draft sources and sizing the draft depth.

``DraftCombiner``   asks the cheap source first (prompt lookup), falls back to the model draft; sources carry
                    a priority boost and a compute cost, the combiner keeps the proposal with the best
                    expected accepted tokens per unit cost.
``UtilityScorer``   expected speed-up of drafting gamma tokens given the acceptance estimate:
                    ``E[tokens] = (1 - a^(g+1)) / (1 - a)``; ``utility = E[tokens] / (1 + g*verify_cost + draft_cost)``;
                    strategies ``fixed`` (static depth), ``ema`` (argmax utility under the acceptance EMA) and
                    ``cascade`` (ema, but depth only moves one step per adjustment interval).
``DepthCalibrator`` closed loop on the measured acceptance rate (native ``AcceptanceTracker``): below
                    ``min_acceptance_rate`` speculation is switched off for the request, the depth is nudged
                    towards ``target_acceptance_rate``.
Reference: ``speculation.{draft_combiner,utility_scorer,calibration}`` (config/schema.json) and
python/orchestrator/{draft_combiner,utility_scorer}.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


@dataclass
class DraftSource:
    name: str
    proposer: object                       # has propose(context, gamma)
    cost: float = 0.1                      # relative to one target decode step
    priority_boost: float = 1.0
    acceptance: float = 0.5                # running estimate
    alpha: float = 0.2

    def update(self, proposed: int, accepted: int):
        if proposed > 0:
            self.acceptance += self.alpha * (accepted / proposed - self.acceptance)


def expected_tokens(a: float, g: int) -> float:
    """Expected committed tokens of one round: accepted prefix + the target's own token."""
    a = min(max(a, 0.0), 0.999999)
    return (1.0 - a ** (g + 1)) / (1.0 - a)


class DraftCombiner:
    def __init__(self, sources: Sequence[DraftSource], enabled: bool = True):
        self.sources = list(sources)
        self.enabled = enabled
        self.last: Optional[DraftSource] = None

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        best, best_score, best_src = [], 0.0, None
        for s in self.sources:
            p = list(s.proposer.propose(context, gamma))
            if not p:
                continue
            # a source that knows how far it trusts THIS proposal (a confidence head's survival probabilities) says so itself;
            # the others are judged by their running acceptance rate
            hint = getattr(s.proposer, "last_expected_tokens", None)
            exp = hint() if callable(hint) else None
            score = s.priority_boost * (exp if exp is not None else expected_tokens(s.acceptance, len(p))) / (1.0 + s.cost)
            if score > best_score:
                best, best_score, best_src = p, score, s
            if not self.enabled:
                break
            if s.cost < 0.02 and len(p) >= gamma:        # a free, full-length proposal: do not pay for the model draft
                break
        self.last = best_src
        return best

    def feedback(self, proposed: int, accepted: int):
        if self.last is not None:
            self.last.update(proposed, accepted)
            fb = getattr(self.last.proposer, "feedback", None)
            if callable(fb):
                fb(proposed, accepted)                       # the chosen source's own planner / scheduler / recorder learns too


class UtilityScorer:
    def __init__(self, strategy: str = "cascade", static_depth: int = 3, utility_threshold: float = 1.0, max_depth: int = 8,
                 verify_cost_per_row: float = 0.03, draft_cost_per_token: float = 0.05):
        assert strategy in ("cascade", "ema", "fixed")
        self.strategy, self.static_depth, self.threshold, self.max_depth = strategy, static_depth, utility_threshold, max_depth
        self.verify_cost, self.draft_cost = verify_cost_per_row, draft_cost_per_token
        self.depth = static_depth

    def utility(self, a: float, g: int) -> float:
        return expected_tokens(a, g) / (1.0 + g * (self.verify_cost + self.draft_cost))

    def best_depth(self, a: float) -> int:
        """0 means: do not speculate (no depth beats plain decoding by the threshold)."""
        best_g, best_u = 0, self.threshold
        for g in range(1, self.max_depth + 1):
            u = self.utility(a, g)
            if u > best_u + 1e-12:
                best_g, best_u = g, u
        return best_g

    def choose(self, a: float) -> int:
        if self.strategy == "fixed":
            return self.static_depth
        target = self.best_depth(a)
        if self.strategy == "ema":
            self.depth = target
        else:
            self.depth += (target > self.depth) - (target < self.depth)
        return self.depth


@dataclass
class DepthCalibrator:
    min_acceptance_rate: float = 0.3
    target_acceptance_rate: float = 0.6
    adjustment_interval_tokens: int = 500
    ema_alpha: float = 0.5
    step: int = 1
    depth: int = 3
    max_depth: int = 8
    enabled: bool = True
    _acc: float = field(default=0.6, repr=False)
    _since: int = field(default=0, repr=False)
    _prop: int = field(default=0, repr=False)
    _hit: int = field(default=0, repr=False)

    def record(self, proposed: int, accepted: int) -> None:
        self._prop += proposed
        self._hit += accepted
        self._since += accepted + 1
        if self._since >= self.adjustment_interval_tokens and self._prop:
            rate = self._hit / self._prop
            self._acc += self.ema_alpha * (rate - self._acc)
            if self._acc < self.min_acceptance_rate:
                self.enabled = False
            elif self._acc > self.target_acceptance_rate and self.depth < self.max_depth:
                self.depth += self.step
            elif self._acc < self.target_acceptance_rate and self.depth > 1:
                self.depth -= self.step
            self._since = self._prop = self._hit = 0

    @property
    def acceptance(self) -> float:
        return self._acc


class DepthPolicy:
    """How many tokens to ask the draft for, round by round: the utility scorer's depth under the running acceptance rate, capped by
    the closed-loop calibrator's depth; 0 = a plain decode step this round.  The calibrator's switch-off holds for the request it
    happened in (``begin_request`` arms it again); while the depth is 0 one single-token round is tried every ``probe_every`` rounds,
    so that a draft that started badly gets another look.  Reference: ``speculation.utility_scorer`` and ``speculation.calibration``
    driving the depth in python/orchestrator/orchestrator_loop.py."""

    def __init__(self, scorer: Optional[UtilityScorer] = None, calibrator: Optional[DepthCalibrator] = None, max_depth: int = 8, alpha: float = 0.2,
                 probe_every: int = 16):
        self.scorer, self.calibrator, self.max_depth, self.alpha, self.probe_every = scorer, calibrator, max_depth, alpha, probe_every
        self.acceptance = 0.6
        self._idle = 0
        self.rounds = self.plain_rounds = 0

    def begin_request(self):
        if self.calibrator is not None:
            self.calibrator.enabled = True

    def depth(self) -> int:
        d = self.max_depth
        if self.calibrator is not None:
            d = min(d, self.calibrator.depth) if self.calibrator.enabled else 0
        if self.scorer is not None and d > 0:
            d = min(d, self.scorer.choose(self.acceptance))
        if d <= 0:
            self._idle += 1
            if self.probe_every > 0 and self._idle >= self.probe_every:
                self._idle, d = 0, 1
            else:
                self.plain_rounds += 1
        else:
            self._idle = 0
        return max(0, d)

    def record(self, proposed: int, accepted: int):
        if proposed <= 0:
            return
        self.rounds += 1
        # per-token acceptance over the positions that were decided (the first rejected one included)
        self.acceptance += self.alpha * (accepted / min(proposed, accepted + 1) - self.acceptance)
        if self.calibrator is not None:
            self.calibrator.record(proposed, accepted)

    @classmethod
    def from_config(cls, sp: dict, max_depth: int) -> Optional["DepthPolicy"]:
        """From the ``speculation`` section; None when neither the scorer nor the calibration is enabled."""
        us, cal = sp.get("utility_scorer") or {}, sp.get("calibration") or {}
        scorer = calibrator = None
        if us.get("enabled"):
            scorer = UtilityScorer(us.get("strategy", "cascade"), min(int(us.get("static_depth", 3)), max_depth), float(us.get("utility_threshold", 1.0)), max_depth)
            scorer.depth = min(scorer.depth, max_depth)
        if cal and cal.get("enabled", True):                # the section has no switch of its own: present means on
            calibrator = DepthCalibrator(float(cal.get("min_acceptance_rate", 0.3)), float(cal.get("target_acceptance_rate", 0.6)),
                                         int(cal.get("adjustment_interval_tokens", 500)), float(cal.get("acceptance_ema_alpha", 0.5)),
                                         depth=min(max_depth, int(us.get("static_depth", 3)) if us else 3), max_depth=max_depth)
        if scorer is None and calibrator is None:
            return None
        return cls(scorer, calibrator, max_depth)
