"""Online calibration of the self-speculative draft: how aggressive the draft pass may be, from the acceptance it earns.

A draft pass is cheaper the fewer routed experts it runs per token and the more layers it skips, and it is accepted less often the
cheaper it is.  ``OnlineCalibrator`` watches the acceptance rate (exponential moving average over speculation rounds) and, every
``adjustment_interval_tokens`` drafted tokens, moves ONE step:
  * acceptance below ``min_acceptance_rate``: first switch layer skipping off (it costs the most acceptance per unit of speed), then
    raise the draft's expert count by one (up to the model's own top-k);
  * acceptance above ``target_acceptance_rate``: first lower the expert count by one (down to 1), then switch layer skipping on.
Between the two thresholds nothing changes.  The verification by the full model is lossless whatever the draft does; the calibrator
only moves speed.  ``SelfSpeculativeDraft`` applies a changed expert count by building a new reduced-expert view of the target (its
draft cache is rebuilt from the context on the next proposal) and a changed layer-skip switch through its skip policy.
Configuration: the ``speculation.calibration`` section.  Reference: python/orchestrator/online_calibrator.py (same priorities).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class DraftParams:
    draft_expert_count: int = 1
    layer_skip_enabled: bool = False
    min_draft_expert_count: int = 1
    max_draft_expert_count: int = 8


class OnlineCalibrator:
    def __init__(self, cfg: dict, params: DraftParams):
        """``cfg``: the ``speculation.calibration`` section."""
        self.min_rate = float(cfg.get("min_acceptance_rate", 0.3))
        self.target_rate = float(cfg.get("target_acceptance_rate", 0.6))
        self.interval = max(1, int(cfg.get("adjustment_interval_tokens", 500)))
        self.alpha = float(cfg.get("acceptance_ema_alpha", 0.5))
        self.params = params
        self.rate = None                 # smoothed acceptance, None before the first round
        self.since = 0                   # drafted tokens since the last decision
        self.adjustments = 0
        self.history = []                # (drafted tokens seen, what changed) of every adjustment

    def update(self, proposed: int, accepted: int) -> bool:
        """One speculation round's outcome.  Returns True when the draft parameters changed."""
        if proposed <= 0:
            return False
        r = accepted / proposed
        self.rate = r if self.rate is None else self.alpha * r + (1.0 - self.alpha) * self.rate
        self.since += proposed
        if self.since < self.interval:
            return False
        self.since = 0
        p, what = self.params, None
        if self.rate < self.min_rate:                          # too aggressive
            if p.layer_skip_enabled:
                p.layer_skip_enabled, what = False, "layer skipping off"
            elif p.draft_expert_count < p.max_draft_expert_count:
                p.draft_expert_count += 1
                what = f"draft experts -> {p.draft_expert_count}"
        elif self.rate > self.target_rate:                     # room to be cheaper
            if p.draft_expert_count > p.min_draft_expert_count:
                p.draft_expert_count -= 1
                what = f"draft experts -> {p.draft_expert_count}"
            elif not p.layer_skip_enabled:
                p.layer_skip_enabled, what = True, "layer skipping on"
        if what is None:
            return False
        self.adjustments += 1
        self.history.append((round(self.rate, 4), what))
        return True
