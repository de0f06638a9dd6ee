"""MTP draft source: the model's own multi-token-prediction blocks propose the next tokens; the target verifies them losslessly.

``MtpDraft`` works on engines that expose the fp32 reference model (the CPU engine): it recomputes the main stream for the context and
runs the MTP blocks over it (``models/mtp.py``), with the planner's dynamic depth gate (stop when the block's confidence in its own
token falls under ``speculation.mtp.confidence_threshold``).  There is no device path: the GPU engine does not execute MTP blocks, so
``speculation.method = mtp`` is available on the CPU engine only.
Reference counterpart: python/orchestrator/mtp_draft.py + the engine's MtpSpeculationMethod.
"""
from __future__ import annotations

from typing import List, Sequence

from ..models.mtp import mtp_draft_tokens
from .policies import MtpDraftPlanner


class MtpDraft:
    def __init__(self, engine, cfg: dict):
        """``engine``: an engine whose ``model`` is the reference ``Oracle`` with MTP weights; ``cfg``: the ``speculation.mtp`` section."""
        self.oracle = engine.model
        mc = self.oracle.cfg
        if mc.n_mtp <= 0:
            raise ValueError("the model has no multi-token-prediction blocks (n_mtp = 0)")
        self.planner = MtpDraftPlanner(cfg, mc.n_layers, mc.n_mtp)
        self.last_confidences: List[float] = []

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        if not self.planner.enabled or gamma <= 0:
            return []
        depth = min(gamma, self.planner.max_depth)
        toks, conf = mtp_draft_tokens(self.oracle, context, depth, stop=lambda step, c: not self.planner.should_continue(step, c))
        self.last_confidences = conf
        return toks

    def feedback(self, proposed: int, accepted: int):
        self.planner.record(proposed, accepted)
