"""MTP draft source: the model's own multi-token-prediction blocks propose the next tokens; the target verifies them losslessly.

``MtpDraft`` works on engines that expose the fp32 reference model (the CPU engine): it recomputes the main stream for the context and
runs the MTP blocks over it (``models/mtp.py``), with the planner's dynamic depth gate (stop when the block's confidence in its own
token falls under ``speculation.mtp.confidence_threshold``).
``DeviceMtpDraft`` is the GPU path: the engine keeps block 0 in step with every sequence (``runtime/mtp.py``: its own latent cache over
the sequence's pages, one pass of the block per committed token) and proposes one token per round from the stream the main model's
last step left on the device - no second model, no second KV allocation, four bytes back per proposal.
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


class DeviceMtpDraft:
    """``speculation.method = mtp`` on the GPU engine.  ``engine``: an ``Engine`` whose model carries MTP blocks on the device
    (``DeviceModel.mtp_supported``); ``cfg``: the ``speculation.mtp`` section.  Raises NotImplementedError when the engine cannot
    host the block (see ``Engine.enable_mtp``)."""

    def __init__(self, engine, cfg: dict):
        self.engine = engine
        engine.enable_mtp()
        mc = engine.cfg
        self.planner = MtpDraftPlanner(cfg, mc.n_layers, max(1, mc.n_mtp))
        self.proposed = 0

    def _sequence_of(self, context: Sequence[int]):
        """The engine's sequence that holds exactly ``context`` without its last token (the orchestrator hands over token lists)."""
        n = len(context) - 1
        for sid, s in self.engine.seqs.items():
            if s.length == n and len(s.tokens) == n and s.tokens[-8:] == [int(t) for t in context[max(0, n - 8): n]]:
                return sid
        return None

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        if not self.planner.enabled or gamma <= 0 or len(context) < 2:
            return []
        sid = self._sequence_of(context)
        if sid is None:
            return []
        out = self.engine.mtp_draft(sid, int(context[-1]))
        self.proposed += len(out)
        return out

    def feedback(self, proposed: int, accepted: int):
        self.planner.record(proposed, accepted)
