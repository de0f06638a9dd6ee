"""Self-speculative draft: the target model drafts for itself with fewer routed experts per token.

``SelfSpeculativeDraft(engine, cfg)`` asks the engine for a reduced-expert view of its own weights (``reduced_expert_view(k)``: same
tensors, ``k`` routed experts per token instead of the model's top-k, own KV cache) and drafts with it exactly like a separate draft
model (``EngineDraft``: incremental sync of the draft cache, ``gamma`` greedy steps, rewind).  The expert bytes streamed per drafted
token fall by top_k / k in the MoE layers while attention and the shared expert stay exact, so acceptance is high where the top expert
dominates the mixture.  Verification by the full model is the ordinary lossless path of the orchestrator.
``plan`` (``policies.SelfSpeculativePlan``) supplies the early-exit rule and the acceptance statistics.  With a ``layer_skip`` section
(``speculation.layer_skip_draft``) and a draft engine that can leave layers out (``Engine.set_layer_skip``) the draft passes also skip
layers: every draft step records, on the device, the cosine similarity between each executed layer's input and the next one's; once the
draft's acceptance rate allows it, ``policies.LayerSkipPolicy`` turns the last step's similarities into the set of layers the NEXT
round's draft steps leave out (protected first / last layers, contiguity and product gates, a cap on the skipped fraction).
Reference counterpart: python/orchestrator/self_speculative.py (reduced-expert full-model draft pass, third draft source after prompt
lookup and MTP).
"""
from __future__ import annotations

from typing import List, Sequence

from .model_draft import EngineDraft
from .policies import SelfSpeculativePlan


class SelfSpeculativeDraft(EngineDraft):
    def __init__(self, engine, cfg: dict, max_gamma: int = 8, layer_skip: dict = None, calibration: dict = None):
        """``engine``: the TARGET engine (or its model holder) offering ``reduced_expert_view``; ``cfg``: ``speculation.self_speculative``;
        ``layer_skip``: ``speculation.layer_skip_draft`` (optional); ``calibration``: ``speculation.calibration`` (optional: the draft's
        expert count and layer skipping then follow the acceptance rate, see ``online_calibrator.py``)."""
        from .policies import LayerSkipPolicy
        k = max(1, int(cfg.get("draft_expert_count", 1)))
        super().__init__(make_reduced_engine(engine, k), max_gamma)
        self._target = engine
        mc = engine.cfg if hasattr(engine, "cfg") else engine.model.cfg
        self.skip_policy = LayerSkipPolicy(layer_skip or {}, mc.n_layers)
        self.skip_set = set()
        self.skipped_layer_steps = 0
        moe = [i for i in range(mc.n_layers) if mc.is_moe_layer(i)]
        self.plan = SelfSpeculativePlan(cfg, moe, mc.n_layers, mc.top_k, max_depth=max_gamma)
        self.expert_fraction = self.plan.expert_fraction(mc.top_k)
        self._model_top_k = mc.top_k
        self.calibrator = None
        if calibration is not None:
            from .online_calibrator import DraftParams, OnlineCalibrator
            self.calibrator = OnlineCalibrator(calibration, DraftParams(draft_expert_count=self.plan.k, layer_skip_enabled=bool(self.skip_policy.enabled),
                                                                        max_draft_expert_count=mc.top_k))
            self._skip_configured = bool(self.skip_policy.enabled)

    def _apply_calibration(self):
        """The calibrator moved: take over its expert count (a new reduced-expert view of the target; the draft cache is rebuilt from
        the context by the next proposal) and its layer-skip switch (only ever on when the configuration enabled skipping)."""
        p = self.calibrator.params
        if p.draft_expert_count != self.plan.k:
            self.reset()
            self.engine = make_reduced_engine(self._target, p.draft_expert_count)
            self.plan.k = p.draft_expert_count
            self.expert_fraction = self.plan.expert_fraction(self._model_top_k)
        self.skip_policy.enabled = bool(p.layer_skip_enabled and self._skip_configured)
        if not self.skip_policy.enabled:
            self.skip_set = set()
            if hasattr(self.engine, "set_layer_skip"):
                self.engine.set_layer_skip(set(), probe=False)

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        if not self.plan.enabled:
            return []
        eng = self.engine
        skipping = self.skip_policy.enabled and hasattr(eng, "set_layer_skip")
        if skipping:
            use = self.skip_set if self.skip_policy.active(self.plan.acceptance_rate) else set()
            eng.set_layer_skip(use, probe=True)
        out = super().propose(context, min(gamma, self.plan.max_depth))
        if skipping:
            self.skipped_layer_steps += len(eng.model.skip_layers) * len(out)
            sims = eng.layer_similarities()              # of the round's last draft step
            if sims:
                self.skip_set = self.skip_policy.skip_set(sims)
        return out

    def feedback(self, proposed: int, accepted: int):
        self.plan.record(proposed, accepted)
        if self.calibrator is not None and self.calibrator.update(proposed, accepted):
            self._apply_calibration()


def make_reduced_engine(engine, top_k: int):
    """Draft engine over the target's weights.  CPU engine: a view of itself.  GPU engine: a second ``Engine`` over
    ``DeviceModel.reduced_expert_view`` with a small cache of its own (one sequence, the target's context length)."""
    if hasattr(engine, "reduced_expert_view"):
        return engine.reduced_expert_view(top_k)
    model = getattr(engine, "model", None)
    if model is None or not hasattr(model, "reduced_expert_view"):
        raise TypeError("this engine cannot draft for itself (no reduced_expert_view)")
    from ..runtime.engine import Engine
    return Engine(model.reduced_expert_view(top_k), max_seqs=2, max_ctx=engine.max_ctx, prefill_chunk=engine.prefill_chunk, max_batch=1,
                  use_graph=getattr(engine, "use_graph", True))
