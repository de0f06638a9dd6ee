"""Self-speculative draft: the target model drafts for itself with fewer routed experts per token.

``SelfSpeculativeDraft(engine, cfg)`` asks the engine for a reduced-expert view of its own weights (``reduced_expert_view(k)``: same
tensors, ``k`` routed experts per token instead of the model's top-k, own KV cache) and drafts with it exactly like a separate draft
model (``EngineDraft``: incremental sync of the draft cache, ``gamma`` greedy steps, rewind).  The expert bytes streamed per drafted
token fall by top_k / k in the MoE layers while attention and the shared expert stay exact, so acceptance is high where the top expert
dominates the mixture.  Verification by the full model is the ordinary lossless path of the orchestrator.
``plan`` (``policies.SelfSpeculativePlan``) supplies the early-exit rule and the acceptance statistics; layer skipping is not applied
by the engines (the policy object exists, no engine has a skip path).
Reference counterpart: python/orchestrator/self_speculative.py (reduced-expert full-model draft pass, third draft source after prompt
lookup and MTP).
"""
from __future__ import annotations

from typing import List, Sequence

from .model_draft import EngineDraft
from .policies import SelfSpeculativePlan


class SelfSpeculativeDraft(EngineDraft):
    def __init__(self, engine, cfg: dict, max_gamma: int = 8):
        """``engine``: the TARGET engine (or its model holder) offering ``reduced_expert_view``; ``cfg``: ``speculation.self_speculative``."""
        k = max(1, int(cfg.get("draft_expert_count", 1)))
        super().__init__(make_reduced_engine(engine, k), max_gamma)
        mc = engine.cfg if hasattr(engine, "cfg") else engine.model.cfg
        moe = [i for i in range(mc.n_layers) if mc.is_moe_layer(i)]
        self.plan = SelfSpeculativePlan(cfg, moe, mc.n_layers, mc.top_k, max_depth=max_gamma)
        self.expert_fraction = self.plan.expert_fraction(mc.top_k)

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        if not self.plan.enabled:
            return []
        return super().propose(context, min(gamma, self.plan.max_depth))

    def feedback(self, proposed: int, accepted: int):
        self.plan.record(proposed, accepted)


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
