"""Model-based draft proposers.

``EngineDraft`` runs a small draft model (by default the 2-layer MLA draft shape with the target's
hidden size and vocabulary, NVFP4 dense weights) on its own ``Engine``: it keeps one draft sequence
in step with the request's context (only the new tokens are prefetched into the draft cache each
round), decodes ``gamma`` greedy tokens with the CUDA-graph decode path and rewinds.  A failure in
the draft never reaches the target: ``propose`` returns an empty proposal instead of raising.

``MarkovHead`` / ``ConfidenceHead`` are the block-draft heads of the reference's DSpark speculator:
``logits_k = base_logits[k] + W2 @ W1[x_{k-1}]`` chained over the block with lowest-index argmax, and
``c_k = sigmoid(w . [hidden_k ; W1[x_{k-1}]] + b)``, the trained survival probability used to cut a
proposal where the cumulative product drops below a threshold.
Reference: src/speculation/dspark_runtime.h:1-61, src/compute/kernels/dspark/dspark_markov.h:1-83,
dspark_confidence.h:1-46.
"""
from __future__ import annotations

import logging
from typing import List, Optional, Sequence

import torch

from ..models.config import ModelConfig

log = logging.getLogger("layerstorm_b200.speculation")


def draft_shape_for(target: ModelConfig, n_layers: int = 2, quant: str = "nvfp4") -> ModelConfig:
    """The draft architecture: ``n_layers`` dense-FFN MLA layers at the target's width and vocabulary."""
    rope = target.qk_rope if target.qk_rope else 64
    return ModelConfig(
        name=f"{target.name}-draft{n_layers}", architecture="deepseek_v3", hidden=target.hidden, n_layers=n_layers,
        vocab=target.vocab, rms_eps=target.rms_eps, n_heads=target.n_heads, q_lora=target.q_lora or 1536, kv_lora=target.kv_lora,
        qk_nope=128, qk_rope=rope, v_head=128, rope_theta=target.rope_theta, max_position=target.max_position,
        dense_inter=target.dense_inter, first_k_dense=n_layers, n_routed=0, top_k=0, n_shared=0, moe_inter=target.moe_inter,
        expert_quant=quant, dense_quant=quant, eos_token_ids=list(target.eos_token_ids))


class EngineDraft:
    """``propose(context, gamma)`` backed by an engine (GPU ``Engine`` or the null engine)."""

    def __init__(self, engine, max_gamma: int = 8, min_confidence: float = 0.0):
        """``min_confidence`` > 0: drafting stops at the first token whose top-1 probability under the draft model is below it (that
        token is not proposed).  The probability comes from the device with the token (``Engine.decode(confidence=True)``); engines that
        cannot report it draft the full depth."""
        self.engine = engine
        self.max_gamma = max_gamma
        self.min_confidence = float(min_confidence)
        self.early_stops = 0
        self.sid: Optional[int] = None
        self.fed: List[int] = []           # tokens whose KV rows are in the draft cache
        self.failures = 0
        self.rounds = 0

    def reset(self):
        if self.sid is not None:
            try:
                self.engine.free_sequence(self.sid)
            except Exception:
                pass
        self.sid, self.fed = None, []

    def _sync(self, context: Sequence[int]):
        """Bring the draft cache to hold exactly ``context[:-1]``."""
        eng = self.engine
        if self.sid is None:
            self.sid = eng.create_sequence()
            self.fed = []
        want = list(context[:-1])
        common = 0
        lim = min(len(want), len(self.fed))
        while common < lim and want[common] == self.fed[common]:
            common += 1
        if common < len(self.fed):
            if getattr(eng, "has_recurrent_state", False):
                # recurrent draft state cannot be cut at an arbitrary earlier position: start the draft sequence over
                eng.free_sequence(self.sid)
                self.sid, self.fed, common = eng.create_sequence(), [], 0
            else:
                eng.rewind(self.sid, common)
                self.fed = self.fed[:common]
        if len(want) > common:
            eng.prefill(self.sid, want[common:], want_logits=False)
            self.fed = want

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        g = min(gamma, self.max_gamma)
        if g <= 0 or not context:
            return []
        self.rounds += 1
        try:
            self._sync(context)
            eng, sid = self.engine, self.sid
            tok = int(context[-1])
            out: List[int] = []
            if getattr(eng, "has_recurrent_state", False) and hasattr(eng, "anchor"):
                eng.anchor(sid)            # the drafted tokens are rolled back through this snapshot
            gate = self.min_confidence > 0.0 and getattr(eng, "supports_confidence", False)
            fed = 0
            for _ in range(g):
                if gate:
                    toks, conf = eng.decode([sid], [tok], confidence=True)
                    fed += 1
                    if conf[0][0] < self.min_confidence:
                        self.early_stops += 1
                        break
                    tok = int(toks[0])
                else:
                    tok = int(eng.decode([sid], [tok])[0])
                    fed += 1
                out.append(tok)
            eng.rewind(sid, len(context) - 1)
            return out
        except Exception as e:            # fail closed: the target continues with plain decode
            self.failures += 1
            log.warning("draft proposal failed (%s); continuing without a draft", e)
            self.reset()
            return []


class MarkovHead:
    """Rank-r first-order correction of block-draft logits."""

    def __init__(self, w1: torch.Tensor, w2: torch.Tensor, bias: Optional[torch.Tensor] = None, d2t: Optional[torch.Tensor] = None):
        self.w1, self.w2 = w1.float(), w2.float()          # [V, r], [V_draft, r]
        self.bias = bias.float() if bias is not None else None
        self.d2t = d2t                                       # draft id -> target id offset (id + d2t[id])

    def chain(self, base_logits: torch.Tensor, prev_token: int) -> tuple[List[int], torch.Tensor]:
        """``base_logits`` [gamma, V_draft].  Returns target-vocabulary ids and the W1 rows used (for the
        confidence head)."""
        ids: List[int] = []
        feats = []
        x = int(prev_token)
        for k in range(base_logits.shape[0]):
            e = self.w1[x]
            feats.append(e)
            lg = base_logits[k].float() + self.w2 @ e
            if self.bias is not None:
                lg = lg + self.bias
            m = lg.max()
            did = int(torch.nonzero(lg == m)[0])             # lowest index on ties
            x = did + (int(self.d2t[did]) if self.d2t is not None else 0)
            ids.append(x)
        return ids, torch.stack(feats)


class ConfidenceHead:
    def __init__(self, w: torch.Tensor, b: float = 0.0):
        self.w, self.b = w.float(), float(b)

    def survival(self, hidden: torch.Tensor, feats: torch.Tensor) -> torch.Tensor:
        return torch.sigmoid(torch.cat([hidden.float(), feats.float()], -1) @ self.w + self.b)

    @staticmethod
    def cut(conf: torch.Tensor, threshold: float) -> int:
        """Number of draft tokens to keep: the longest prefix whose cumulative survival stays >= threshold."""
        keep, p = 0, 1.0
        for c in conf.tolist():
            p *= c
            if p < threshold:
                break
            keep += 1
        return keep
